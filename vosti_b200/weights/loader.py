"""Load the tensors a built model asks for, by name, and check them.

Every part declares the tensors it needs (`WeightSpec`: shape and how a random
model would draw it). The loader compares that list with the folder and raises
one `WeightError` that lists every missing tensor, every unexpected tensor and
every wrong shape (the reference reports the same classes of error one at a
time: python/vosti_kernels/checkpoint.py:42-62,
python/vosti_kernels/model_families/qwen3/physical.py:36-196).

Floating tensors must be stored as BF16 or F32 (the reference takes BF16 only,
checkpoint.py:61-62); anything else (F16, F64, 8-bit floats) is listed in the error
instead of being rounded silently. They are kept in bfloat16 when serving in bfloat16,
except that a tensor stored in 32-bit stays 32-bit; integer tables become int32. Serving
in float32 widens every floating tensor (exactly) to float32.

A tensor the model does not read because it stands for another one (the output head of a
model with tied embeddings) may be present, but then it must hold that tensor's values
(python/vosti_kernels/model_families/qwen3/physical.py:131-134); a different one is a
conflict and listed too.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Mapping, Optional, Tuple

import torch

from .safetensors_io import open_model_shards


class WeightError(ValueError):
    """Missing, unexpected or misshapen tensors, tensors of a dtype that is not taken, and
    stand-ins that differ from what they stand for; `.missing`, `.unexpected`, `.wrong_shape`,
    `.wrong_dtype`, `.conflicts` hold the details."""

    def __init__(self, missing, unexpected, wrong_shape, where="", wrong_dtype=(), conflicts=()):
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong_shape
        self.wrong_dtype, self.conflicts = list(wrong_dtype), list(conflicts)
        lines = [f"weights in {where} do not match the model:" if where
                 else "weights do not match the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        for name, got, want in wrong_shape:
            lines.append(f"  wrong shape: {name} has {list(got)}, expected {list(want)}")
        for name, got in self.wrong_dtype:
            lines.append(f"  wrong dtype: {name} is stored as {got}; floating tensors must be BF16 or F32")
        for name, other, why in self.conflicts:
            lines.append(f"  conflict: {name} must equal {other} (the configuration ties them) but {why}")
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class WeightSpec:
    """Shape of a tensor and the distribution a random model draws it from:
    'linear' and 'embedding' are N(0, std); 'norm' is 1 + N(0, std); 'zeros'."""

    shape: Tuple[int, ...]
    init: str = "linear"
    std: float = 0.02
    integer: bool = False
    optional: bool = False


def _resident_dtype(stored: torch.dtype, mode: torch.dtype, integer: bool) -> torch.dtype:
    if integer or not stored.is_floating_point:
        return torch.int32
    if mode == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


_FLOAT_STORAGE = (torch.bfloat16, torch.float32)


def _dtype_fault(name: str, stored: torch.dtype, integer: bool):
    if integer or not stored.is_floating_point or stored in _FLOAT_STORAGE:
        return None
    return (name, str(stored).replace("torch.", ""))


def _conflict(name: str, other: str, a: torch.Tensor, b: torch.Tensor):
    if tuple(a.shape) != tuple(b.shape):
        return (name, other, f"has shape {list(a.shape)}, not {list(b.shape)}")
    if a.dtype != b.dtype:
        return (name, other, f"is stored as {a.dtype}, not {b.dtype}")
    if not torch.equal(a, b):
        return (name, other, "holds different values")
    return None


def load_weights(model_dir: str | Path, expected: Mapping[str, WeightSpec], *,
                 device: torch.device | str, dtype: torch.dtype,
                 ignore: Tuple[str, ...] = (),
                 aliases: Optional[Mapping[str, str]] = None) -> Dict[str, torch.Tensor]:
    """Return name -> tensor on `device` for every expected tensor. `aliases` maps a tensor
    that may be present although the model does not read it to the tensor it must equal."""
    if dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("serving dtype must be torch.bfloat16 or torch.float32")
    shards = open_model_shards(model_dir)
    missing = sorted(n for n, s in expected.items() if n not in shards and not s.optional)
    unexpected = sorted(n for n in shards if n not in expected and n not in ignore)
    wrong = []
    for name, spec in expected.items():
        if name in shards:
            _, shape = shards[name].info(name)
            if tuple(shape) != tuple(spec.shape):
                wrong.append((name, tuple(shape), tuple(spec.shape)))
    aliases = dict(aliases or {})
    unexpected = [n for n in unexpected if n not in aliases]
    bad_dtype = [(n, shards[n].info(n)[0]) for n, s in expected.items()
                 if n in shards and not s.integer and shards[n].info(n)[0] in ("F16", "F64")]
    conflicts = []
    for name, other in aliases.items():
        if name in shards and other in shards:
            fault = _conflict(name, other, shards[name].tensor(name), shards[other].tensor(other))
            if fault:
                conflicts.append(fault)
    if missing or unexpected or wrong or bad_dtype or conflicts:
        raise WeightError(missing, unexpected, wrong, where=str(model_dir), wrong_dtype=bad_dtype,
                          conflicts=conflicts)
    out: Dict[str, torch.Tensor] = {}
    for name, spec in expected.items():
        if name not in shards:
            continue
        host = shards[name].tensor(name)
        target = _resident_dtype(host.dtype, dtype, spec.integer)
        out[name] = host.to(device=device, dtype=target).contiguous()
    return out


def check_tensors(tensors: Mapping[str, torch.Tensor], expected: Mapping[str, WeightSpec],
                  ignore: Tuple[str, ...] = (), aliases: Optional[Mapping[str, str]] = None) -> None:
    """The same check for tensors that are already in memory."""
    aliases = dict(aliases or {})
    missing = sorted(n for n, s in expected.items() if n not in tensors and not s.optional)
    unexpected = sorted(n for n in tensors if n not in expected and n not in ignore and n not in aliases)
    wrong = [(n, tuple(tensors[n].shape), tuple(s.shape)) for n, s in expected.items()
             if n in tensors and tuple(tensors[n].shape) != tuple(s.shape)]
    bad_dtype = [f for f in (_dtype_fault(n, tensors[n].dtype, s.integer) for n, s in expected.items()
                             if n in tensors) if f]
    conflicts = [f for f in (_conflict(n, o, tensors[n], tensors[o]) for n, o in aliases.items()
                             if n in tensors and o in tensors) if f]
    if missing or unexpected or wrong or bad_dtype or conflicts:
        raise WeightError(missing, unexpected, wrong, wrong_dtype=bad_dtype, conflicts=conflicts)
