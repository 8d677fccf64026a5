"""Load the tensors a built model asks for, by name, and check them.

Every part declares the tensors it needs (`WeightSpec`: shape and how a random
model would draw it). The loader compares that list with the folder and raises
one `WeightError` that lists every missing tensor, every unexpected tensor and
every wrong shape (the reference reports the same classes of error one at a
time: python/vosti_kernels/checkpoint.py:42-62,
python/vosti_kernels/model_families/qwen3/physical.py:36-196).

Floating tensors are kept in bfloat16 when serving in bfloat16, except that a
tensor stored in 32-bit stays 32-bit; integer tables become int32. Serving in
float32 widens every floating tensor (exactly) to float32.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Mapping, Optional, Tuple

import torch

from .safetensors_io import open_model_shards


class WeightError(ValueError):
    """Missing, unexpected or misshapen tensors; `.missing`, `.unexpected`,
    `.wrong_shape` hold the details."""

    def __init__(self, missing, unexpected, wrong_shape, where=""):
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong_shape
        lines = [f"weights in {where} do not match the model:" if where
                 else "weights do not match the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        for name, got, want in wrong_shape:
            lines.append(f"  wrong shape: {name} has {list(got)}, expected {list(want)}")
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


def load_weights(model_dir: str | Path, expected: Mapping[str, WeightSpec], *,
                 device: torch.device | str, dtype: torch.dtype,
                 ignore: Tuple[str, ...] = ()) -> Dict[str, torch.Tensor]:
    """Return name -> tensor on `device` for every expected tensor."""
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
    if missing or unexpected or wrong:
        raise WeightError(missing, unexpected, wrong, where=str(model_dir))
    out: Dict[str, torch.Tensor] = {}
    for name, spec in expected.items():
        if name not in shards:
            continue
        host = shards[name].tensor(name)
        target = _resident_dtype(host.dtype, dtype, spec.integer)
        out[name] = host.to(device=device, dtype=target).contiguous()
    return out


def check_tensors(tensors: Mapping[str, torch.Tensor], expected: Mapping[str, WeightSpec],
                  ignore: Tuple[str, ...] = ()) -> None:
    """The same check for tensors that are already in memory."""
    missing = sorted(n for n, s in expected.items() if n not in tensors and not s.optional)
    unexpected = sorted(n for n in tensors if n not in expected and n not in ignore)
    wrong = [(n, tuple(tensors[n].shape), tuple(s.shape)) for n, s in expected.items()
             if n in tensors and tuple(tensors[n].shape) != tuple(s.shape)]
    if missing or unexpected or wrong:
        raise WeightError(missing, unexpected, wrong)
