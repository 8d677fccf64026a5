"""Random-weights mode: draw every tensor a model asks for from a seed, and
write a model folder (config.json, model.safetensors) that loads like any other.

The reference has only an all-zero zero-layer fixture
(tests/support/model_families/qwen3.rs:26-35); the distributions here are those
of the benchmark configuration: linear and embedding weights N(0, 0.02), every
RMSNorm weight (q/k head norms too) 1 + N(0, 0.1). Each tensor has a stream of
its own, keyed by (seed, tensor name), so a draw does not depend on which other
tensors exist or in which order they are drawn.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Dict, Mapping

import torch

from .loader import WeightSpec
from .safetensors_io import write_safetensors


def _stream_seed(seed: int, name: str) -> int:
    digest = hashlib.blake2b(f"{seed}:{name}".encode(), digest_size=8).digest()
    return int.from_bytes(digest, "little") & ((1 << 63) - 1)


def draw_tensor(name: str, spec: WeightSpec, seed: int, *, device: torch.device | str = "cpu",
                dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Draw one tensor in float32 and round it once to `dtype`."""
    device = torch.device(device)
    if spec.integer:
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    generator = torch.Generator(device=device)
    generator.manual_seed(_stream_seed(seed, name))
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=dtype, device=device)
    if dtype == torch.bfloat16 and device.type == "cuda":
        # large tensors on the device: draw directly in the storage type
        values = torch.empty(spec.shape, dtype=dtype, device=device)
        values.normal_(0.0, spec.std, generator=generator)
    else:
        values = torch.empty(spec.shape, dtype=torch.float32, device=device)
        values.normal_(0.0, spec.std, generator=generator)
    if spec.init == "norm":
        values = values + 1.0
    elif spec.init not in ("linear", "embedding"):
        raise ValueError(f"tensor '{name}': unknown init '{spec.init}'")
    return values.to(dtype)


def draw_tensors(expected: Mapping[str, WeightSpec], seed: int, *,
                 device: torch.device | str = "cpu",
                 dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    return {name: draw_tensor(name, spec, seed, device=device, dtype=dtype)
            for name, spec in expected.items() if not spec.optional}


def write_random_model(model_dir: str | Path, config: Mapping, seed: int,
                       dtype: torch.dtype = torch.bfloat16) -> Path:
    """Write config.json and model.safetensors for `config` (the architecture's own
    config.json content) with weights drawn from `seed`."""
    from ..config import model_spec_from_config
    from ..models import expected_weights

    root = Path(model_dir)
    root.mkdir(parents=True, exist_ok=True)
    spec = model_spec_from_config(config)
    tensors = draw_tensors(expected_weights(spec), seed, device="cpu", dtype=dtype)
    (root / "config.json").write_text(json.dumps(dict(config), indent=1, sort_keys=True))
    write_safetensors(root / "model.safetensors", tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    return root
