"""Rotary position encoding: half-split pairing of the whole head for Qwen3; `rotary_dim` below
the head size (the rest of the head is not rotated) and `interleaved` pairs (2i, 2i + 1) are
parameters for other architectures.

inv_freq[i] = 1 / theta^(2i/d) in float32 from an integer arange; angle = inv_freq *
float(position) (python/vosti_kernels/rotary.py:80-88, 155-158). The reference casts the
cos/sin table to the serving dtype (:160); here the table stays float32 in both serving
dtypes, so rotation angles are 32-bit everywhere. The mixer applies the table
(pairs (i, i + d/2): kernels/triton_kernels/rope.py:78-101).
"""
from __future__ import annotations

import torch

from ..config.schema import ConfigError, PartSpec
from .base import PositionEncoding, register_part


class RotaryEncoding(PositionEncoding):
    def __init__(self, spec: PartSpec, hidden_size: int, head_dim: int):
        super().__init__(spec, hidden_size, head_dim)
        self.theta = float(spec["theta"])
        self.max_positions = int(spec["max_positions"])
        rotary_dim = int(spec.get("rotary_dim", head_dim) or head_dim)
        if rotary_dim <= 0 or rotary_dim > head_dim or rotary_dim % 2:
            raise ConfigError(f"rope: rotary_dim {rotary_dim} must be even and at most head_dim {head_dim}")
        self.rotary_dim = rotary_dim
        self.interleaved = bool(spec.get("interleaved", False))
        self.cos = self.sin = None

    def setup(self, device, dtype):
        exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.int64).to(torch.float32) / self.rotary_dim
        inv_freq = 1.0 / (self.theta ** exponent)
        angles = torch.arange(self.max_positions, dtype=torch.float32)[:, None] * inv_freq[None, :]
        self.cos = angles.cos().to(device).contiguous()
        self.sin = angles.sin().to(device).contiguous()

    def rotation_tables(self):
        return self.cos, self.sin


register_part("position", "rope", RotaryEncoding, replace=True)
