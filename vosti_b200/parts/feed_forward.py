"""Gated feed-forward with SiLU: down( silu(gate(x)) * up(x) ).

gate and up are one [2I, hidden] matrix (gate rows first) so that the projection is a
single product, as the reference's loader concatenates them
(python/vosti_kernels/model_families/qwen3/loader.py:55-58); the activation is
gate * sigmoid(gate) * up in float32 (kernels/triton_kernels/silu_mul.py:66-87).
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..config.schema import ConfigError, PartSpec
from ..weights.loader import WeightSpec
from .base import FeedForward, register_part
from .linear import linear


class SwiGLU(FeedForward):
    def __init__(self, spec: PartSpec, hidden_size: int):
        super().__init__(spec, hidden_size)
        self.inter = int(spec["intermediate_size"])
        if self.inter <= 0:
            raise ConfigError("swiglu: intermediate_size must be positive")
        self.w_gate_up = self.w_down = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        h, i = self.hidden_size, self.inter
        return {"gate_proj.weight": WeightSpec((i, h)), "up_proj.weight": WeightSpec((i, h)),
                "down_proj.weight": WeightSpec((h, i))}

    def load(self, tensors, dtype):
        gate, up = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        common = torch.float32 if torch.float32 in (gate.dtype, up.dtype) else gate.dtype
        self.w_gate_up = torch.cat([gate.to(common), up.to(common)], dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"]

    def forward(self, ctx, x):
        gate_up = linear(ctx, x, self.w_gate_up)
        return linear(ctx, ops.silu_mul(gate_up), self.w_down)


register_part("feed_forward", "swiglu", SwiGLU, replace=True)
