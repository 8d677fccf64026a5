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
from .linear import linear, prepare_weight, uses_tensor_cores


class SwiGLU(FeedForward):
    def __init__(self, spec: PartSpec, hidden_size: int):
        super().__init__(spec, hidden_size)
        self.inter = int(spec["intermediate_size"])
        if self.inter <= 0:
            raise ConfigError("swiglu: intermediate_size must be positive")
        self.w_gate_up = self.w_down = None
        self.fused = False

    def weight_specs(self) -> Dict[str, WeightSpec]:
        h, i = self.hidden_size, self.inter
        return {"gate_proj.weight": WeightSpec((i, h)), "up_proj.weight": WeightSpec((i, h)),
                "down_proj.weight": WeightSpec((h, i))}

    def load(self, tensors, dtype):
        gate, up = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        common = torch.float32 if torch.float32 in (gate.dtype, up.dtype) else gate.dtype
        self.w_down = prepare_weight(tensors["down_proj.weight"], dtype)
        stacked = torch.cat([gate.to(common), up.to(common)], dim=0)
        # On the tensor-core path SiLU(gate)*up is the product's epilogue: rows are laid out
        # as blocks of 16 gate rows followed by their 16 up rows, so that both halves of an
        # output land in one warp's slice of the accumulator.
        self.fused = (dtype == torch.bfloat16 and self.inter % 16 == 0 and uses_tensor_cores(dtype, stacked))
        if self.fused:
            h = stacked.shape[1]
            blocks = torch.stack([stacked[:self.inter].view(-1, 16, h), stacked[self.inter:].view(-1, 16, h)], dim=1)
            self.w_gate_up = prepare_weight(blocks.reshape(2 * self.inter, h).contiguous(), dtype)
        else:
            self.w_gate_up = stacked.contiguous()

    def first_weight(self):
        return self.w_gate_up

    def forward(self, ctx, x):
        if self.fused:
            mlp = ops.gemm_tc(ops.materialize(x), self.w_gate_up, ctx.status, swiglu=True)
        else:
            mlp = ops.silu_mul(linear(ctx, x, self.w_gate_up))
        return linear(ctx, mlp, self.w_down, allow_partial=True)     # summed by the norm that follows


register_part("feed_forward", "swiglu", SwiGLU, replace=True)
