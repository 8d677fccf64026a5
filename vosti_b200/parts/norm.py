"""RMSNorm with a plain weight (no 1 + w offset), optionally fused with the residual add.

o = x * rsqrt(mean(x^2) + eps) * w in float32 (kernels/triton_kernels/rmsnorm.py:63-93);
with a residual the sum is stored as the new residual and normed unrounded
(kernels/triton_kernels/rmsnorm_residual.py:86-125).
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..config.schema import PartSpec
from ..weights.loader import WeightSpec
from .base import Norm, register_part


class RMSNorm(Norm):
    def __init__(self, spec: PartSpec, width: int):
        super().__init__(spec, width)
        self.eps = float(spec["eps"])
        self.width = width
        self.weight = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"weight": WeightSpec((self.width,), init="norm", std=0.1)}

    def load(self, tensors, dtype):
        self.weight = tensors["weight"]

    def forward(self, ctx, x):
        return ops.rmsnorm(x, self.weight, self.eps)[0]

    def forward_add(self, ctx, x, residual):
        # the sum overwrites the residual buffer in place
        return ops.rmsnorm(x, self.weight, self.eps, residual=residual, residual_out=residual)


register_part("norm", "rmsnorm", RMSNorm, replace=True)
