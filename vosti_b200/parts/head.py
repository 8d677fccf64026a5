"""The output head: logits = x @ W^T in float32 (src/exec/dense_swiglu_model.rs:897-984), where
W is the embedding table when the model ties them. Optional constants, none of which Qwen3
uses: a `bias` vector, a `scale` on the logits and a `softcap` c (logits <- c * tanh(logits / c));
they are applied to the float32 product by one row kernel.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..config.schema import ConfigError, PartSpec
from ..weights.loader import WeightSpec
from .base import Head, register_part
from .linear import linear, prepare_weight


class LinearHead(Head):
    def __init__(self, spec: PartSpec, hidden_size: int, vocab_size: int, tied: bool):
        super().__init__(spec, hidden_size, vocab_size, tied)
        self.has_bias = bool(spec.get("bias", False))
        self.scale = float(spec.get("scale", 1.0) or 1.0)
        self.softcap = float(spec.get("softcap", 0.0) or 0.0)
        if self.softcap < 0 or self.scale != self.scale:
            raise ConfigError("head: softcap must be >= 0 and scale a number")
        self.weight = self.bias = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = {} if self.tied else {"weight": WeightSpec((self.vocab_size, self.hidden_size))}
        if self.has_bias:
            specs["bias"] = WeightSpec((self.vocab_size,), init="zeros")
        return specs

    def load(self, tensors, dtype, tied: Optional[torch.Tensor] = None):
        if self.tied:
            if tied is None:
                raise ConfigError("head: the model ties the head to an embedding that has no table")
            self.weight = tied              # also read by rows: it stays a plain tensor
        else:
            self.weight = prepare_weight(tensors["weight"], dtype)
        self.bias = tensors.get("bias")

    def first_weight(self):
        return self.weight

    def forward(self, ctx, x):
        logits = linear(ctx, x, self.weight, out_dtype=torch.float32)
        if self.bias is not None or self.scale != 1.0 or self.softcap > 0.0:
            logits = ops.affine_rows(logits, bias=self.bias, scale=self.scale, softcap=self.softcap)
        return logits


register_part("head", "linear", LinearHead, replace=True)
