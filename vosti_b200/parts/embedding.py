"""The embedding table: hidden rows by token id (kernels/triton_kernels/embedding.py:62-84),
optionally multiplied by a constant `scale` in float32 (Qwen3 has none; architectures that
scale their embeddings by sqrt(hidden) name it in their spec).
"""
from __future__ import annotations

from typing import Dict

from .. import ops
from ..config.schema import ConfigError, PartSpec
from ..weights.loader import WeightSpec
from .base import Embedding, register_part


class TableEmbedding(Embedding):
    def __init__(self, spec: PartSpec, hidden_size: int, vocab_size: int):
        super().__init__(spec, hidden_size, vocab_size)
        self.scale = float(spec.get("scale", 1.0) or 1.0)
        if not self.scale == self.scale or self.scale in (float("inf"), float("-inf")):
            raise ConfigError("embedding: scale must be a finite number")
        self.weight = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"weight": WeightSpec((self.vocab_size, self.hidden_size), init="embedding")}

    def load(self, tensors, dtype):
        self.weight = tensors["weight"]

    def table(self):
        return self.weight

    def forward(self, ctx, tokens, feedback=None):
        return ops.embedding(tokens, self.weight, ctx.status, feedback=feedback, scale=self.scale)


register_part("embedding", "table", TableEmbedding, replace=True)
