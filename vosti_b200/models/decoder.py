"""A decoder-only model put together from a `ModelSpec`: embedding, blocks in run
order, final norm, output head.

The loop is the reference's (src/exec/dense_swiglu_model.rs:131-1041): embed; each
block maps (hidden, residual) to (hidden, residual); a last add-and-norm; rows that are
wanted are gathered (here inside the head's product) and multiplied with the head,
which is the embedding table when the embeddings are tied. Logits are float32.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from ..config.schema import ModelSpec
from ..parts import build_block, build_norm, linear, prepare_weight
from ..weights.loader import WeightSpec


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        spec.validate()
        self.spec = spec
        self.blocks = [build_block(layer, spec.hidden_size) for layer in spec.layers]
        self.final_norm = build_norm(spec.final_norm, spec.hidden_size)
        self.embed = None
        self.head = None
        self.device = None
        self.dtype = None

    # ------------------------------------------------------------ weights
    def _final_norm_prefix(self) -> str:
        name = self.spec.final_norm_name
        return name[: -len("weight")] if name.endswith("weight") else name + "."

    def expected_weights(self) -> Dict[str, WeightSpec]:
        spec = self.spec
        out = {spec.embed_name: WeightSpec((spec.vocab_size, spec.hidden_size), init="embedding")}
        for i, block in enumerate(self.blocks):
            prefix = spec.layer_prefix.format(i=i)
            for key, w in block.weight_specs().items():
                out[prefix + key] = w
        for key, w in self.final_norm.weight_specs().items():
            out[self._final_norm_prefix() + key] = w
        if not spec.tie_word_embeddings:
            out[spec.lm_head_name] = WeightSpec((spec.vocab_size, spec.hidden_size))
        return out

    def ignorable_weights(self):
        """Tensors a checkpoint may carry that this model does not read."""
        return (self.spec.lm_head_name,) if self.spec.tie_word_embeddings else ()

    def load(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype) -> None:
        spec = self.spec
        self.embed = tensors[spec.embed_name]
        for i, block in enumerate(self.blocks):
            prefix = spec.layer_prefix.format(i=i)
            block.load({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}, dtype)
        prefix = self._final_norm_prefix()
        self.final_norm.load({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}, dtype)
        # a tied head is also read by rows (the embedding): it stays a plain tensor
        self.head = self.embed if spec.tie_word_embeddings else prepare_weight(tensors[spec.lm_head_name], dtype)
        self.device, self.dtype = self.embed.device, dtype
        for block in self.blocks:
            block.setup(self.device, dtype)

    def weight_bytes(self) -> int:
        """Bytes of every distinct weight tensor one step reads."""
        seen, total = set(), 0

        def visit(obj):
            nonlocal total
            for value in vars(obj).values():
                if isinstance(value, ops.PackedWeight):
                    value = value.data
                if isinstance(value, torch.Tensor) and value.is_cuda:
                    base = value.untyped_storage().data_ptr()
                    if base not in seen:
                        seen.add(base)
                        total += value.untyped_storage().nbytes()
        for block in self.blocks:
            for _, part in block._children():
                visit(part)
        visit(self.final_norm)
        if self.head is not None:
            head = self.head.data if isinstance(self.head, ops.PackedWeight) else self.head
            seen_head = head.untyped_storage().data_ptr()
            if seen_head not in seen:
                total += head.untyped_storage().nbytes()
        return total

    # ------------------------------------------------------------ forward
    def forward(self, ctx, layer_caches: List):
        """Run every entry of the run order over the batch in `ctx`; returns the last
        block's (hidden, residual), both [T, hidden] (residual None without blocks)."""
        source = ctx.extras.get("feedback") if ctx.extras else None
        hidden = ops.embedding(ctx.tokens, self.embed, ctx.status,
                               feedback=None if source is None else (source, ctx.feedback_values))
        residual: Optional[torch.Tensor] = None
        for entry in self.spec.run_order:
            owner = entry.layer if entry.cache_from is None else entry.cache_from
            hidden, residual = self.blocks[entry.layer].forward(
                ctx, hidden, residual, layer_caches[owner], writes_cache=entry.cache_from is None)
        return hidden, residual

    def logits(self, ctx, hidden: torch.Tensor, residual: Optional[torch.Tensor], rows: torch.Tensor) -> torch.Tensor:
        """float32 logits [len(rows), vocab] of the rows (flat token indices) asked for:
        only those rows are gathered, added, normed and multiplied with the head."""
        hidden = ops.gather_rows(ops.materialize(hidden), rows, ctx.status)
        if residual is None:
            final = self.final_norm.forward(ctx, hidden)
        else:
            final = self.final_norm.forward_add(ctx, hidden, ops.gather_rows(residual, rows, ctx.status))[0]
        return linear(ctx, final, self.head, out_dtype=torch.float32)
