"""A decoder-only model put together from a `ModelSpec`: embedding, blocks in run
order, final norm, output head, each of them a part chosen by the spec.

The loop is the reference's (src/exec/dense_swiglu_model.rs:131-1041): embed; each
block maps (hidden, residual) to (hidden, residual); a last add-and-norm; rows that are
wanted are gathered and multiplied with the head, which is the embedding table when the
embeddings are tied. Logits are float32.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from ..config.schema import ModelSpec
from ..parts import build_block, build_embedding, build_head, build_norm
from ..weights.loader import WeightSpec


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        spec.validate()
        self.spec = spec
        self.blocks = [build_block(layer, spec.hidden_size) for layer in spec.layers]
        self.final_norm = build_norm(spec.final_norm, spec.hidden_size)
        self.embedding = build_embedding(spec.embedding, spec.hidden_size, spec.vocab_size)
        self.head = build_head(spec.head, spec.hidden_size, spec.vocab_size, spec.tie_word_embeddings)
        self.device = None
        self.dtype = None

    def parts(self):
        """Every part of the model."""
        yield self.embedding
        for block in self.blocks:
            for _, part in block._children():
                yield part
            position = getattr(block.mixer, "position", None)
            if position is not None:
                yield position
        yield self.final_norm
        yield self.head

    @property
    def capture_safe(self) -> bool:
        """Whether a decode step of this model may be recorded as a CUDA graph and replayed:
        every part must launch the same kernels with the same arguments for every step of a
        shape (see parts.base.Part.capture_safe)."""
        return all(getattr(part, "capture_safe", True) for part in self.parts()) and \
            all(getattr(block, "capture_safe", True) for block in self.blocks)

    # ------------------------------------------------------------ weights
    @staticmethod
    def _prefix_of(name: str) -> str:
        """'model.norm.weight' -> 'model.norm.': the names in a spec are those of a part's
        `weight` tensor; its other tensors (a bias) stand beside it."""
        return name[: -len("weight")] if name.endswith("weight") else name + "."

    def _final_norm_prefix(self) -> str:
        return self._prefix_of(self.spec.final_norm_name)

    def expected_weights(self) -> Dict[str, WeightSpec]:
        spec = self.spec
        out = {self._prefix_of(spec.embed_name) + key: w for key, w in self.embedding.weight_specs().items()}
        for i, block in enumerate(self.blocks):
            prefix = spec.layer_prefix.format(i=i)
            for key, w in block.weight_specs().items():
                out[prefix + key] = w
        for key, w in self.final_norm.weight_specs().items():
            out[self._final_norm_prefix() + key] = w
        for key, w in self.head.weight_specs().items():
            out[self._prefix_of(spec.lm_head_name) + key] = w
        return out

    def ignorable_weights(self):
        """Tensors a checkpoint may carry that this model does not read."""
        return (self.spec.lm_head_name,) if self.spec.tie_word_embeddings else ()

    def tied_weights(self) -> Dict[str, str]:
        """Tensors a checkpoint may carry although this model reads another in their place,
        mapped to that other tensor: if present they must hold the same values."""
        spec = self.spec
        return {spec.lm_head_name: spec.embed_name} if spec.tie_word_embeddings else {}

    def load(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype) -> None:
        spec = self.spec
        under = lambda prefix: {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}
        self.embedding.load(under(self._prefix_of(spec.embed_name)), dtype)
        for i, block in enumerate(self.blocks):
            block.load(under(spec.layer_prefix.format(i=i)), dtype)
        self.final_norm.load(under(self._final_norm_prefix()), dtype)
        expected = self.head.weight_specs()
        head_tensors = {k: v for k, v in under(self._prefix_of(spec.lm_head_name)).items() if k in expected}
        self.head.load(head_tensors, dtype, tied=self.embedding.table() if spec.tie_word_embeddings else None)
        self.device = next(iter(tensors.values())).device
        self.dtype = dtype
        for part in (self.embedding, self.final_norm, self.head):
            part.setup(self.device, dtype)
        for block in self.blocks:
            block.setup(self.device, dtype)

    def weight_bytes(self) -> int:
        """Bytes of every distinct weight tensor one step reads whole: the blocks, the final
        norm and the head. The embedding table is not among them (a step reads one row per
        token) unless the head is tied to it."""
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
        visit(self.head)          # a tied head is the embedding table, read whole by the head's product
        return total

    # ------------------------------------------------------------ forward
    def forward(self, ctx, layer_caches: List):
        """Run every entry of the run order over the batch in `ctx`; returns the last
        block's (hidden, residual), both [T, hidden] (residual None without blocks)."""
        source = ctx.extras.get("feedback") if ctx.extras else None
        hidden = self.embedding.forward(ctx, ctx.tokens,
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
        return self.head.forward(ctx, final)
