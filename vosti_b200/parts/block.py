"""A block: mixer, feed-forward and their norms around the residual stream.

'pre_norm' is the reference's wiring with a deferred add
(src/exec/dense_swiglu_decoder.rs:556-615, 740-813, 370-383): a block receives
(hidden, residual), norms hidden + residual (the first block norms the embedding and
adds nothing), runs the mixer, norms mixer_out + residual, runs the feed-forward and
returns (feed_forward_out, residual); the model's final norm does the last add.
"""
from __future__ import annotations

from typing import Dict

from .. import ops
from ..config.schema import ConfigError, LayerSpec
from ..weights.loader import WeightSpec
from .base import build_feed_forward, build_mixer, build_norm, part_factory, register_part


class PreNormBlock:
    def __init__(self, spec: LayerSpec, hidden_size: int):
        self.spec = spec
        self.mixer = build_mixer(spec.mixer, hidden_size, spec.position)
        self.feed_forward = build_feed_forward(spec.feed_forward, hidden_size)
        self.input_norm = build_norm(spec.norm, hidden_size)
        self.post_norm = build_norm(spec.norm, hidden_size) if self.feed_forward is not None else None

    def _children(self):
        n = self.spec.name_of
        yield n("input_norm"), self.input_norm
        yield n("mixer"), self.mixer
        if self.feed_forward is not None:
            yield n("post_norm"), self.post_norm
            yield n("feed_forward"), self.feed_forward

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {f"{name}.{key}": spec for name, part in self._children()
                for key, spec in part.weight_specs().items()}

    def load(self, tensors, dtype):
        for name, part in self._children():
            prefix = name + "."
            part.load({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}, dtype)

    def setup(self, device, dtype):
        for _, part in self._children():
            part.setup(device, dtype)

    def forward(self, ctx, hidden, residual, cache, writes_cache=True):
        # In a step of few tokens a norm leaves HBM idle: it is told which weight the product
        # after it will stream, so that it can ask for it ahead of time (ops.hint_prefetch).
        few = ctx.num_tokens <= ops.PREFETCH_MAX_TOKENS
        if residual is None:
            residual = hidden = ops.materialize(hidden)
            normed = self.input_norm.forward(ctx, hidden)
        else:
            hinted = few and ops.hint_prefetch(self.mixer.first_weight())
            normed, residual = self.input_norm.forward_add(ctx, hidden, residual)
            if hinted:
                ops.hint_prefetch(None)
        out = self.mixer.forward(ctx, normed, cache, writes_cache)
        # (a mixer or feed-forward may return its last product as unsummed K splits; the
        # norm that follows adds them, see ops.PartialSum)
        if self.feed_forward is not None:
            hinted = few and ops.hint_prefetch(self.feed_forward.first_weight())
            normed, residual = self.post_norm.forward_add(ctx, out, residual)
            if hinted:
                ops.hint_prefetch(None)
            out = self.feed_forward.forward(ctx, normed)
        return out, residual


register_part("arrangement", "pre_norm", PreNormBlock, replace=True)


def build_block(spec: LayerSpec, hidden_size: int):
    return part_factory("arrangement", spec.arrangement)(spec, hidden_size)
