"""Interfaces of the parts a layer is put together from, and their registries.

A part is built from a `PartSpec` (its kind and constants) and the model's
hidden width; it declares the tensors it needs by name (`weight_specs`), takes
them in `load`, and computes in `forward`. No part knows which model it is in.

* Norm:            forward(x) / forward_add(x, residual)
* PositionEncoding: tables the mixer applies (cos/sin for a rotation), or nothing
* Mixer:           forward(ctx, x, cache, writes_cache) -> y. It declares what it keeps per
                   token in pages (`cache_spec`) and what it keeps per request in a slot
                   of fixed size (`state_spec`).
* FeedForward:     forward(ctx, x) -> y
* Arrangement:     how a block wires mixer, feed-forward and norms around the residual.
* Embedding:       forward(ctx, tokens, feedback) -> hidden rows; `table()` for a tied head
* Head:            forward(ctx, x) -> float32 logits

A part whose `forward` reads the step's host-side copies (`ctx.host_q_lens`,
`ctx.host_kv_lens`, `ctx.host_state_slots`), or lets the host decide anything from a step's
values, sets `capture_safe = False`: a CUDA graph would replay the launches of the step it
was recorded in. The engine replays decode steps as graphs only for models all of whose
parts are capture-safe.

The reference has the same roles as closed Rust records
(src/boundary/dense_swiglu_decoder.rs:18-24, 96-106).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional, Tuple

import torch

from ..config.schema import ConfigError, PartSpec
from ..weights.loader import WeightSpec


@dataclass(frozen=True)
class PagedCacheSpec:
    """Per-token cache of a mixer: `entries` tensors (keys and values: 2), each
    [tokens, heads, width] per token; `window` > 0 means only the last `window`
    tokens are ever read again, so older pages may be given back."""

    entries: int
    heads: int
    width: int
    window: int = 0


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size: one tensor of `shape` per request slot,
    zeroed when a request takes the slot."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    capture_safe = True     # False: this part's launches depend on host-side values of the step

    def __init__(self, spec: PartSpec, hidden_size: int):
        self.spec = spec
        self.hidden_size = hidden_size

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {}

    def load(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype) -> None:
        """Take the tensors named in `weight_specs` (relative names)."""

    def setup(self, device: torch.device, dtype: torch.dtype) -> None:
        """Build device tables that do not come from the checkpoint."""

    def first_weight(self):
        """The weight this part's first product streams, if the kernel before it may ask for it
        to be brought into L2 ahead of time (ops.hint_prefetch), else None."""
        return None


class Norm(Part):
    def forward(self, ctx, x):
        raise NotImplementedError

    def forward_add(self, ctx, x, residual):
        """Return (norm(x + residual), x + residual)."""
        raise NotImplementedError


class PositionEncoding(Part):
    def __init__(self, spec: PartSpec, hidden_size: int, head_dim: int):
        super().__init__(spec, hidden_size)
        self.head_dim = head_dim

    # A rotation takes the first `rotary_dim` elements of every q and k head (None: the whole
    # head) in pairs (i, i + rotary_dim/2), or neighbours (2i, 2i + 1) if `interleaved`.
    rotary_dim: Optional[int] = None
    interleaved: bool = False

    def rotation_tables(self) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
        """float32 cos and sin [max_positions, rotary_dim/2] for the rotation of q and k, or
        None if this encoding is not a rotation."""
        return None


class Mixer(Part):
    def __init__(self, spec: PartSpec, hidden_size: int, position: Optional[PositionEncoding]):
        super().__init__(spec, hidden_size)
        self.position = position

    def cache_spec(self) -> Optional[PagedCacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def forward(self, ctx, x, cache, writes_cache: bool = True):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, x):
        raise NotImplementedError


class Embedding(Part):
    """Token ids to rows of the hidden width. `feedback` = (source, values) names tokens to take
    from a device array instead (see ops.embedding)."""

    def __init__(self, spec: PartSpec, hidden_size: int, vocab_size: int):
        super().__init__(spec, hidden_size)
        self.vocab_size = vocab_size

    def forward(self, ctx, tokens, feedback=None):
        raise NotImplementedError

    def table(self) -> Optional[torch.Tensor]:
        """The [vocab, hidden] tensor a tied output head multiplies with, or None if this
        embedding has no such table."""
        return None


class Head(Part):
    """Final hidden rows to float32 logits [rows, vocab]. `load` gets `tied`, the embedding's
    table, when the model ties them (then `weight_specs` must not ask for a matrix)."""

    def __init__(self, spec: PartSpec, hidden_size: int, vocab_size: int, tied: bool):
        super().__init__(spec, hidden_size)
        self.vocab_size, self.tied = vocab_size, tied

    def load(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype, tied: Optional[torch.Tensor] = None) -> None:
        raise NotImplementedError

    def forward(self, ctx, x):
        raise NotImplementedError


_REGISTRIES: Dict[str, Dict[str, Callable]] = {
    "norm": {}, "position": {}, "mixer": {}, "feed_forward": {}, "arrangement": {}, "embedding": {}, "head": {},
}


# Step-layout providers: a kind of part that needs index arrays of its own for a step (the
# attention kernels want the step's tokens sorted into work lists) registers a function,
# q_lens -> (int32 arrays by name, host values by name). The step layout calls every provider for
# every step; the arrays travel in the step's one host-to-device copy and appear in ctx.extras as
# "<provider>.<array>", the host values in ctx.layout[provider]. The layout knows no provider by name.
_STEP_LAYOUTS: Dict[str, Callable] = {}


def register_step_layout(name: str, provider: Callable) -> None:
    _STEP_LAYOUTS[name] = provider


def step_layout_providers() -> Dict[str, Callable]:
    return _STEP_LAYOUTS


def register_part(role: str, kind: str, factory: Callable, *, replace: bool = False) -> None:
    """Register `factory` for parts of `role` ('norm', 'position', 'mixer', 'feed_forward',
    'arrangement', 'embedding', 'head') with the given kind."""
    if role not in _REGISTRIES:
        raise ConfigError(f"unknown part role '{role}'; roles: {sorted(_REGISTRIES)}")
    if kind in _REGISTRIES[role] and not replace:
        raise ConfigError(f"{role} kind '{kind}' is already registered")
    _REGISTRIES[role][kind] = factory


def unregister_part(role: str, kind: str) -> None:
    _REGISTRIES[role].pop(kind, None)


def part_factory(role: str, kind: str) -> Callable:
    table = _REGISTRIES[role]
    if kind not in table:
        raise ConfigError(f"unknown {role} kind '{kind}'; known: {sorted(table)}")
    return table[kind]


def build_norm(spec: PartSpec, width: int) -> Norm:
    return part_factory("norm", spec.kind)(spec, width)


def build_position(spec: Optional[PartSpec], hidden_size: int, head_dim: int) -> Optional[PositionEncoding]:
    if spec is None:
        return None
    return part_factory("position", spec.kind)(spec, hidden_size, head_dim)


def build_mixer(spec: PartSpec, hidden_size: int, position_spec: Optional[PartSpec]) -> Mixer:
    """The mixer with its position encoding, which is built for the mixer's `head_dim` parameter
    or, for a mixer without heads, for the hidden width."""
    factory = part_factory("mixer", spec.kind)
    width = spec.get("head_dim", 0) or hidden_size
    return factory(spec, hidden_size, build_position(position_spec, hidden_size, width))


def build_embedding(spec: PartSpec, hidden_size: int, vocab_size: int) -> Embedding:
    return part_factory("embedding", spec.kind)(spec, hidden_size, vocab_size)


def build_head(spec: PartSpec, hidden_size: int, vocab_size: int, tied: bool) -> Head:
    return part_factory("head", spec.kind)(spec, hidden_size, vocab_size, tied)


def build_feed_forward(spec: Optional[PartSpec], hidden_size: int) -> Optional[FeedForward]:
    if spec is None:
        return None
    return part_factory("feed_forward", spec.kind)(spec, hidden_size)
