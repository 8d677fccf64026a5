"""Architecture-neutral description of a model: parts, layers and run order.

A model is a list of layers; each layer names its parts (mixer, feed-forward,
norm, position encoding) by *kind* with the constants of that part as plain
parameters. The order in which layers run is data as well (`RunEntry`), so a
layer may run twice or read the cache another layer wrote. Nothing here knows
a model family; families translate their own ``config.json`` into a
`ModelSpec` (see `vosti_b200.config.qwen3`).

The reference keeps the same information in closed enums
(src/model_config.rs:10-60: ModelArchitecture, AttentionKind, DenseGeometry);
this schema is open so that new kinds register without touching it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


class ConfigError(ValueError):
    """A configuration that is missing a key or holds an unusable value."""


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: a registered kind and that kind's constants."""

    kind: str
    params: Tuple[Tuple[str, Any], ...] = ()

    @staticmethod
    def make(kind: str, **params: Any) -> "PartSpec":
        return PartSpec(kind, tuple(sorted(params.items())))

    def get(self, name: str, default: Any = None) -> Any:
        for key, value in self.params:
            if key == name:
                return value
        return default

    def __getitem__(self, name: str) -> Any:
        for key, value in self.params:
            if key == name:
                return value
        raise ConfigError(f"part '{self.kind}' has no parameter '{name}'")

    def as_dict(self) -> dict:
        return dict(self.params)


@dataclass(frozen=True)
class LayerSpec:
    """A block: which mixer, feed-forward, norm and position encoding it uses
    and how they are arranged. ``names`` maps the block's roles to the weight
    name fragments of the checkpoint it is loaded from."""

    mixer: PartSpec
    feed_forward: Optional[PartSpec]
    norm: PartSpec
    position: Optional[PartSpec]
    arrangement: str = "pre_norm"
    names: Tuple[Tuple[str, str], ...] = ()

    def name_of(self, role: str) -> str:
        for key, value in self.names:
            if key == role:
                return value
        return role


@dataclass(frozen=True)
class RunEntry:
    """One entry of the run order: run ``layer``; if ``cache_from`` is set the
    layer's mixer reads the cache (or state) that layer wrote instead of
    keeping one of its own."""

    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    layers: Tuple[LayerSpec, ...]
    run_order: Tuple[RunEntry, ...]
    final_norm: PartSpec
    tie_word_embeddings: bool
    embed_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm.weight"
    lm_head_name: str = "lm_head.weight"
    layer_prefix: str = "model.layers.{i}."
    embedding: PartSpec = PartSpec("table")      # token ids -> hidden rows (parameter: scale)
    head: PartSpec = PartSpec("linear")          # hidden rows -> logits (parameters: bias, scale, softcap)
    extra: Mapping[str, Any] = field(default_factory=dict)

    def validate(self) -> None:
        if self.hidden_size <= 0 or self.vocab_size <= 0 or self.max_positions <= 0:
            raise ConfigError("hidden_size, vocab_size and max_positions must be positive")
        if not self.layers and self.run_order:
            raise ConfigError("run order names layers but the model has none")
        for entry in self.run_order:
            if not 0 <= entry.layer < len(self.layers):
                raise ConfigError(f"run order names layer {entry.layer}, "
                                  f"model has {len(self.layers)}")
            if entry.cache_from is not None:
                if not 0 <= entry.cache_from < len(self.layers):
                    raise ConfigError(f"run order reads cache of layer {entry.cache_from}, "
                                      f"model has {len(self.layers)}")
