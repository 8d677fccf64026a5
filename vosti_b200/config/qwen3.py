"""Typed Qwen3 dense configuration, read from the family's own config.json keys.

Mirrors the reference's profile projection and validation
(python/vosti_kernels/model_families/qwen3/profile.py:41-61 required fields,
:92-100 "no defaults: a missing key is an error", :129-164 value checks) and its
typed record (src/boundary/model_families/qwen3/config.rs:9-18). Unlike the
reference, any geometry that passes the checks is accepted (there is no closed
list of profiles) and rms_norm_eps / rope_theta come from the file.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, asdict
from pathlib import Path
from typing import Any, Mapping

from .schema import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry

ARCHITECTURE = "Qwen3ForCausalLM"

_REQUIRED = (
    "model_type", "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
    "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings",
    "rms_norm_eps", "rope_theta", "tie_word_embeddings", "attention_bias",
    "attention_dropout", "hidden_act", "use_sliding_window", "sliding_window", "rope_scaling",
)
_POSITIVE_INTS = (
    "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
    "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings",
)


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool

    @staticmethod
    def from_dict(raw: Mapping[str, Any]) -> "Qwen3Config":
        if not isinstance(raw, Mapping):
            raise ConfigError("Qwen3 config must be a JSON object")
        missing = sorted(k for k in _REQUIRED if k not in raw)
        if missing:
            raise ConfigError(f"Qwen3 config lacks required keys {missing}")
        if raw["model_type"] != "qwen3":
            raise ConfigError(f"Qwen3 config has model_type {raw['model_type']!r}, expected 'qwen3'")
        for key in _POSITIVE_INTS:
            value = raw[key]
            if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
                raise ConfigError(f"Qwen3 config: {key} must be a positive integer, got {value!r}")
        for key in ("rms_norm_eps", "rope_theta"):
            value = raw[key]
            if (isinstance(value, bool) or not isinstance(value, (int, float))
                    or not math.isfinite(float(value)) or value <= 0):
                raise ConfigError(f"Qwen3 config: {key} must be a finite positive number, got {value!r}")
        if raw["num_attention_heads"] % raw["num_key_value_heads"] != 0:
            raise ConfigError("Qwen3 config: num_attention_heads must be a multiple of "
                              "num_key_value_heads")
        if raw["head_dim"] % 2 != 0:
            raise ConfigError("Qwen3 config: head_dim must be even (half-split rotation)")
        if raw["hidden_act"] != "silu":
            raise ConfigError(f"Qwen3 config: hidden_act must be 'silu', got {raw['hidden_act']!r}")
        if raw["attention_bias"] is not False:
            raise ConfigError("Qwen3 config: attention_bias must be false")
        if raw["attention_dropout"] != 0.0:
            raise ConfigError("Qwen3 config: attention_dropout must be 0.0")
        if raw["use_sliding_window"] is not False or raw["sliding_window"] is not None:
            raise ConfigError("Qwen3 config: sliding-window attention is not part of this "
                              "architecture (use_sliding_window=false, sliding_window=null)")
        if raw["rope_scaling"] is not None:
            raise ConfigError("Qwen3 config: rope_scaling must be null")
        if not isinstance(raw["tie_word_embeddings"], bool):
            raise ConfigError("Qwen3 config: tie_word_embeddings must be a boolean")
        return Qwen3Config(
            vocab_size=raw["vocab_size"], hidden_size=raw["hidden_size"],
            intermediate_size=raw["intermediate_size"],
            num_hidden_layers=raw["num_hidden_layers"],
            num_attention_heads=raw["num_attention_heads"],
            num_key_value_heads=raw["num_key_value_heads"], head_dim=raw["head_dim"],
            max_position_embeddings=raw["max_position_embeddings"],
            rms_norm_eps=float(raw["rms_norm_eps"]), rope_theta=float(raw["rope_theta"]),
            tie_word_embeddings=raw["tie_word_embeddings"],
        )

    def to_dict(self) -> dict:
        """The config.json this configuration is read back from."""
        out = asdict(self)
        out.update(
            architectures=[ARCHITECTURE], model_type="qwen3", hidden_act="silu",
            attention_bias=False, attention_dropout=0.0, use_sliding_window=False,
            sliding_window=None, rope_scaling=None, torch_dtype="bfloat16",
        )
        return out

    def to_model_spec(self) -> ModelSpec:
        """Qwen3 dense: every layer is pre-norm GQA attention with per-head q/k RMSNorm
        and full-width half-split RoPE, then a SwiGLU feed-forward
        (src/exec/dense_swiglu_decoder.rs:43-441)."""
        norm = PartSpec.make("rmsnorm", eps=self.rms_norm_eps)
        mixer = PartSpec.make(
            "attention", num_heads=self.num_attention_heads,
            num_kv_heads=self.num_key_value_heads, head_dim=self.head_dim,
            head_norm_eps=self.rms_norm_eps, window=0,
            scale=float(self.head_dim) ** -0.5,
        )
        position = PartSpec.make("rope", theta=self.rope_theta, rotary_dim=self.head_dim,
                                 max_positions=self.max_position_embeddings)
        ffn = PartSpec.make("swiglu", intermediate_size=self.intermediate_size)
        names = (("input_norm", "input_layernorm"), ("post_norm", "post_attention_layernorm"),
                 ("mixer", "self_attn"), ("feed_forward", "mlp"))
        layer = LayerSpec(mixer=mixer, feed_forward=ffn, norm=norm, position=position,
                          arrangement="pre_norm", names=names)
        n = self.num_hidden_layers
        spec = ModelSpec(
            architecture=ARCHITECTURE, hidden_size=self.hidden_size, vocab_size=self.vocab_size,
            max_positions=self.max_position_embeddings, layers=tuple(layer for _ in range(n)),
            run_order=tuple(RunEntry(i) for i in range(n)), final_norm=norm,
            tie_word_embeddings=self.tie_word_embeddings,
        )
        spec.validate()
        return spec


def spec_from_config(raw: Mapping[str, Any]) -> ModelSpec:
    return Qwen3Config.from_dict(raw).to_model_spec()


def load_config(model_dir: str | Path) -> Qwen3Config:
    return Qwen3Config.from_dict(json.loads((Path(model_dir) / "config.json").read_text()))
