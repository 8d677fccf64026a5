from .base import (FeedForward, Mixer, Norm, PagedCacheSpec, Part, PositionEncoding, StateSpec,
                   build_feed_forward, build_mixer, build_norm, build_position, part_factory,
                   register_part, unregister_part)
from .linear import linear, prepare_weight
from .norm import RMSNorm
from .rope import RotaryEncoding
from .attention import Attention
from .feed_forward import SwiGLU
from .block import PreNormBlock, build_block

__all__ = [
    "FeedForward", "Mixer", "Norm", "PagedCacheSpec", "Part", "PositionEncoding", "StateSpec",
    "build_feed_forward", "build_mixer", "build_norm", "build_position", "part_factory",
    "register_part", "unregister_part", "linear", "RMSNorm", "RotaryEncoding", "Attention",
    "SwiGLU", "PreNormBlock", "build_block",
]
