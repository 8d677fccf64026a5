from .base import (Embedding, FeedForward, Head, Mixer, Norm, PagedCacheSpec, Part, PositionEncoding, StateSpec,
                   build_embedding, build_feed_forward, build_head, build_mixer, build_norm, build_position,
                   part_factory, register_part, register_step_layout, unregister_part)
from .linear import linear, prepare_weight
from .norm import RMSNorm
from .rope import RotaryEncoding
from .attention import Attention
from .feed_forward import SwiGLU
from .block import PreNormBlock, build_block
from .embedding import TableEmbedding
from .head import LinearHead

__all__ = [
    "Embedding", "Head", "build_embedding", "build_head", "TableEmbedding", "LinearHead", "FeedForward", "Mixer", "Norm", "PagedCacheSpec", "Part", "PositionEncoding", "StateSpec",
    "build_feed_forward", "build_mixer", "build_norm", "build_position", "part_factory",
    "register_part", "register_step_layout", "unregister_part", "linear", "RMSNorm", "RotaryEncoding", "Attention",
    "SwiGLU", "PreNormBlock", "build_block",
]
