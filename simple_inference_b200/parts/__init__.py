"""Parts a model is put together from: mixers, feed-forwards, norms, position encodings, blocks."""

from .base import (Block, CacheSpec, FeedForward, LayerCache, Mixer, Norm, PagedKVSpec, Part,
                   PartSpec, PositionEncoding, Runtime, StateSpec, TensorSpec)
from .registry import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, UnknownPartError,
                       register_block, register_feed_forward, register_mixer, register_norm,
                       register_position_encoding)
from . import norm, rope, attention, mlp, embedding, block  # noqa: F401  (register the built-in kinds)

__all__ = [
    "Block", "CacheSpec", "FeedForward", "LayerCache", "Mixer", "Norm", "PagedKVSpec", "Part",
    "PartSpec", "PositionEncoding", "Runtime", "StateSpec", "TensorSpec", "BLOCKS",
    "FEED_FORWARDS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "UnknownPartError",
    "register_block", "register_feed_forward", "register_mixer", "register_norm",
    "register_position_encoding",
]
