"""Parts a model is put together from: embeddings, mixers, feed-forwards, norms, position
encodings, blocks and output heads."""

from .base import (Block, CacheSpec, Embedding, FeedForward, Head, LayerCache, Mixer, Norm,
                   PagedKVSpec, Part, PartSpec, PositionEncoding, Runtime, StateSpec, StepPlanner,
                   TensorSpec)
from .registry import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS,
                       UnknownPartError, register_block, register_embedding, register_feed_forward,
                       register_head, register_mixer, register_norm, register_position_encoding)
from . import norm, rope, attention, mlp, embedding, block  # noqa: F401  (register the built-in kinds)

__all__ = [
    "Block", "CacheSpec", "Embedding", "FeedForward", "Head", "LayerCache", "Mixer", "Norm",
    "PagedKVSpec", "Part", "PartSpec", "PositionEncoding", "Runtime", "StateSpec", "StepPlanner",
    "TensorSpec", "BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS",
    "POSITION_ENCODINGS", "UnknownPartError", "register_block", "register_embedding",
    "register_feed_forward", "register_head", "register_mixer", "register_norm",
    "register_position_encoding",
]
