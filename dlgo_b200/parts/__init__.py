"""Parts a layer is put together from, each chosen by the configuration through a registry."""
from .base import Block, CacheNeed, FeedForward, Mixer, Norm, ParamSpec, Part, PositionEncoding, StateNeed
from .registry import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS,
                       register_block, register_feed_forward, register_mixer, register_norm,
                       register_position_encoding)
from . import attention, block, embedding, feedforward, norm, rope  # noqa: F401  (fill the registries)

__all__ = [
    "BLOCKS", "Block", "CacheNeed", "EMBEDDINGS", "FEED_FORWARDS", "FeedForward", "HEADS", "MIXERS", "Mixer",
    "NORMS", "Norm", "POSITION_ENCODINGS", "ParamSpec", "Part", "PositionEncoding", "StateNeed",
    "register_block", "register_feed_forward", "register_mixer", "register_norm", "register_position_encoding",
]
