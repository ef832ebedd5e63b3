"""Parts: norms, position encodings, mixers, feed-forwards and blocks."""
from .base import (Adapter, Block, FeedForward, FixedStateNeed, Mixer, Norm, PagedKVNeed, Part,
                   PositionEncoding, Runtime, TensorSpec, make_adapter, make_block, make_feed_forward,
                   make_mixer, make_norm, make_position, register_adapter, register_block,
                   register_feed_forward, register_mixer, register_norm, register_position)
from . import norm, rope, attention, mlp, block  # noqa: F401  (registers the built-in kinds)

__all__ = ["Adapter", "make_adapter", "register_adapter", "Block", "FeedForward", "FixedStateNeed", "Mixer", "Norm", "PagedKVNeed", "Part",
           "PositionEncoding", "Runtime", "TensorSpec", "make_block", "make_feed_forward",
           "make_mixer", "make_norm", "make_position", "register_block", "register_feed_forward",
           "register_mixer", "register_norm", "register_position"]
