"""Parts: norm, position encoding, mixer, feed-forward, embedding, head, block arrangement."""

from .base import (Block, Embedding, FeedForward, Head, LayerCache, Mixer, Norm, Part, PositionEncoding,
                   ResidualStream)
from .registry import (kinds, lookup, register_block, register_embedding, register_feed_forward, register_head,
                       register_mixer, register_norm, register_position)
from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401  (register the built-in kinds)

__all__ = ["Block", "Embedding", "FeedForward", "Head", "LayerCache", "Mixer", "Norm", "Part", "PositionEncoding",
           "ResidualStream", "kinds", "lookup", "register_block", "register_embedding", "register_feed_forward",
           "register_head", "register_mixer", "register_norm", "register_position"]
