from . import attention, block, embedding, feed_forward, head, norms, positions  # noqa: F401  (register)
from .interfaces import (Block, Embedding, FeedForward, Head, KVSpec, LayerCache, Mixer, Norm,
                         PositionEncoding, StateSpec)
from .linear import Linear
from .registry import build_part, part_factory, register_part, registered_parts

__all__ = ["Block", "Embedding", "FeedForward", "Head", "KVSpec", "LayerCache", "Mixer", "Norm",
           "PositionEncoding", "StateSpec", "Linear", "build_part", "part_factory",
           "register_part", "registered_parts"]
