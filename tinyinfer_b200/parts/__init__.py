from .base import (Block, CacheNeed, FeedForward, Mixer, Norm, Part, PositionEncoding, StateNeed,
                   TensorSpec, build_block, build_feed_forward, build_mixer, build_norm,
                   build_position, register_block, register_feed_forward, register_mixer,
                   register_norm, register_position)
from . import attention, block, feedforward, norm, position  # noqa: F401  (register the built-in parts)

__all__ = [
    "Block", "CacheNeed", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "StateNeed",
    "TensorSpec", "build_block", "build_feed_forward", "build_mixer", "build_norm",
    "build_position", "register_block", "register_feed_forward", "register_mixer",
    "register_norm", "register_position",
]
