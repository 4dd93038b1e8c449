from .base import (Arrangement, FeedForward, FixedState, Mixer, Norm, PagedKV, Part,
                   PositionEncoding, Precision, build_arrangement, build_feed_forward,
                   build_mixer, build_norm, build_position, register_arrangement,
                   register_feed_forward, register_mixer, register_norm, register_position)
from . import attention, block, norm, rope, shortconv, swiglu  # noqa: F401  (register the parts)

__all__ = [
    "Arrangement", "FeedForward", "FixedState", "Mixer", "Norm", "PagedKV", "Part",
    "PositionEncoding", "Precision", "build_arrangement", "build_feed_forward", "build_mixer",
    "build_norm", "build_position", "register_arrangement", "register_feed_forward",
    "register_mixer", "register_norm", "register_position",
]
