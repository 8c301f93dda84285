"""Layer parts: mixers, feed-forwards, norms, position encodings, block arrangements."""
from .base import (FeedForward, Mixer, Norm, PagedNeed, ParamDecl, Part, Position, StateNeed)
from .registry import (build_block, build_feed_forward, build_mixer, build_norm, build_position,
                       register_block, register_feed_forward, register_mixer, register_norm,
                       register_position, registered, unregister)
from . import attention, block, feed_forward, norm, rope, short_conv  # noqa: F401  (register the built-in parts)

__all__ = [
    "FeedForward", "Mixer", "Norm", "PagedNeed", "ParamDecl", "Part", "Position", "StateNeed",
    "build_block", "build_feed_forward", "build_mixer", "build_norm", "build_position",
    "register_block", "register_feed_forward", "register_mixer", "register_norm",
    "register_position", "registered", "unregister",
]
