"""The parts a layer is put together from: mixers, feed-forwards, norms,
position encodings and their arrangement in a block.  Each takes its sizes
and constants as parameters; none knows which model it is in."""

from . import attention, block, feed_forward, norm, position  # noqa: F401  (register the built-in kinds)
from .block import build_block
from .linear import Linear
from .registry import (ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, register_arrangement,
                       register_feed_forward, register_mixer, register_norm, register_position)
from .runtime import Runtime

__all__ = [
    "build_block", "Linear", "Runtime", "ARRANGEMENTS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS",
    "register_arrangement", "register_feed_forward", "register_mixer", "register_norm", "register_position",
]
