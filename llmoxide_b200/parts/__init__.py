"""The parts a layer is put together from: mixers, feed-forwards, norms,
position encodings and their arrangement in a block.  Each takes its sizes
and constants as parameters; none knows which model it is in."""

from . import attention, block, embedding, feed_forward, head, norm, position  # noqa: F401  (register the built-in kinds)
from .block import build_block
from .linear import Linear
from .registry import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS,
                       register_arrangement, register_embedding, register_feed_forward, register_head,
                       register_mixer, register_norm, register_position)
from .runtime import Runtime

__all__ = [
    "build_block", "Linear", "Runtime", "ARRANGEMENTS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS",
    "POSITIONS", "register_arrangement", "register_embedding", "register_feed_forward", "register_head",
    "register_mixer", "register_norm", "register_position",
]
