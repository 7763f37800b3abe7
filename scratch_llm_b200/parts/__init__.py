"""Parts a layer is put together from: mixer, feed-forward, norm, position encoding, block."""

from . import (attention, biased_attention, block, delta_rule, feed_forward, norm,  # noqa: F401
               position, token_side)                                  # (registration)
from .base import (Block, BuildContext, CacheView, FeedForward, KVSpec, Mixer, Norm, Part,
                   PositionEncoding, SideInput, StateSpec)
from .registry import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, SIDE_INPUTS, make,
                       register_block, register_feed_forward, register_mixer, register_norm,
                       register_position_encoding, register_side_input)

__all__ = ["BLOCKS", "Block", "BuildContext", "CacheView", "FEED_FORWARDS", "FeedForward", "KVSpec",
           "MIXERS", "Mixer", "NORMS", "Norm", "POSITION_ENCODINGS", "Part",
           "PositionEncoding", "SIDE_INPUTS", "SideInput", "StateSpec", "make", "register_side_input", "register_block", "register_feed_forward",
           "register_mixer", "register_norm", "register_position_encoding"]
