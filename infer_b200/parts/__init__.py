"""Parts of a layer. Importing this package registers the built-in parts."""
from . import base, rmsnorm, rotary, attention, swiglu, block  # noqa: F401
from .base import (Block, DeferredNorm, FeedForward, Mixer, Norm, PagedKVNeed, Part, PositionEncoding, StateNeed, build_part,
                   part_class, register_block, register_feed_forward, register_mixer, register_norm,
                   register_position, unregister)
