"""Parts of a layer. Importing this package registers the built-in parts."""
from . import base, rmsnorm, rotary, attention, swiglu, block, vocab  # noqa: F401
from .base import (Block, DeferredNorm, Embedding, FeedForward, Head, Mixer, Norm, PagedKVNeed, Part, PositionEncoding,
                   StateNeed, build_part, part_class, register_block, register_embedding, register_feed_forward,
                   register_head, register_mixer, register_norm, register_position, unregister)
