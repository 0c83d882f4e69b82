"""Arrangements of parts into a layer. "prenorm": h += mixer(norm(h)); h += feed_forward(norm(h))
(src/forward.cpp:200-244), over the slots mixer_norm, mixer, feed_forward_norm, feed_forward. The residual stream h
is float32; the sums happen in the parts' last matrix product, in float32."""
from __future__ import annotations

from .base import Block, DeferredNorm, register_block


def normed_input(norm, consumer, h):
    """norm(h), or, for as few rows as the streaming product takes and a consumer that can normalise inside its
    first kernel, the norm deferred. How many rows that is, is the kernel library's answer, not a constant here."""
    if consumer.accepts_deferred_norm and getattr(norm, "fusable", False) and norm.rt.fast("norm"):
        from .. import fast_ops
        if h.shape[0] <= fast_ops.skinny_limits()[0]:
            return DeferredNorm(norm, h)
    return norm.forward(h)


@register_block("prenorm")
class PreNormBlock(Block):
    def __init__(self, mixer_norm, mixer, feed_forward_norm, feed_forward):
        super().__init__(mixer_norm=mixer_norm, mixer=mixer, feed_forward_norm=feed_forward_norm, feed_forward=feed_forward)

    def forward(self, h, step, cache, write_cache=True):
        h = self.mixer.forward(normed_input(self.mixer_norm, self.mixer, h), step, cache, h, write_cache)
        return self.feed_forward.forward(normed_input(self.feed_forward_norm, self.feed_forward, h), h)
