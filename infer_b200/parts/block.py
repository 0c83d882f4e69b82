"""Arrangements of parts into a layer. "prenorm": h += mixer(norm(h)); h += feed_forward(norm(h))
(src/forward.cpp:200-244). The residual stream h is float32; the sums happen in the parts' last
matrix product, in float32."""
from __future__ import annotations

from .base import Block, DeferredNorm, register_block

DEFER_MAX_ROWS = 16      # the kernels that normalise on the fly take up to this many rows


def normed_input(norm, consumer, h):
    """norm(h), or, for a few rows and a consumer that can normalise inside its first kernel, the norm deferred."""
    if (consumer.accepts_deferred_norm and h.shape[0] <= DEFER_MAX_ROWS and norm.rt.fast("norm")
            and getattr(norm, "fusable", False)):
        return DeferredNorm(norm, h)
    return norm.forward(h)


@register_block("prenorm")
class PreNormBlock(Block):
    def forward(self, h, step, cache, write_cache=True):
        h = self.mixer.forward(normed_input(self.mixer_norm, self.mixer, h), step, cache, h, write_cache)
        return self.feed_forward.forward(normed_input(self.feed_forward_norm, self.feed_forward, h), h)
