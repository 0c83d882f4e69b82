"""Arrangements of parts into a layer. "prenorm": h += mixer(norm(h)); h += feed_forward(norm(h))
(src/forward.cpp:200-244). The residual stream h is float32; the sums happen in the parts' last
matrix product, in float32."""
from __future__ import annotations

from .base import Block, register_block


@register_block("prenorm")
class PreNormBlock(Block):
    def forward(self, h, step, cache, write_cache=True):
        h = self.mixer.forward(self.mixer_norm.forward(h), step, cache, h, write_cache)
        return self.feed_forward.forward(self.feed_forward_norm.forward(h), h)
