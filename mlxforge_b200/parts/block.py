"""Arrangements of a layer's parts around the residual stream.

``prenorm``: ``h += mixer(norm1(h)); h += feed_forward(norm2(h))`` — the
reference's block (src/model/decoder_model.cpp:288-293).  The residual stream is
32-bit; every add is fused with the norm that follows it, so a block takes the
previous block's last delta as ``pending`` and hands its own on.
"""
from __future__ import annotations

from .base import Block, register_block


@register_block("prenorm")
class PreNormBlock(Block):
    roles = ("mixer", "mixer_norm", "feed_forward", "feed_forward_norm")

    def forward(self, residual, pending, batch, cache, writes_cache: bool = True):
        x = self.mixer_norm.add_forward(residual, pending)
        d = self.mixer.forward(x, batch, cache, writes_cache)
        x = self.feed_forward_norm.add_forward(residual, d)
        d = self.feed_forward.forward(x, batch)
        return residual, d
