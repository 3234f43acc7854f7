"""Arrangements of parts in a layer.  ``PreNormBlock``:
``h = x + mixer(norm_1(x)); out = h + feed_forward(norm_2(h))``
(mlx_lm/models/gpt2.py:104-108).  The residual stream is updated in place by
the epilogues of the mixer's and the feed-forward's last products."""

from __future__ import annotations

from .base import Block, FeedForward, Mixer, Norm, register_part


class PreNormBlock(Block):
    replayable = True
    def __init__(self, norm_1: Norm, mixer: Mixer, norm_2: Norm, feed_forward: FeedForward):
        self.norm_1, self.mixer, self.norm_2, self.feed_forward = norm_1, mixer, norm_2, feed_forward

    def children(self):
        return (self.norm_1, self.mixer, self.norm_2, self.feed_forward)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, ctx, x, cache):
        h = self.mixer.forward(ctx, self.norm_1.forward(ctx, x), x, cache)
        return self.feed_forward.forward(ctx, self.norm_2.forward(ctx, h), h)


register_part("block", "pre_norm", PreNormBlock)
