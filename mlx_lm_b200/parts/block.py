"""Arrangements of parts in a layer.  ``PreNormBlock``:
``h = x + mixer(norm_1(x)); out = h + feed_forward(norm_2(h))``
(mlx_lm/models/gpt2.py:104-108).  The residual stream is updated in place by
the epilogues of the mixer's and the feed-forward's last products."""

from __future__ import annotations

import os

import torch

from .base import Block, FeedForward, Mixer, Norm, register_part

# In bfloat16 a block lets its mixer and its feed-forward fold the norm before them into their first linear
# layer (parts/linear.py, ``Linear.fold_norm``): steps of few rows then run no norm kernels inside the blocks.
# MLXB_FOLD_NORMS=0 (or setting this to False before a model is loaded) keeps every norm a kernel of its own.
FOLD_NORMS = os.environ.get("MLXB_FOLD_NORMS", "1") != "0"


class PreNormBlock(Block):
    replayable = True
    def __init__(self, norm_1: Norm, mixer: Mixer, norm_2: Norm, feed_forward: FeedForward):
        self.norm_1, self.mixer, self.norm_2, self.feed_forward = norm_1, mixer, norm_2, feed_forward
        self._defer_1 = self._defer_2 = False

    def children(self):
        return (self.norm_1, self.mixer, self.norm_2, self.feed_forward)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def bind_all(self, tensors, dtype, device) -> None:
        super().bind_all(tensors, dtype, device)
        fold = FOLD_NORMS and dtype == torch.bfloat16
        self._defer_1 = fold and self.mixer.fold_input_norm(self.norm_1)
        self._defer_2 = fold and self.feed_forward.fold_input_norm(self.norm_2)

    def forward(self, ctx, x, cache):
        n1 = self.norm_1.deferred(ctx, x) if self._defer_1 else self.norm_1.forward(ctx, x)
        h = self.mixer.forward(ctx, n1, x, cache)
        n2 = self.norm_2.deferred(ctx, h) if self._defer_2 else self.norm_2.forward(ctx, h)
        return self.feed_forward.forward(ctx, n2, h)


register_part("block", "pre_norm", PreNormBlock)
