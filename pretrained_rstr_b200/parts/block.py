"""Arrangements of parts in a block.  ``pre_norm``:
x += mixer(norm_1(x)); x += feed_forward(norm_2(x))  (``dev/examples/gpt2.clj:149-166``).
The block knows its parts only through their interfaces."""
from __future__ import annotations

from .interfaces import Block, FeedForward, LayerCache, Mixer, Norm
from .registry import register_part


class PreNormBlock(Block):
    graph_safe = True
    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm,
                 feed_forward_norm: Norm, width: int, runtime):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        self.width, self.runtime = width, runtime

    def forward(self, ctx, x, cache: LayerCache) -> None:
        t = x.shape[0]
        h = ctx.scratch("block_normed", (ctx.token_capacity, self.width), self.runtime.dtype)[:t]
        self.mixer_norm.forward(ctx, x, h)
        self.mixer.forward(ctx, h, x, cache)
        self.feed_forward_norm.forward(ctx, x, h)
        self.feed_forward.forward(ctx, h, x)


register_part("arrangement", "pre_norm", PreNormBlock)
