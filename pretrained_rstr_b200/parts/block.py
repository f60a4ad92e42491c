"""Arrangements of parts in a block.  ``pre_norm``:
x += mixer(norm_1(x)); x += feed_forward(norm_2(x))  (``dev/examples/gpt2.clj:149-166``).
The block knows its parts only through their interfaces."""
from __future__ import annotations

from typing import Dict

from .interfaces import Block, FeedForward, LayerCache, Mixer, Norm
from .linear import LazyNorm
from .registry import register_part


class PreNormBlock(Block):
    graph_safe = True
    def __init__(self, mixer: Mixer, feed_forward: FeedForward, norms: Dict[str, Norm],
                 width: int, runtime):
        missing = {"mixer", "feed_forward"} - set(norms)
        if missing or len(norms) != 2:
            raise ValueError(f"pre_norm wants the norms 'mixer' and 'feed_forward', got {sorted(norms)}")
        self.mixer, self.feed_forward = mixer, feed_forward
        self.norms = dict(norms)
        self.mixer_norm, self.feed_forward_norm = norms["mixer"], norms["feed_forward"]
        self.width, self.runtime = width, runtime

    def forward(self, ctx, x, cache: LayerCache) -> None:
        t = x.shape[0]
        h = ctx.scratch("block_normed", (ctx.token_capacity, self.width), self.runtime.dtype)[:t]
        self.mixer.forward(ctx, self._normed(ctx, self.mixer, self.mixer_norm, x, h), x, cache)
        self.feed_forward.forward(
            ctx, self._normed(ctx, self.feed_forward, self.feed_forward_norm, x, h), x)

    @staticmethod
    def _normed(ctx, consumer, norm, x, out):
        """The consumer's input: a norm that has run, or, for consumers that say they take
        one (``accepts_lazy_norm``), a :class:`LazyNorm` they may fuse into their first
        matrix product."""
        lazy = LazyNorm(ctx, norm, x, out)
        return lazy if getattr(consumer, "accepts_lazy_norm", False) else lazy.tensor()


register_part("arrangement", "pre_norm", PreNormBlock)
