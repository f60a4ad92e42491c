"""Output head.  ``tied_head``: logits[r, v] = sum_d h[r, d] * table[v, d] with the token
table as the matrix and no bias (``dev/examples/gpt2.clj:108-122``); logits are float32."""
from __future__ import annotations

import torch

from .interfaces import Head
from .linear import Linear
from .registry import register_part


class TiedHead(Head):
    graph_safe = True
    accepts_lazy_norm = True        # ``h`` may be a LazyNorm: few rows are normed inside the product
    def __init__(self, table: torch.Tensor, vocab: int, width: int, runtime):
        if tuple(table.shape) != (vocab, width):
            raise ValueError(f"tied_head: table is {list(table.shape)}, expected [{vocab}, {width}]")
        self.linear = Linear(table, None, runtime)      # [vocab, width] is already [out, in]
        self.vocab = vocab

    def forward(self, ctx, h, logits) -> None:
        self.linear.forward(ctx, h, logits)


register_part("head", "tied_head",
              lambda p, store, rt: TiedHead(store.get(p["weights"] + ".weight", rt.dtype),
                                            p["vocab"], p["width"], rt))
