"""Token embedding: x[t] = table[token[t]] + position row, gathered on the device from
token ids (the reference builds prompt embeddings on the host,
``src/pretrained/continuation/paged_decoder.clj:683-693``; here only ids cross)."""
from __future__ import annotations

import torch

from ..csrc import ops
from .interfaces import Embedding
from .registry import register_part


class TokenEmbedding(Embedding):
    graph_safe = True
    def __init__(self, table: torch.Tensor, vocab: int, width: int, runtime):
        if tuple(table.shape) != (vocab, width):
            raise ValueError(f"token_embedding: table is {list(table.shape)}, "
                             f"expected [{vocab}, {width}]")
        self.table = table.to(runtime.dtype).contiguous()
        self.vocab, self.width = vocab, width

    def forward(self, ctx, position, x) -> None:
        ops.embed(x, ctx.tokens, ctx.positions, self.table, position.table(), ctx.status)


register_part("embedding", "token_embedding",
              lambda p, store, rt: TokenEmbedding(store.get(p["weights"] + ".weight", rt.dtype),
                                                  p["vocab"], p["width"], rt))
