"""Position encodings.  ``learned_absolute``: a table with one row per position that is
added to the token embedding (``dev/examples/gpt2.clj:49-62``).  ``none``: nothing."""
from __future__ import annotations

import torch

from .interfaces import PositionEncoding
from .registry import register_part


class LearnedAbsolute(PositionEncoding):
    graph_safe = True
    def __init__(self, table: torch.Tensor, positions: int, width: int, runtime):
        if tuple(table.shape) != (positions, width):
            raise ValueError(f"learned_absolute: table is {list(table.shape)}, "
                             f"expected [{positions}, {width}]")
        self._table = table.to(runtime.dtype).contiguous()
        self.positions = positions

    def table(self):
        return self._table


class NoPosition(PositionEncoding):
    graph_safe = True
    pass


register_part("position", "learned_absolute",
              lambda p, store, rt: LearnedAbsolute(store.get(p["weights"] + ".weight", rt.dtype),
                                                   p["positions"], p["width"], rt))
register_part("position", "none", lambda p, store, rt: NoPosition())
