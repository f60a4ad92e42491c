"""Device memory of the cache: pages per group and state slots.

Pages of a group: one tensor ``[pools, pages, kv_heads, page_size, head_dim]`` with
``pools = 2 * layers`` (keys of layer i at pool 2i, values at 2i+1), so one page id
addresses every layer of the group (``src/pretrained/continuation/page_pool.clj:4-6``)
and a page of one (layer, head) is one contiguous tile.  Element type: the runtime's
(bfloat16 when serving, float32 on the 32-bit path).

State: one tensor ``[slots, *shape]`` per (layer, name) a mixer declared, zero-filled.
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import torch

from ..csrc import ops
from .manager import GroupSpec


class CacheStorage:
    def __init__(self, groups: Sequence[GroupSpec], num_pages: Sequence[int], page_size: int,
                 dtype: torch.dtype, device, state_specs: Dict[Tuple[int, str], object],
                 num_slots: int):
        self.groups = list(groups)
        self.page_size = page_size
        self.num_pages = list(num_pages)
        self.kv: List[torch.Tensor] = []
        for g, n in zip(self.groups, self.num_pages):
            self.kv.append(torch.zeros((2 * len(g.layers), n, g.kv_heads, page_size, g.head_dim),
                                       dtype=dtype, device=device))
        self.state: Dict[Tuple[int, str], torch.Tensor] = {
            key: torch.zeros((num_slots,) + tuple(spec.shape), dtype=spec.dtype, device=device)
            for key, spec in state_specs.items()}

    def layer_pages(self, group: int, index_in_group: int):
        kv = self.kv[group]
        return kv[2 * index_in_group], kv[2 * index_in_group + 1]

    def copy_pages(self, group: int, pairs: torch.Tensor, n_pairs: int, status) -> None:
        """Copy-on-write: page pairs[i,0] -> pairs[i,1] in every pool of the group."""
        ops.copy_pages(self.kv[group], pairs, n_pairs, status)

    def copy_state(self, src_slot: int, dst_slot: int) -> None:
        """Every state tensor's row of ``src_slot`` -> row of ``dst_slot`` (a fork takes the
        source's state as it is now), on the current stream."""
        for t in self.state.values():
            t[dst_slot].copy_(t[src_slot])

    def bytes(self) -> int:
        total = sum(t.numel() * t.element_size() for t in self.kv)
        return total + sum(t.numel() * t.element_size() for t in self.state.values())
