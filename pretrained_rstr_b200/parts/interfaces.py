"""The interfaces parts implement.  The step function and the block only use these.

Conventions shared by all parts
-------------------------------
* The residual stream ``x`` is float32 ``[T, width]`` in both precisions; a part that
  adds to it does so in place, in 32-bit.
* Normed activations and everything between two matrix products are in the runtime's
  activation type (float32, or bfloat16 when serving).
* ``ctx`` is the step's :class:`~pretrained_rstr_b200.engine.batch.StepContext`: token
  positions, request of each token, block tables and slots per cache group, state
  slots, scratch memory, and the device status word.
* A part allocates its scratch through ``ctx.scratch(key, shape, dtype)`` so that
  addresses are stable from step to step.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch


@dataclass(frozen=True)
class KVSpec:
    """A mixer that keeps keys and values per token asks for pages of this shape."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None      # None: all keys; w: only the last w


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size per-request state: one tensor ``[slots, *shape]`` per (layer, name)."""
    name: str
    shape: Tuple[int, ...]
    dtype: torch.dtype


@dataclass
class LayerCache:
    """What a block hands to its mixer: the pages of the cache layer it attends over
    (``k``/``v``: [pages, kv_heads, page_size, head_dim]; ``group`` indexes
    ``ctx.groups``), whether this run entry writes them, and its state tensors."""
    group: int = -1
    k: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None
    writes: bool = True
    state: Optional[dict] = None       # name -> tensor [slots, *shape]


class Norm:
    def forward(self, ctx, x: torch.Tensor, out: torch.Tensor, rows=None) -> None:
        """out[r] = norm(x[rows[r]] or x[r]); x float32; statistics in 32-bit."""
        raise NotImplementedError


class Mixer:
    def kv_spec(self) -> Optional[KVSpec]:
        return None

    def state_specs(self) -> List[StateSpec]:
        return []

    def work_planners(self) -> list:
        """Planners (:class:`~pretrained_rstr_b200.engine.batch.WorkPlanner`) of the work lists
        this mixer's kernels want in every step's description; see ``ctx.work``."""
        return []

    def forward(self, ctx, h: torch.Tensor, x: torch.Tensor, cache: LayerCache) -> None:
        """x += mix(h) for the T tokens of the step, reading and (if ``cache.writes``)
        extending the cache."""
        raise NotImplementedError


class FeedForward:
    def work_planners(self) -> list:
        return []

    def forward(self, ctx, h: torch.Tensor, x: torch.Tensor) -> None:
        """x += feed_forward(h)."""
        raise NotImplementedError


class PositionEncoding:
    """Two hooks; an encoding implements the one it needs.
    ``table()`` returns a table the embedding adds per position (learned absolute) or
    None; ``rotate(ctx, q, k)`` changes queries and keys in place before they are
    cached (rotary and the like)."""

    def table(self) -> Optional[torch.Tensor]:
        return None

    def rotate(self, ctx, q: torch.Tensor, k: torch.Tensor) -> None:
        return None


class Embedding:
    def forward(self, ctx, position: PositionEncoding, x: torch.Tensor) -> None:
        """x[t] = table[token[t]] (+ position table row); x float32 [T, width]."""
        raise NotImplementedError


class Head:
    """``accepts_lazy_norm`` (optional, False): the head takes the final norm as a ``LazyNorm``
    (of the wanted rows of the residual stream) and may compute it inside its product."""

    def forward(self, ctx, h: torch.Tensor, logits: torch.Tensor) -> None:
        """logits[r] = h[r] . W^T, float32 [R, vocab]."""
        raise NotImplementedError


class Block:
    """Keeps ``mixer``, ``feed_forward`` and ``norms`` (a dict) as attributes: the assembly
    reads the cache needs of the mixer and the work lists of all of them."""

    def forward(self, ctx, x: torch.Tensor, cache: LayerCache) -> None:
        raise NotImplementedError
