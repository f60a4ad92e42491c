"""The batch of one step as the kernels see it.

The reference already describes a ragged batch at its attention interface: packed
queries with ``row_offsets int32[B+1]`` and ``positions int32[tokens]``, a dense
``page_table`` padded with -1, ``lengths`` and a ``slot_mapping``
(``src/pretrained/continuation/paged_attention.clj:196-205``,
``paged_decoder.clj:562-573``).  The same arrays are used here for the whole step, for
any mix of prompt portions and single decoded tokens.

All integer arrays of a step live in ONE int32 buffer: it is filled on the host in
pinned memory and reaches the device in a single copy.  The offsets inside the buffer
depend only on the capacities (tokens, requests) the layout was made for, so a layout's
device addresses do not change from step to step; unused token rows carry request -1
and slot -1 and are skipped by every kernel that touches the cache.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch


class WorkPlanner:
    """Work lists a part wants in the description of every step.

    The step's description knows requests, tokens, positions and cache slots; how a part's
    kernels cut that into work items (tiles of queries, lists of single tokens, groups of
    tokens per expert, ...) is the part's own business.  A part that needs such lists
    returns planners from ``work_planners()``; the model gathers them (one per ``key``),
    the layout gives their arrays room in the step's one int32 buffer, and
    :func:`fill_host_buffer` lets them write their lists for every step.  Parts find the
    device views in ``ctx.work[key]`` (a :class:`WorkView`).
    """

    #: name under which parts find the lists in ``ctx.work``
    key: str = ""
    #: names of the counters (one int32 each on the device, beside the arrays)
    counters: Tuple[str, ...] = ()

    def arrays(self, t_cap: int, b_cap: int) -> Dict[str, Tuple[int, int]]:
        """array name -> (capacity in int32 words, value of unused entries) for a layout of
        ``t_cap`` tokens and ``b_cap`` requests."""
        raise NotImplementedError

    #: whether ``fill`` also wants the position of every request's first token of the step
    wants_starts: bool = False
    #: counter name -> (step, name of the array the counter counts): in a step that is
    #: replayed from a CUDA graph the kernels of such a list are launched for the host's count
    #: rounded up to a multiple of the step (the rounded count is part of the graph's key)
    #: instead of for the array's capacity
    launch_steps: Dict[str, Tuple[int, str]] = {}

    def absorb(self, other: "WorkPlanner") -> None:
        """Several parts of a model may bring a planner of the same key (one per layer): the
        model keeps the first and lets it absorb the others (what they were told to plan for)."""

    def fill(self, arrays: Dict[str, np.ndarray], lengths: Sequence[int]) -> Dict[str, int]:
        """Write the lists of a step whose requests bring ``lengths[b]`` tokens each (token
        rows are concatenated in request order); returns the counters.  A planner with
        ``wants_starts`` is called as ``fill(arrays, lengths, starts)``: ``starts[b]`` is the
        position of request b's first token of this step.  Under the key "_used" it may name
        the arrays this step needs on the device (the others hold nothing its kernels read,
        as its counters say); arrays that are often unused belong last in ``arrays()``."""
        raise NotImplementedError


@dataclass
class WorkView:
    """One planner's lists as a part sees them in a step."""
    arrays: Dict[str, torch.Tensor]            # device int32 views
    counts: Dict[str, torch.Tensor]            # device views of one int32 each
    caps: Dict[str, int]                       # capacity of every array
    #: the counters as the host knows them; None while a step is replayed from a CUDA graph
    #: (kernels then take the capacity as their grid and the device-side counter as the bound)
    host_counts: Dict[str, Optional[int]]
    #: for counters the planner lists in ``launch_steps``: the launch size of a replayed step
    launch: Dict[str, int] = field(default_factory=dict)
    #: the planner that filled the lists (what it planned for: a part may ask it)
    planner: Optional["WorkPlanner"] = None


@dataclass
class Entry:
    """One request's share of a step: its next tokens and the places (indices into
    ``tokens``) whose logits are wanted."""
    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass(frozen=True)
class Runtime:
    """How a model is instantiated on the device."""
    device: torch.device
    dtype: torch.dtype                 # weights, activations between products, cache
    page_size: int = 64
    max_batched_tokens: int = 2048
    max_requests: int = 64
    use_graphs: bool = True            # replay small steps as CUDA graphs

    @property
    def serving(self) -> bool:
        return self.dtype == torch.bfloat16


class BatchLayout:
    """Offsets (in int32 words) of every array for given capacities."""

    def __init__(self, t_cap: int, b_cap: int, n_groups: int, max_pages: int,
                 planners: Sequence[WorkPlanner] = ()):
        self.t_cap, self.b_cap, self.n_groups, self.max_pages = t_cap, b_cap, n_groups, max_pages
        self.planners = tuple(planners)
        off = 0

        def take(n: int) -> int:
            nonlocal off
            start = off
            off += (n + 3) // 4 * 4          # keep every array 16-byte aligned
            return start

        self.tokens = take(t_cap)
        self.positions = take(t_cap)
        self.seq_of_token = take(t_cap)
        # rows of logits are padded to a power of two, which may exceed the token capacity
        self.row_cap = 1 << max(3, (t_cap - 1).bit_length())
        self.logit_rows = take(self.row_cap)
        self.q_start = take(b_cap + 1)
        self.kv_len = take(b_cap)
        self.state_slot = take(b_cap)
        self.fresh = take(b_cap)
        self.slots = [take(t_cap) for _ in range(n_groups)]
        self.first_pos = [take(b_cap) for _ in range(n_groups)]
        self.block_table = [take(b_cap * max_pages) for _ in range(n_groups)]
        # work lists of the parts that asked for some (see WorkPlanner): counters that live on
        # the device too, then the arrays.  The arrays come last, in the planners' own order,
        # so that a step which leaves the last ones unused need not copy them to the device
        # (fill_host_buffer says how many words a step uses): a copy of up to a kilobyte,
        # which a small decode step fits, measured 7 microseconds faster than a larger one.
        n_counters = sum(len(p.counters) for p in self.planners)
        self.counts = take(2 + n_counters)    # [tokens, requests, planners' counters ...]
        self.work_arrays: Dict[str, Dict[str, Tuple[int, int, int]]] = {}   # key -> name -> (offset, words, fill)
        for planner in self.planners:
            self.work_arrays[planner.key] = {
                name: (take(words), words, fill)
                for name, (words, fill) in planner.arrays(t_cap, b_cap).items()}
        self.work_counts: Dict[str, Dict[str, int]] = {}
        at = self.counts + 2
        for planner in self.planners:
            self.work_counts[planner.key] = {}
            for name in planner.counters:
                self.work_counts[planner.key][name] = at
                at += 1
        self.size = off
        self._views = None
        self._work_views = None

    def device_views(self, buf: torch.Tensor):
        if self._views is None:
            lay = self
            self._views = (
                buf[lay.tokens:lay.tokens + lay.t_cap],
                buf[lay.positions:lay.positions + lay.t_cap],
                buf[lay.seq_of_token:lay.seq_of_token + lay.t_cap],
                buf[lay.logit_rows:lay.logit_rows + lay.row_cap],
                buf[lay.q_start:lay.q_start + lay.b_cap + 1],
                buf[lay.kv_len:lay.kv_len + lay.b_cap],
                buf[lay.state_slot:lay.state_slot + lay.b_cap],
                buf[lay.fresh:lay.fresh + lay.b_cap],
                buf[lay.counts:lay.counts + 2])
        return self._views

    def work_views(self, buf: torch.Tensor):
        """Per planner: (array views, counter views, capacities), made once per layout."""
        if self._work_views is None:
            out = {}
            for key, arrays in self.work_arrays.items():
                out[key] = ({name: buf[off:off + words] for name, (off, words, _f) in arrays.items()},
                            {name: buf[off:off + 1] for name, off in self.work_counts[key].items()},
                            {name: words for name, (_o, words, _f) in arrays.items()})
            self._work_views = out
        return self._work_views


@dataclass
class GroupView:
    """A cache group's arrays for this step (device int32 views)."""
    slots: torch.Tensor            # [t_cap]   slot of each new token, -1 = none
    block_table: torch.Tensor      # [b_cap, max_pages], -1 = no page
    first_pos: torch.Tensor        # [b_cap]   lowest position still held (windows)
    window: Optional[int]
    page_size: int
    num_pages: int


@dataclass
class HostBatch:
    """The same step in plain Python, for parts written with array-library calls
    (tests' toy parts) and for the engine's own book-keeping."""
    rids: List[Hashable]
    q_start: List[int]             # B+1 offsets into the token rows
    start_pos: List[int]           # position of each request's first token in this step
    state_slot: List[int]
    fresh: List[bool]
    tokens: List[int]


class StepContext:
    """Everything a part may ask about the step."""

    def __init__(self, runtime: Runtime, layout: BatchLayout, device_buf: torch.Tensor,
                 n_tokens: int, n_requests: int, n_rows: int, host: HostBatch,
                 groups: List[GroupView], status: torch.Tensor, scratch_pool: "ScratchPool",
                 max_context: int, max_q_len: int, launch_tokens: int, launch_rows: int,
                 max_positions: int = 0):
        self.runtime = runtime
        self.layout = layout
        self.n_tokens = n_tokens            # real tokens of the step
        self.n_requests = n_requests
        self.n_rows = n_rows                # logits rows wanted
        self.launch_tokens = launch_tokens  # rows the kernels run (>= n_tokens when padded)
        self.launch_rows = launch_rows      # logits rows computed (>= n_rows when padded)
        self.host = host
        self.groups = groups
        self.status = status
        self.max_context = max_context      # upper bound of any request's length after the step
        self.max_q_len = max_q_len
        self.max_positions = max_positions or max_context
        self._scratch = scratch_pool
        # device views of the step's arrays: made once per layout, their addresses never change
        views = layout.device_views(device_buf)
        (self.tokens, self.positions, self.seq_of_token, self.logit_rows, self.q_start,
         self.kv_len, self.state_slot, self.fresh, self.counts) = views
        # the parts' own work lists; the host-side counters are filled in by the runner
        by_key = {planner.key: planner for planner in layout.planners}
        self.work: Dict[str, WorkView] = {
            key: WorkView(arrays, counts, caps, {name: None for name in counts},
                          planner=by_key.get(key))
            for key, (arrays, counts, caps) in layout.work_views(device_buf).items()}
        self.feedback = False               # token ids below zero name tokens chosen last
        self.used_words: Optional[int] = None      # words of the step's buffer that go to the device

    @property
    def dtype(self) -> torch.dtype:
        return self.runtime.dtype

    @property
    def token_capacity(self) -> int:
        """Rows to give scratch tensors that hold one row per token."""
        return self.runtime.max_batched_tokens

    @staticmethod
    def row_capacity(rows: int) -> int:
        """Rows to give scratch tensors that hold one row per wanted logits row."""
        cap = 8
        while cap < rows:
            cap *= 2
        return cap

    def scratch(self, key: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        """Scratch memory with a stable address for (key, shape, dtype).  Contents do not
        survive the step; two parts that use the same key share the memory."""
        return self._scratch.get(key, shape, dtype)

    def scratch_zero(self, key: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        """Scratch that is zero when first handed out; whoever uses it leaves it zero
        (counters that their kernel resets)."""
        return self._scratch.get(key, shape, dtype, zero=True)


class ScratchPool:
    def __init__(self, device: torch.device):
        self.device = device
        self._bufs: Dict[Tuple, torch.Tensor] = {}

    def get(self, key: str, shape: Tuple[int, ...], dtype: torch.dtype,
            zero: bool = False) -> torch.Tensor:
        k = (key, tuple(shape), dtype)
        buf = self._bufs.get(k)
        if buf is None:
            make = torch.zeros if zero else torch.empty
            buf = make(tuple(shape), dtype=dtype, device=self.device)
            self._bufs[k] = buf
        return buf

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._bufs.values())


_IOTA = np.arange(64, dtype=np.int32)


def _iota(n: int) -> np.ndarray:
    global _IOTA
    if n > len(_IOTA):
        _IOTA = np.arange(max(n, 2 * len(_IOTA)), dtype=np.int32)
    return _IOTA[:n]


def fill_host_buffer(host_np: np.ndarray, layout: BatchLayout, entries_tokens: List[List[int]],
                     start_pos: List[int], state_slots: List[int], fresh: List[bool],
                     group_slots: List[List[List[int]]], group_tables: List,
                     group_first: List[List[int]], logit_rows: List[int]) -> Dict[str, Dict[str, int]]:
    """Write one step into the pinned host buffer (``group_tables[g]``: the block tables of
    the requests, as lists of pages or as an array of rows padded with -1).  Returns the
    counters of the parts' work lists, by planner key and counter name, and under "_words"
    how many words of the buffer the step uses (what lies beyond need not be copied to the
    device)."""
    lay = layout
    n_req = len(entries_tokens)
    t = 0
    tok = host_np[lay.tokens:lay.tokens + lay.t_cap]
    pos = host_np[lay.positions:lay.positions + lay.t_cap]
    seq = host_np[lay.seq_of_token:lay.seq_of_token + lay.t_cap]
    rows = host_np[lay.logit_rows:lay.logit_rows + lay.row_cap]
    qs = host_np[lay.q_start:lay.q_start + lay.b_cap + 1]
    kv = host_np[lay.kv_len:lay.kv_len + lay.b_cap]
    ss = host_np[lay.state_slot:lay.state_slot + lay.b_cap]
    fr = host_np[lay.fresh:lay.fresh + lay.b_cap]
    if all(len(toks) == 1 for toks in entries_tokens):
        # every request brings one token (a decode step): whole arrays at once
        n_tok = n_req
        iota = _iota(n_req)
        tok[:n_req] = [toks[0] for toks in entries_tokens]
        pos[:n_req] = start_pos
        seq[:n_req] = iota
        qs[:n_req] = iota
        np.add(pos[:n_req], 1, out=kv[:n_req])
        ss[:n_req] = state_slots
        fr[:n_req] = fresh
    else:
        for b, toks in enumerate(entries_tokens):
            n = len(toks)
            tok[t:t + n] = toks
            pos[t:t + n] = np.arange(start_pos[b], start_pos[b] + n, dtype=np.int32)
            seq[t:t + n] = b
            qs[b] = t
            kv[b] = start_pos[b] + n
            ss[b] = state_slots[b]
            fr[b] = 1 if fresh[b] else 0
            t += n
        n_tok = t
    tok[n_tok:] = 0
    pos[n_tok:] = 0
    seq[n_tok:] = -1
    qs[n_req:] = n_tok
    kv[n_req:] = 0
    ss[n_req:] = 0
    fr[n_req:] = 0
    rows[:len(logit_rows)] = logit_rows
    rows[len(logit_rows):] = 0
    for g in range(lay.n_groups):
        sl = host_np[lay.slots[g]:lay.slots[g] + lay.t_cap]
        if n_tok == n_req:
            sl[:n_req] = [s[0] for s in group_slots[g]]
        else:
            t = 0
            for b in range(n_req):
                n = len(group_slots[g][b])
                sl[t:t + n] = group_slots[g][b]
                t += n
        sl[n_tok:] = -1
        fp = host_np[lay.first_pos[g]:lay.first_pos[g] + lay.b_cap]
        fp[:n_req] = group_first[g]
        fp[n_req:] = 0
        bt2 = host_np[lay.block_table[g]:lay.block_table[g] + lay.b_cap * lay.max_pages] \
            .reshape(lay.b_cap, lay.max_pages)
        tables = group_tables[g]
        if isinstance(tables, np.ndarray):          # rows in their device form already
            bt2[:n_req, :tables.shape[1]] = tables
            bt2[:n_req, tables.shape[1]:] = -1
            bt2[n_req:] = -1
        else:
            bt2[:] = -1
            for b in range(n_req):
                table = tables[b]
                bt2[b, :len(table)] = table
    # the parts' work lists
    lengths = [len(toks) for toks in entries_tokens]
    counts: Dict[str, Dict[str, int]] = {}
    n_counters = sum(len(p.counters) for p in lay.planners)
    used_words = lay.counts + (2 + n_counters + 3) // 4 * 4       # everything up to the counters
    at = lay.counts + 2
    for planner in lay.planners:
        views = {}
        for name, (off, words, fill) in lay.work_arrays[planner.key].items():
            views[name] = host_np[off:off + words]
            views[name][:] = fill              # entries the planner leaves unused
        got = planner.fill(views, lengths, list(start_pos)) if planner.wants_starts \
            else planner.fill(views, lengths)
        counts[planner.key] = {name: int(got[name]) for name in planner.counters}
        # (arrays the planner did not write hold nothing a kernel reads: its counters say so)
        for name in got.get("_used", views.keys()):
            off, words, _fill = lay.work_arrays[planner.key][name]
            used_words = max(used_words, off + words)
        for name in planner.counters:
            host_np[at] = counts[planner.key][name]
            at += 1
    host_np[lay.counts:lay.counts + 2] = (n_tok, n_req)
    counts["_words"] = used_words
    return counts
