"""The step function.

``ModelRunner.step(entries)`` takes a batch of (request, its next tokens, wanted
places): portions of prompts beside single decoded tokens, cut anywhere.  It runs only
the tokens it is given, as one batch, from the cache earlier steps left, and returns the
logits at the wanted places.  It is the reference's ``step-lanes!`` and
``prefill-range!`` (``src/pretrained/continuation/paged_decoder.clj:512-583, 638-711``)
made one: reserve slots -> describe the batch -> run -> commit, and abort the
reservation if anything fails (``:580-583``).
"""
from __future__ import annotations

from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..cache.storage import CacheStorage
from ..csrc import ops
from ..settings import SETTINGS
from .batch import (BatchLayout, Entry, GroupView, HostBatch, Runtime, ScratchPool, StepContext,
                    fill_host_buffer)


class StepError(RuntimeError):
    pass


# A step whose description is at most this long is read from the pinned buffer by a kernel;
# a longer one (a large portion of a prompt) goes through the copy engine, whose bandwidth
# then counts for more than the hand-over it costs.
FETCH_BY_KERNEL_WORDS = 4096


def _bucket(n: int, floor: int, cap: int) -> int:
    """Capacity a count is rounded up to: powers of two up to 64, multiples of 64 up to 512,
    multiples of 256 beyond (few shapes, little padding)."""
    if n <= 64:
        b = floor
        while b < n:
            b *= 2
    elif n <= 512:
        b = -(-n // 64) * 64
    else:
        b = -(-n // 256) * 256
    return min(b, cap) if cap >= n else n


class ModelRunner:
    def __init__(self, model, runtime: Runtime, cache: CacheManager, storage: CacheStorage):
        self.model, self.runtime, self.cache, self.storage = model, runtime, cache, storage
        self.device = runtime.device
        model.attach_storage(storage)
        self.n_groups = len(cache.groups)
        self.max_pages = cache.max_pages_per_request
        self._layouts: Dict[tuple, BatchLayout] = {}
        self._group_views: Dict[int, list] = {}
        self.planners = tuple(getattr(model, "planners", ()))
        biggest = BatchLayout(runtime.max_batched_tokens, runtime.max_requests, self.n_groups,
                              self.max_pages, self.planners)
        # two pinned staging buffers, used in turn, each guarded by an event
        self._hosts = [torch.empty(biggest.size, dtype=torch.int32, pin_memory=True)
                       for _ in range(2)]
        self._host_events = [torch.cuda.Event() for _ in range(2)]
        self._host_turn = 0
        self._dev = torch.zeros(biggest.size, dtype=torch.int32, device=self.device)
        # sampled tokens and the device status word share one buffer, so that one copy
        # brings both to the host
        self.result = torch.zeros(runtime.max_requests + 4, dtype=torch.int32, device=self.device)
        self.result_host = torch.zeros(runtime.max_requests + 4, dtype=torch.int32,
                                       pin_memory=True)
        # two host copies take turns, so that a step's tokens can be read while the next
        # step's copy is already queued
        self._result_hosts = [self.result_host,
                              torch.zeros_like(self.result_host).pin_memory()]
        self._result_events = [torch.cuda.Event(), torch.cuda.Event()]
        self._result_turn = 0
        # Small steps cross the bus inside kernels that read and write the pinned buffers
        # directly (no hand-over between copy engine and kernels on the stream); 0 where
        # kernels cannot reach a buffer, and then the copy engine moves it.
        by_kernel = SETTINGS.step_words_by_kernel
        self._host_addresses = [ops.host_device_address(h) if by_kernel else 0
                                for h in self._hosts]
        self._result_addresses = [ops.host_device_address(h) if by_kernel else 0
                                  for h in self._result_hosts]
        self.tokens_out = self.result[:runtime.max_requests]
        self.status = self.result[runtime.max_requests:]
        self._status_host = torch.zeros(4, dtype=torch.int32, pin_memory=True)
        # CUDA graphs of whole steps, by (token capacity, request capacity, logits rows)
        self.use_graphs = bool(runtime.use_graphs) and getattr(model, "graph_safe", False)
        self.graph_max_tokens = runtime.max_batched_tokens
        self._graphs: Dict[tuple, tuple] = {}
        self._seen: Dict[tuple, int] = {}
        self._pairs_host = torch.empty((runtime.max_requests, 2), dtype=torch.int32,
                                       pin_memory=True)
        self._pairs_dev = torch.zeros((runtime.max_requests, 2), dtype=torch.int32,
                                      device=self.device)
        self.scratch = ScratchPool(self.device)
        self.fail_next_step: Optional[Exception] = None      # host-side fault injection (tests)
        self.counters = {"steps": 0, "launched": 0, "tokens": 0, "cow_copies": 0}
        self.last_h2d_bytes = 0
        self.start_event = None                       # optional CUDA event recorded before the copy

    # ------------------------------------------------------------------ layout
    def layout_for(self, n_tokens: int, n_requests: int) -> BatchLayout:
        key = (_bucket(n_tokens, 8, self.runtime.max_batched_tokens),
               _bucket(n_requests, 1, self.runtime.max_requests))
        lay = self._layouts.get(key)
        if lay is None:
            lay = BatchLayout(key[0], key[1], self.n_groups, self.max_pages, self.planners)
            self._layouts[key] = lay
        return lay

    # -------------------------------------------------------------------- step
    def step(self, entries: Sequence[Entry]) -> torch.Tensor:
        """Run one batch; returns float32 logits ``[wanted, vocab]`` in the order of the
        entries and of each entry's ``want`` (a view of scratch memory, valid until the
        next step).  New requests must have been opened in the cache manager."""
        return self.launch(self.prepare(entries), entries)

    def launch(self, ctx: StepContext, entries: Sequence[Entry]) -> torch.Tensor:
        """Second half of a step: copy the prepared arrays to the device, run, commit.
        Token ids below zero name places among the tokens chosen last (``prepare`` with
        ``feedback``); they are put in on the device before the model runs."""
        try:
            if self.fail_next_step is not None:
                exc, self.fail_next_step = self.fail_next_step, None
                raise exc
            self.upload(ctx)
            logits = self._run(ctx)
        except Exception:
            self.abort(entries)
            raise
        self.commit(entries)
        self.counters["launched"] += 1
        return logits[:ctx.n_rows]

    def patch_tokens(self, ctx: StepContext, entries: Sequence[Entry]) -> None:
        """Put the real token ids into a step that was prepared ahead of time with
        placeholders (same requests, same token counts)."""
        lay = ctx.layout
        flat = [int(t) for e in entries for t in e.tokens]
        if len(flat) != ctx.n_tokens:
            raise StepError("patch_tokens: token count differs from the prepared step")
        vocab = self.model.vocab
        if flat and (min(flat) < 0 or max(flat) >= vocab):
            raise StepError(f"token id outside the vocabulary of {vocab}")
        ctx.staging.numpy()[lay.tokens:lay.tokens + len(flat)] = flat
        ctx.host.tokens = flat
        ctx.feedback = False

    def _run(self, ctx: StepContext) -> torch.Tensor:
        """Run the model for a prepared step: directly, or, for small steps when graphs are
        on, as a CUDA graph of the whole step.  A graph is captured for fixed capacities
        (tokens, requests, logits rows, longest context); rows beyond the real ones are padding that no
        kernel lets touch the cache.  The first step of a shape runs directly with the
        padded sizes (which also sizes all scratch memory), the second is captured."""
        lay = ctx.layout
        # which of the parts' work lists hold something: a step without prompt tiles (or
        # without single tokens) gets a graph without the kernels of that list, since an idle
        # launch per layer is a tenth of a small decode step
        filled = tuple(bool(c) for view in ctx.work.values() for c in view.host_counts.values())
        if not self.use_graphs or lay.t_cap > self.graph_max_tokens:
            return self.model.forward(ctx)
        rows_cap = StepContext.row_capacity(max(ctx.n_rows, 1)) if ctx.n_rows else 0
        # the longest context the graph is planned for: the step's own bound rounded up to
        # 256, 512, 1,024, ... (the attention kernels choose their splits, and which of them
        # runs, by it; a graph for every length would be captured all the time)
        reach = 256
        while reach < ctx.max_context:
            reach *= 2
        reach = min(reach, self.model.max_positions)
        # lists whose kernels are launched for a rounded count rather than their capacity
        bounds = []
        for planner in self.planners:
            view = ctx.work[planner.key]
            for name, (step, array) in planner.launch_steps.items():
                count = view.host_counts.get(name) or 0
                view.launch[name] = min(view.caps[array], -(-count // step) * step)
                bounds.append(view.launch[name])
        key = (lay.t_cap, lay.b_cap, rows_cap, filled, reach, tuple(bounds))
        ctx.launch_tokens, ctx.launch_rows = lay.t_cap, rows_cap
        self._counts_from_device(ctx)
        ctx.max_context = reach
        hit = self._graphs.get(key)
        if hit is not None:
            hit[0].replay()
            ops.add_launches(hit[2])
            return hit[1]
        seen = self._seen.get(key, 0)
        self._seen[key] = seen + 1
        if seen == 0:
            return self.model.forward(ctx)
        graph = torch.cuda.CUDAGraph()
        before = ops.launch_count()
        with torch.cuda.graph(graph):
            logits = self.model.forward(ctx)
        kernels = ops.launch_count() - before      # recorded, not run: counted at each replay
        ops.add_launches(-kernels)
        self._graphs[key] = (graph, logits, kernels)
        graph.replay()
        ops.add_launches(kernels)
        return logits

    @staticmethod
    def _counts_from_device(ctx: StepContext) -> None:
        """For a step that is recorded or replayed: a work list that holds something is run
        at its capacity with the device-side counter as the bound (None), an empty one not
        at all (0)."""
        for view in ctx.work.values():
            view.host_counts = {name: (None if c else 0) for name, c in view.host_counts.items()}

    def prepare(self, entries: Sequence[Entry], feedback: bool = False) -> StepContext:
        """First half of a step: validate the batch, reserve cache slots, and describe the
        step in pinned host memory (nothing touches the device yet).  With ``feedback`` a
        token id -(k + 1) is allowed: the k-th token the sampling kernel chose last."""
        if not entries:
            raise StepError("a step needs at least one entry")
        rids = [e.rid for e in entries]
        if len(set(rids)) != len(rids):
            raise StepError("a request appears twice in one step")
        if len(entries) > self.runtime.max_requests:
            raise StepError(f"{len(entries)} requests in one step; the runtime takes "
                            f"{self.runtime.max_requests}")
        total = sum(len(e.tokens) for e in entries)
        if total > self.runtime.max_batched_tokens:
            raise StepError(f"{total} tokens in one step; the runtime takes "
                            f"{self.runtime.max_batched_tokens}")
        vocab = self.model.vocab
        lowest = -self.runtime.max_requests if feedback else 0
        for e in entries:
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.rid!r}: no tokens in this step")
            for w in e.want:
                if not 0 <= w < n:
                    raise StepError(f"request {e.rid!r}: wanted place {w} outside its "
                                    f"{n} tokens")
            if n == 1:
                t = e.tokens[0]
                fine = isinstance(t, (int, np.integer)) and lowest <= t < vocab
            else:
                toks = np.asarray(e.tokens)
                fine = toks.dtype.kind in "iu" and int(toks.min()) >= lowest and \
                    int(toks.max()) < vocab
            if not fine:
                bad = [t for t in e.tokens if not (isinstance(t, (int, np.integer)) and 0 <= t < vocab)]
                raise StepError(f"request {e.rid!r}: token id {bad[0] if bad else '?'} outside the "
                                f"vocabulary of {vocab}")
            held = self.cache.length(e.rid)
            if held + n > self.model.max_positions:
                raise StepError(f"request {e.rid!r}: {held}+{n} "
                                f"tokens exceed the model's {self.model.max_positions} positions")
        reserved: List[Hashable] = []
        try:
            reservations = []
            for e in entries:
                reservations.append(self.cache.reserve(e.rid, len(e.tokens)))
                reserved.append(e.rid)
        except Exception:
            for rid in reserved:
                self.cache.abort(rid)
            raise
        try:
            ctx = self._describe(entries, reservations)
        except Exception:
            self.abort(entries)
            raise
        ctx.feedback = feedback and any(t < 0 for e in entries for t in e.tokens)
        return ctx

    def _describe(self, entries, reservations) -> StepContext:
        n_req = len(entries)
        total = sum(len(e.tokens) for e in entries)
        layout = self.layout_for(total, n_req)
        start_pos = [r.start for r in reservations]
        records = [self.cache.peek(e.rid) for e in entries]
        state_slots = [r.slot for r in records]
        fresh = [r.fresh for r in records]
        group_slots = [[r.slots[g] for r in reservations] for g in range(self.n_groups)]
        # block tables: the manager keeps them in their device form, one row per state slot
        group_tables = [rows[state_slots] for rows in self.cache.table_rows]
        group_first = [[0] * n_req if spec.window is None else
                       [self.cache.first_visible(e.rid, g) for e in entries]
                       for g, spec in enumerate(self.cache.groups)]
        logit_rows: List[int] = []
        q_start = [0]
        for e in entries:
            at = q_start[-1]
            for w in e.want:
                logit_rows.append(at + w)
            q_start.append(at + len(e.tokens))
        turn = self._host_turn
        self._host_turn ^= 1
        self._host_events[turn].synchronize()        # the copy that last used this buffer is done
        staging = self._hosts[turn]
        work_counts = fill_host_buffer(staging.numpy(), layout, [list(e.tokens) for e in entries],
                                       start_pos, state_slots, fresh, group_slots, group_tables,
                                       group_first, logit_rows)
        groups = self._group_views.get(id(layout))
        if groups is None:
            groups = []
            for g, spec in enumerate(self.cache.groups):
                lay = layout
                groups.append(GroupView(
                    slots=self._dev[lay.slots[g]:lay.slots[g] + lay.t_cap],
                    block_table=self._dev[lay.block_table[g]:lay.block_table[g]
                                          + lay.b_cap * lay.max_pages].view(lay.b_cap, lay.max_pages),
                    first_pos=self._dev[lay.first_pos[g]:lay.first_pos[g] + lay.b_cap],
                    window=spec.window, page_size=self.cache.page_size,
                    num_pages=self.cache.allocators[g].num_pages))
            self._group_views[id(layout)] = groups
        host = HostBatch(rids=[e.rid for e in entries], q_start=q_start, start_pos=start_pos,
                         state_slot=state_slots, fresh=fresh,
                         tokens=[t for e in entries for t in e.tokens])
        max_len = max(s + len(e.tokens) for s, e in zip(start_pos, entries))
        max_context = min(self.model.max_positions, -(-max_len // 256) * 256)
        max_q = max(len(e.tokens) for e in entries)
        self.counters["steps"] += 1
        self.counters["tokens"] += total
        ctx = StepContext(self.runtime, layout, self._dev, total, n_req, len(logit_rows), host,
                          groups, self.status, self.scratch, max_context, max_q,
                          launch_tokens=total, launch_rows=len(logit_rows),
                          max_positions=self.model.max_positions)
        ctx.used_words = work_counts.pop("_words", None)
        for key, counts in work_counts.items():
            ctx.work[key].host_counts = dict(counts)
        ctx.staging, ctx.staging_turn = staging, turn
        ctx.copies = [c for r in reservations for c in r.copies]
        return ctx

    def upload(self, ctx: StepContext) -> None:
        """The step's arrays go to the device in one piece (a kernel that reads the pinned
        buffer for a small step, one copy for a large one), token ids that name places among
        the tokens chosen last are put in, and copy-on-write page copies come before anything
        reads or writes the new pages."""
        layout = ctx.layout
        if self.start_event is not None:             # measurement: device work of the step begins
            self.start_event.record()
        words = ctx.used_words or layout.size
        address = self._host_addresses[ctx.staging_turn]
        if address and words <= FETCH_BY_KERNEL_WORDS:
            ops.fetch_step(self._dev, address, words, layout.tokens, ctx.n_tokens,
                           self.tokens_out if ctx.feedback else None, self.status)
        else:
            self._dev[:words].copy_(ctx.staging[:words], non_blocking=True)
            if ctx.feedback:
                ops.resolve_tokens(ctx.tokens, ctx.n_tokens, self.tokens_out, self.status)
        self._host_events[ctx.staging_turn].record()
        self.last_h2d_bytes = words * 4
        for g in range(self.n_groups):
            pairs = [(src, dst) for (gg, src, dst) in ctx.copies if gg == g]
            for i in range(0, len(pairs), self._pairs_host.shape[0]):
                chunk = pairs[i:i + self._pairs_host.shape[0]]
                self._pairs_host[:len(chunk)] = torch.tensor(chunk, dtype=torch.int32)
                self._pairs_dev[:len(chunk)].copy_(self._pairs_host[:len(chunk)], non_blocking=True)
                self.storage.copy_pages(g, self._pairs_dev, len(chunk), self.status)
                torch.cuda.current_stream().synchronize()      # pinned pairs buffer is reused
                self.counters["cow_copies"] += len(chunk)

    def commit(self, entries: Sequence[Entry]) -> None:
        for e in entries:
            # ids that are not known on the host yet are not recorded (such pages are not
            # offered for sharing)
            known = min(e.tokens) >= 0
            self.cache.commit(e.rid, list(e.tokens) if known else None)

    def abort(self, entries: Sequence[Entry]) -> None:
        for e in entries:
            self.cache.abort(e.rid)

    # ------------------------------------------------------------------ status
    def fetch_result(self) -> torch.Tensor:
        """One device-to-host copy of the sampled tokens and the status word
        (synchronises); raises if a kernel recorded an index out of range."""
        return self.wait_result(self.queue_result())

    def queue_result(self) -> int:
        """Queue the copy of the sampled tokens and the status word to the host behind the
        work launched so far; returns a ticket for :meth:`wait_result`.  Work launched
        afterwards does not delay the ticket."""
        turn, _address = self.begin_result()
        return self.end_result(turn, published=False)

    def begin_result(self):
        """The host buffer the next result goes to: (ticket, address under which kernels
        reach it, or 0).  A kernel that is the last of its step may write ``self.result``
        there itself (``ops.sample(..., publish=...)``); :meth:`end_result` follows."""
        turn = self._result_turn
        self._result_turn ^= 1
        return turn, self._result_addresses[turn]

    def end_result(self, turn: int, published: bool) -> int:
        """Second half of :meth:`queue_result`: bring the result to the host unless the
        step's last kernel has done so, and mark the place in the stream."""
        if not published:
            if self._result_addresses[turn]:
                ops.publish_result(self._result_addresses[turn], self.result, self.result.numel())
            else:
                self._result_hosts[turn].copy_(self.result, non_blocking=True)
        self._result_events[turn].record()
        return turn

    def wait_result(self, ticket: int) -> torch.Tensor:
        """Wait for a queued copy; raises if a kernel had recorded an index out of range."""
        self._result_events[ticket].synchronize()
        host = self._result_hosts[ticket]
        n = self.runtime.max_requests
        code = int(host[n])
        if code != 0:
            detail = [int(v) for v in host[n + 1:]]
            torch.cuda.current_stream().synchronize()
            self.status.zero_()
            raise StepError(f"device status {code}: {ops.STATUS_TEXT.get(code, 'unknown')} "
                            f"{detail}")
        return host

    def check_status(self) -> None:
        """Read the device status word (synchronises); raises if a kernel recorded an
        index out of range.  The word is cleared afterwards."""
        self._status_host.copy_(self.status, non_blocking=False)
        code = int(self._status_host[0])
        if code != 0:
            detail = [int(v) for v in self._status_host[1:]]
            self.status.zero_()
            raise StepError(f"device status {code}: {ops.STATUS_TEXT.get(code, 'unknown')} "
                            f"{detail}")
