"""The generation engine: scheduler above the step function, sampling below it.

One iteration (the reference's ``execute-lanes!``,
``src/pretrained/continuation/paged_runtime.clj:214-286``): plan the iteration, build
the batch from the plan, run one step, choose a token for every request that asked for
logits, report the tokens to the scheduler, which advances, finishes and frees.
Only token ids cross the host/device boundary: ids in, one int32 per sampled row out
(``paged_decoder.clj:562-579``).
"""
from __future__ import annotations

from typing import Callable, Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..csrc import ops
from .batch import Entry
from .loading import LoadedModel
from ..sampling import Sampler, SamplingParams
from .scheduler import Plan, Request, Scheduled, Scheduler, SchedulerOptions


class Engine:
    def __init__(self, lm: LoadedModel, opts: Optional[SchedulerOptions] = None):
        self.lm = lm
        rt = lm.runtime
        self.opts = opts or SchedulerOptions(max_batched_tokens=rt.max_batched_tokens,
                                             max_lanes=rt.max_requests)
        if self.opts.max_batched_tokens > rt.max_batched_tokens or \
                self.opts.max_lanes > rt.max_requests:
            raise ValueError("scheduler capacities exceed what the runtime was loaded with")
        self.scheduler = Scheduler(self.opts, lm.cache)
        self.runner = lm.runner
        # per-request sampler state lives in the request's state slot
        self.sampler = Sampler(rt.max_requests, rt.device, lm.cache.slot)
        self._tokens_dev = self.runner.tokens_out
        # optional (start events, end events) lists: step ``step_index`` records its pair
        # around the device work of the step (measurement only)
        self.timing_events = None
        self.step_index = 0
        self.launched_entries = None       # the entries of the step launched last
        self._prepared = None              # (entries, context, requests) of a step described ahead
        self._flight = None                # (plan, entries, samplers, ticket) of a launched step
        self.ahead = {"used": 0, "dropped": 0, "dead_rows": 0}

    # ------------------------------------------------------------------ requests
    def submit(self, rid: Hashable, prompt: Sequence[int], max_new_tokens: int,
               sampling: Optional[SamplingParams] = None, eos_ids: Sequence[int] = (),
               on_token: Optional[Callable[[Hashable, int], None]] = None) -> Request:
        sampling = sampling or SamplingParams()
        sampling.validate(self.lm.model.vocab, self.sampler.max_top_k)
        vocab = self.lm.model.vocab
        ids = np.asarray(prompt)
        if ids.ndim != 1 or (ids.size and ids.dtype.kind not in "iu"):
            ids = np.asarray([int(t) for t in prompt], dtype=np.int64)      # (raises on what is no integer)
        if ids.size and (int(ids.min()) < 0 or int(ids.max()) >= vocab):
            bad = next(int(t) for t in ids if not 0 <= int(t) < vocab)
            raise ValueError(f"prompt token id {bad} outside the vocabulary of {vocab}")
        req = Request(rid=rid, prompt=ids.tolist(), max_new_tokens=int(max_new_tokens),
                      sampling=sampling, eos_ids=tuple(int(e) for e in eos_ids), on_token=on_token)
        self.scheduler.submit(req)
        return req

    def cancel(self, rid: Hashable) -> None:
        self.scheduler.cancel(rid)

    # ---------------------------------------------------------------------- step
    def step(self, ahead: bool = False) -> List[Request]:
        """One iteration; returns the requests that finished.

        While the GPU runs a step, the host already describes the next one (who decodes at
        which position into which slot) on the assumption that nobody stops on a stop token
        and nobody new arrives.  ``ahead=False``: the call waits for its step's tokens, and
        the described step only needs its token ids patched in.  ``ahead=True``: the
        described step is launched at the start of the next call, before the tokens of the
        step in flight have reached the host (it names them by place and the device puts
        them in); the call then returns what finished in the step launched by the call
        before, so the host runs one step behind the GPU (:meth:`flush` catches up).  A
        request that stops on a stop token has by then one token too many in flight: its
        row is dropped, its pages are freed when it ends."""
        flight, prepared = self._flight, self._prepared
        self._flight = self._prepared = None
        launched = None
        if flight is not None and prepared is not None and self._still_steady(prepared[0]):
            entries, ctx, samplers = prepared
            launched = self._launch(Plan(tuple(Scheduled(e.rid, "decode", 1) for e in entries),
                                         (), 0, 0), entries, ctx, samplers)
            self.scheduler.stats["iterations"] += 1
            self.scheduler.stats["scheduled_tokens"] += len(entries)
            self.ahead["used"] += 1
            prepared = None
        done = self._finish(flight) if flight is not None else []
        if launched is None:
            plan = self.scheduler.next_plan()
            if not plan.scheduled:
                self._drop(prepared)
                return done
            entries: List[Entry] = []
            samplers: List[Request] = []
            for item in plan.scheduled:
                tokens = self.scheduler.step_tokens(item)
                wants = self.scheduler.wants_logits(item)
                entries.append(Entry(item.rid, tokens, [len(tokens) - 1] if wants else []))
                if wants:
                    samplers.append(self.scheduler.running[item.rid])
            ctx = self._take_prepared(prepared, entries)
            if ctx is None:
                ctx = self.runner.prepare(entries)
            launched = self._launch(plan, entries, ctx, samplers)
        self._prepared = self._prepare_ahead(launched)     # overlaps the GPU's work
        if ahead:
            self._flight = launched
            return done
        return done + self._finish(launched)

    def flush(self) -> List[Request]:
        """Catch up with the GPU: wait for the step in flight (``step(ahead=True)``) and
        return the requests that finished in it."""
        flight, self._flight = self._flight, None
        done = self._finish(flight) if flight is not None else []
        return done

    # ------------------------------------------------------------- launch and finish
    def _launch(self, plan: Plan, entries: List[Entry], ctx, samplers: List[Request]):
        if self.timing_events is not None:
            self.runner.start_event = self.timing_events[0][self.step_index]
        self.launched_entries = entries
        logits = self.runner.launch(ctx, entries)
        self.runner.start_event = None
        ticket = None
        if samplers:
            # the kernel that chooses the tokens is the step's last: it also writes them, and
            # the status word, to the pinned buffer the host will read
            turn, address = self.runner.begin_result()
            publish = (address, self.runner.result, self.runner.result.numel()) if address else None
            self.sampler.launch(self._tokens_dev, logits, samplers, publish=publish)
        if self.timing_events is not None:             # the step's device work ends here
            self.timing_events[1][self.step_index].record()
        if samplers:
            ticket = self.runner.end_result(turn, published=publish is not None)
        return (plan, entries, samplers, ticket)

    def _finish(self, flight) -> List[Request]:
        """Wait for a launched step's tokens and report them to the scheduler."""
        plan, _entries, samplers, ticket = flight
        new_tokens: Dict[Hashable, int] = {}
        if ticket is not None:
            chosen = self.runner.wait_result(ticket)[:len(samplers)].tolist()
            new_tokens = {r.rid: t for r, t in zip(samplers, chosen)}
            self.ahead["dead_rows"] += sum(1 for r in samplers if r.rid not in self.scheduler.running)
        done = self.scheduler.complete(plan, new_tokens)
        for r in done:
            self.sampler.forget(r.rid)
        return done

    # ------------------------------------------------------------- preparing ahead
    def _prepare_ahead(self, launched):
        """Describe the step after ``launched`` before its tokens are known.  Only in the
        steady state: nothing waiting or deferred, and every scheduled request will be
        decoding.  Token ids are given by place among the tokens ``launched`` chooses."""
        plan, _entries, samplers, ticket = launched
        sched = self.scheduler
        if ticket is None or sched.waiting or plan.deferred or \
                len(plan.scheduled) != len(sched.running):
            return None
        row = {r.rid: i for i, r in enumerate(samplers)}
        ahead = []
        for item in plan.scheduled:
            r = sched.running.get(item.rid)
            if r is None:
                return None                             # ended while the step was in flight
            if item.phase == "prefill" and r.computed + item.tokens < len(r.prompt):
                return None                             # still in its prompt: not predicted
            n_out = len(r.output) + 1
            if r.cancelled or n_out >= r.max_new_tokens or \
                    len(r.prompt) + n_out > self.lm.cache.max_positions:
                continue                                # finishes with this step
            ahead.append(r)
        if not ahead:
            return None
        ahead.sort(key=lambda r: (r.arrival, str(r.rid)))
        entries = [Entry(r.rid, [-(row[r.rid] + 1)], [0]) for r in ahead]
        try:
            ctx = self.runner.prepare(entries, feedback=True)
        except Exception:
            return None
        return (entries, ctx, ahead)

    def _still_steady(self, entries: List[Entry]) -> bool:
        """May the step described ahead be launched before the step in flight is known?"""
        sched = self.scheduler
        if sched.waiting or len(entries) > len(sched.running):
            return False
        return all(e.rid in sched.running and not sched.running[e.rid].cancelled for e in entries)

    def _take_prepared(self, prepared, entries: List[Entry]):
        """The step described ahead, with the real token ids, if it is exactly the step
        that is now due."""
        if prepared is None:
            return None
        ahead, ctx, _ = prepared
        same = len(ahead) == len(entries) and all(
            a.rid == e.rid and len(e.tokens) == 1 and list(e.want) == [0]
            for a, e in zip(ahead, entries))
        if not same:
            self._drop(prepared)
            return None
        self.runner.patch_tokens(ctx, entries)
        self.ahead["used"] += 1
        return ctx

    def _drop(self, prepared) -> None:
        if prepared is None:
            return
        for e in prepared[0]:                           # requests that ended are closed already
            if e.rid in self.lm.cache.requests:
                self.lm.cache.abort(e.rid)
        self.ahead["dropped"] += 1

    # ------------------------------------------------------------------ generate
    def run(self) -> None:
        """Iterate until every submitted request has finished."""
        while not self.scheduler.idle:
            before = (len(self.scheduler.waiting), len(self.scheduler.running))
            in_flight = self._flight is not None
            done = self.step(ahead=True)
            if not done and not in_flight and self._flight is None and \
                    not self.scheduler.running and self.scheduler.waiting and \
                    before == (len(self.scheduler.waiting), 0):
                raise RuntimeError("scheduler made no progress: a waiting request cannot be admitted")
        self.flush()
        self._drop(self._prepared)
        self._prepared = None

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int,
                 sampling: Optional[SamplingParams] = None,
                 eos_ids: Sequence[int] = ()) -> List[List[int]]:
        """Generate for several prompts at once (continuous batching); returns the new
        tokens of each."""
        base = len(self.scheduler.finished)
        rids = [("gen", base, i) for i in range(len(prompts))]
        for rid, p in zip(rids, prompts):
            self.submit(rid, p, max_new_tokens, sampling, eos_ids)
        self.run()
        return [self.scheduler.finished.pop(rid).output for rid in rids]

    def stats(self) -> Dict[str, object]:
        """Counters in the manner of the reference's runtime and pool statistics
        (``paged_runtime.clj:434-440``, ``page_pool.clj:423-435``)."""
        cache = self.lm.cache
        return {
            "scheduler": dict(self.scheduler.stats),
            "runner": dict(self.runner.counters),
            "prepared_ahead": dict(self.ahead),
            "cache": dict(cache.stats),
            "free_pages": [a.free_count for a in cache.allocators],
            "pages": [a.num_pages for a in cache.allocators],
            "running": len(self.scheduler.running),
            "waiting": len(self.scheduler.waiting),
        }
