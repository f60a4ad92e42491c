"""The scheduler: admission, cutting prompts into portions, decoding, finishing.

:func:`plan_iteration` is a pure function in the manner of the reference's planner
(``src/pretrained/continuation/scheduler.clj:42-105``): requests are ordered decode
first, then prefill by arrival, then by id; a decoding request takes one token, a
prefilling one ``min(available, remaining, prefill_chunk)``; ``minimum_prefill_tokens``
keeps that many tokens and one lane back for waiting prompts so that a full set of
decoding requests cannot starve them (``:63-76, 83-89``).

:class:`Scheduler` keeps the queue and the running set around it.  What happens when
pages run out is decided at *admission*, as in the reference
(``page_pool.clj:567-611``, ``doc/serving-architecture.md:276-277``): a request enters
only when the pages for its whole prompt and all the tokens it may generate can be
promised to it; otherwise it waits in arrival order and nothing is pre-empted.  A
request that could never fit (more pages than the pool has, or more tokens than the
model has positions) is refused at once with an error.
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Callable, Dict, Hashable, List, Optional, Sequence, Tuple

from ..cache.manager import CacheError, CacheManager, OutOfPages
from ..sampling.sampler import SamplingParams


@dataclass
class Request:
    rid: Hashable
    prompt: List[int]
    max_new_tokens: int
    sampling: SamplingParams = field(default_factory=SamplingParams)
    eos_ids: Tuple[int, ...] = ()
    arrival: int = 0
    on_token: Optional[Callable[[Hashable, int], None]] = None
    # progress
    phase: str = "waiting"            # waiting | prefill | decode | finished
    computed: int = 0                 # tokens whose keys and values are in the cache
    output: List[int] = field(default_factory=list)
    finish_reason: Optional[str] = None
    cancelled: bool = False
    page_keys: Optional[List[bytes]] = None     # prefix-index keys of the prompt's full pages

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def remaining_prefill(self) -> int:
        return len(self.prompt) - self.computed


@dataclass(frozen=True)
class SchedulerOptions:
    max_batched_tokens: int = 2048
    max_lanes: int = 64
    prefill_chunk: int = 128          # the reference's default (scheduler.clj:52-55)
    minimum_prefill_tokens: int = 0
    keep_finished: int = 4096         # finished requests remembered for their caller to fetch

    def validate(self) -> None:
        for name in ("max_batched_tokens", "max_lanes", "prefill_chunk"):
            v = getattr(self, name)
            if not isinstance(v, int) or v <= 0:
                raise ValueError(f"scheduler capacity {name} must be a positive integer, got {v!r}")
        if not isinstance(self.minimum_prefill_tokens, int) or self.minimum_prefill_tokens < 0:
            raise ValueError("minimum_prefill_tokens must be a non-negative integer")


@dataclass(frozen=True)
class Scheduled:
    rid: Hashable
    phase: str
    tokens: int


@dataclass(frozen=True)
class Plan:
    scheduled: Tuple[Scheduled, ...]
    deferred: Tuple[Hashable, ...]
    unused_tokens: int
    unused_lanes: int


def _rank(phase: str) -> int:
    return 0 if phase == "decode" else 2


def plan_iteration(opts: SchedulerOptions,
                   requests: Sequence[Tuple[Hashable, str, int, int]]) -> Plan:
    """One iteration's work.  ``requests``: (id, phase, remaining tokens, arrival) of the
    running requests, phase "decode" or "prefill".  Pure: the input is not changed."""
    opts.validate()
    for rid, phase, remaining, _arrival in requests:
        if phase not in ("decode", "prefill"):
            raise ValueError(f"request {rid!r}: unsupported phase {phase!r}")
        if remaining <= 0:
            raise ValueError(f"request {rid!r}: remaining tokens must be positive")
    ordered = sorted(requests, key=lambda r: (_rank(r[1]), r[3], str(r[0])))
    waiting_prefill = any(r[1] != "decode" for r in ordered)
    reserved_tokens = min(opts.minimum_prefill_tokens, opts.max_batched_tokens) \
        if waiting_prefill else 0
    reserved_lane = waiting_prefill and reserved_tokens > 0
    tokens_left, lanes_left = opts.max_batched_tokens, opts.max_lanes
    scheduled: List[Scheduled] = []
    deferred: List[Hashable] = []
    for rid, phase, remaining, _arrival in ordered:
        decode = phase == "decode"
        avail_tokens = max(0, tokens_left - reserved_tokens) if decode else tokens_left
        avail_lanes = max(0, lanes_left - 1) if (decode and reserved_lane) else lanes_left
        if avail_tokens == 0 or avail_lanes == 0:
            deferred.append(rid)
            continue
        n = min(avail_tokens, remaining, 1 if decode else opts.prefill_chunk)
        tokens_left -= n
        lanes_left -= 1
        scheduled.append(Scheduled(rid, phase, n))
    return Plan(tuple(scheduled), tuple(deferred), tokens_left, lanes_left)


class Scheduler:
    """Queue, running set, admission and completion.  Holds no tensors; the engine calls
    :meth:`next_plan`, runs the step, and reports the sampled tokens to :meth:`complete`."""

    def __init__(self, opts: SchedulerOptions, cache: CacheManager):
        opts.validate()
        self.opts = opts
        self.cache = cache
        self.waiting: List[Request] = []
        self.running: Dict[Hashable, Request] = {}
        # finished requests until their caller fetches them (``finished.pop(id)``); the oldest
        # are forgotten beyond ``keep_finished`` so that a long-running loop does not grow
        self.finished: "OrderedDict[Hashable, Request]" = OrderedDict()
        self._arrivals = 0
        self.stats = {"iterations": 0, "scheduled_tokens": 0, "admitted": 0,
                      "deferred_admissions": 0, "finished": 0, "prefix_waits": 0}
        # prefix-index key of a page -> the running request that will compute it first
        self._producing: Dict[bytes, Hashable] = {}

    # ------------------------------------------------------------------ submit
    def submit(self, request: Request) -> None:
        if not request.prompt:
            raise ValueError(f"request {request.rid!r}: empty prompt")
        if request.max_new_tokens < 0:
            raise ValueError(f"request {request.rid!r}: max_new_tokens must be >= 0")
        if request.rid in self.running or request.rid in self.finished or \
                any(r.rid == request.rid for r in self.waiting):
            raise ValueError(f"request id {request.rid!r} is already in use")
        total = self._reserve_tokens(request)
        if len(request.prompt) > self.cache.max_positions:
            raise CacheError(
                f"request {request.rid!r}: prompt of {len(request.prompt)} tokens exceeds the "
                f"model's {self.cache.max_positions} positions")
        for gi in range(len(self.cache.groups)):
            need = self.cache.pages_needed(gi, total, self.opts.prefill_chunk)
            have = self.cache.allocators[gi].num_pages
            if need > have:
                raise CacheError(
                    f"request {request.rid!r} needs {need} pages of group "
                    f"{self.cache.groups[gi].name!r}; the pool has {have}: it can never run")
        request.arrival = self._arrivals
        self._arrivals += 1
        request.phase = "waiting"
        self.waiting.append(request)

    def _reserve_tokens(self, request: Request) -> int:
        # The last generated token is returned but never written to the cache.
        total = len(request.prompt) + max(0, request.max_new_tokens - 1)
        return min(total, self.cache.max_positions)

    def cancel(self, rid: Hashable) -> None:
        """Honoured between steps (``paged_runtime.clj:606-620``)."""
        for r in self.waiting:
            if r.rid == rid:
                r.cancelled = True
        if rid in self.running:
            self.running[rid].cancelled = True

    # ------------------------------------------------------------------- admit
    def admit(self) -> List[Request]:
        """Move waiting requests into the running set, in arrival order, while a lane is
        free and their pages can be promised.  Stops at the first that does not fit.  A
        request whose prompt begins with pages that a running request is computing right now
        (the same tokens, not yet in the prefix index) is passed over until those pages are
        there: requests that arrive together with a common prefix then compute it once."""
        admitted: List[Request] = []
        for r in [w for w in self.waiting if w.cancelled]:
            self.waiting.remove(r)
            self._finish(r, "cancelled", opened=False)
        at = 0
        while at < len(self.waiting) and len(self.running) < self.opts.max_lanes:
            r = self.waiting[at]
            if self._awaits_prefix(r):
                self.stats["prefix_waits"] += 1
                at += 1
                continue
            try:
                self.cache.open(r.rid, reserve_tokens=self._reserve_tokens(r),
                                longest_step=self.opts.prefill_chunk)
            except OutOfPages:
                self.stats["deferred_admissions"] += 1
                break
            self.waiting.pop(at)
            r.computed = self.cache.match_prefix(r.rid, r.prompt)
            r.phase = "prefill"
            self.running[r.rid] = r
            for key in r.page_keys or ():
                if not self.cache.is_indexed(key):
                    self._producing.setdefault(key, r.rid)
            admitted.append(r)
            self.stats["admitted"] += 1
        return admitted

    def _awaits_prefix(self, r: Request) -> bool:
        """Whether the first page of ``r``'s prompt that the prefix index does not hold is one
        a running request is about to compute (it still prefills and has not passed it)."""
        if r.page_keys is None:
            r.page_keys = self.cache.page_keys(r.prompt)
        for i, key in enumerate(r.page_keys):
            if self.cache.is_indexed(key):
                continue
            owner = self.running.get(self._producing.get(key))
            if owner is None or owner.cancelled or owner.phase != "prefill" or \
                    owner.computed >= (i + 1) * self.cache.page_size:
                self._producing.pop(key, None)          # nobody (any more): compute it yourself
                return False
            return True
        return False

    # -------------------------------------------------------------------- plan
    def next_plan(self) -> Plan:
        for r in [x for x in self.running.values() if x.cancelled]:
            self._finish(r, "cancelled")
        self.admit()
        items = []
        for r in self.running.values():
            if r.phase == "prefill":
                items.append((r.rid, "prefill", r.remaining_prefill, r.arrival))
            else:
                items.append((r.rid, "decode", 1, r.arrival))
        plan = plan_iteration(self.opts, items)
        self.stats["iterations"] += 1
        self.stats["scheduled_tokens"] += sum(s.tokens for s in plan.scheduled)
        return plan

    def step_tokens(self, item: Scheduled) -> List[int]:
        """The token ids ``item`` feeds to the step: the next prompt portion, or the last
        generated token."""
        r = self.running[item.rid]
        if item.phase == "prefill":
            return r.prompt[r.computed:r.computed + item.tokens]
        return [r.output[-1]]

    def wants_logits(self, item: Scheduled) -> bool:
        """Logits are needed where a token will be chosen: at a decode token, and at the
        last token of a prompt."""
        r = self.running[item.rid]
        if item.phase == "decode":
            return True
        return r.computed + item.tokens == len(r.prompt) and r.max_new_tokens > 0

    # ---------------------------------------------------------------- complete
    def complete(self, plan: Plan, new_tokens: Dict[Hashable, int]) -> List[Request]:
        """Advance every scheduled request; ``new_tokens[rid]`` is the token chosen for the
        requests that wanted logits.  Returns the requests that finished."""
        done: List[Request] = []
        for item in plan.scheduled:
            r = self.running.get(item.rid)
            if r is None:           # ended while this step was already in flight
                continue
            r.computed += item.tokens
            if item.phase == "prefill" and r.computed < len(r.prompt):
                continue
            if r.max_new_tokens == 0:
                done.append(self._finish(r, "length"))
                continue
            tok = int(new_tokens[item.rid])
            r.output.append(tok)
            r.phase = "decode"
            if r.on_token is not None:
                r.on_token(r.rid, tok)
            reason = self.stop_reason(r, tok)
            if reason is not None:
                done.append(self._finish(r, reason))
        return done

    def stop_reason(self, r: Request, tok: int) -> Optional[str]:
        """``eos`` (the stop token stays in the output), ``length`` (budget used up) or
        ``capacity`` (no position left), as ``paged_runtime.clj:165-173``."""
        if tok in r.eos_ids:
            return "eos"
        if len(r.output) >= r.max_new_tokens:
            return "length"
        if len(r.prompt) + len(r.output) > self.cache.max_positions:
            return "capacity"
        return None

    def _finish(self, r: Request, reason: str, opened: bool = True) -> Request:
        r.phase = "finished"
        r.finish_reason = reason
        if opened:
            self.cache.close(r.rid)
            del self.running[r.rid]
        self.finished[r.rid] = r
        while len(self.finished) > self.opts.keep_finished:
            self.finished.popitem(last=False)
        self.stats["finished"] += 1
        return r

    @property
    def idle(self) -> bool:
        return not self.waiting and not self.running
