"""The scheduler's decisions without a GPU."""
import pytest

from pretrained_rstr_b200.cache import CacheError, CacheManager, GroupSpec
from pretrained_rstr_b200.engine.scheduler import (Request, SamplingParams, Scheduler,
                                                   SchedulerOptions, plan_iteration)

FULL = GroupSpec("full", (0,), 2, 16, None)


def test_decode_before_bounded_prefill():
    opts = SchedulerOptions(max_batched_tokens=10, max_lanes=4, prefill_chunk=6)
    plan = plan_iteration(opts, [("p1", "prefill", 20, 0), ("d1", "decode", 1, 5),
                                 ("d2", "decode", 1, 3), ("p2", "prefill", 3, 1)])
    assert [(s.rid, s.tokens) for s in plan.scheduled] == [("d2", 1), ("d1", 1), ("p1", 6), ("p2", 2)]
    assert plan.unused_tokens == 0 and plan.unused_lanes == 0 and plan.deferred == ()


def test_capacity_defers_without_changing_input():
    opts = SchedulerOptions(max_batched_tokens=4, max_lanes=2, prefill_chunk=128)
    reqs = [("a", "decode", 1, 0), ("b", "decode", 1, 1), ("c", "decode", 1, 2)]
    plan = plan_iteration(opts, reqs)
    assert [s.rid for s in plan.scheduled] == ["a", "b"] and plan.deferred == ("c",)
    assert reqs == [("a", "decode", 1, 0), ("b", "decode", 1, 1), ("c", "decode", 1, 2)]


def test_prefill_reservation_prevents_starvation():
    opts = SchedulerOptions(max_batched_tokens=4, max_lanes=4, prefill_chunk=8,
                            minimum_prefill_tokens=2)
    reqs = [(f"d{i}", "decode", 1, i) for i in range(4)] + [("p", "prefill", 9, 9)]
    plan = plan_iteration(opts, reqs)
    assert [(s.rid, s.tokens) for s in plan.scheduled] == [("d0", 1), ("d1", 1), ("p", 2)]
    assert set(plan.deferred) == {"d2", "d3"}
    starved = plan_iteration(SchedulerOptions(4, 4, 8, 0), reqs)
    assert "p" in starved.deferred


def test_bad_capacities_and_requests():
    with pytest.raises(ValueError, match="positive"):
        plan_iteration(SchedulerOptions(max_batched_tokens=0), [])
    with pytest.raises(ValueError, match="phase"):
        plan_iteration(SchedulerOptions(), [("a", "repairing", 1, 0)])
    with pytest.raises(ValueError, match="remaining"):
        plan_iteration(SchedulerOptions(), [("a", "decode", 0, 0)])


def _drive(sched, pick=lambda r: 7):
    """Run the scheduler to the end with a fake step: token = pick(request)."""
    trace = []
    guard = 0
    while not sched.idle:
        guard += 1
        assert guard < 1000
        plan = sched.next_plan()
        if not plan.scheduled:
            break
        for item in plan.scheduled:
            n = len(sched.step_tokens(item))
            sched.cache.reserve(item.rid, n)
            sched.cache.commit(item.rid)
        new = {s.rid: pick(sched.running[s.rid]) for s in plan.scheduled if sched.wants_logits(s)}
        trace.append([(s.rid, s.phase, s.tokens) for s in plan.scheduled])
        sched.complete(plan, new)
        sched.cache.check()
    return trace


def test_prompt_is_cut_into_portions_then_decoded_and_freed():
    cache = CacheManager([FULL], 16, 16, 4, 128)
    sched = Scheduler(SchedulerOptions(max_batched_tokens=12, max_lanes=2, prefill_chunk=8), cache)
    sched.submit(Request("a", list(range(20)), 3))
    sched.submit(Request("b", list(range(5)), 2))
    trace = _drive(sched)
    assert trace[0] == [("a", "prefill", 8), ("b", "prefill", 4)]
    assert trace[1] == [("a", "prefill", 8), ("b", "prefill", 1)]
    assert trace[2] == [("b", "decode", 1), ("a", "prefill", 4)]
    assert sched.finished["a"].output == [7, 7, 7] and sched.finished["a"].finish_reason == "length"
    assert sched.finished["b"].output == [7, 7]
    assert cache.free_pages(0) == 16 and cache.slots.free_count == 4


def test_finish_reasons():
    cache = CacheManager([FULL], 16, 16, 4, 32)
    sched = Scheduler(SchedulerOptions(64, 4, 64), cache)
    sched.submit(Request("eos", [1, 2, 3], 10, eos_ids=(7,)))
    sched.submit(Request("cap", list(range(30)), 10))
    sched.submit(Request("none", [1], 0))
    _drive(sched)
    assert sched.finished["eos"].output == [7] and sched.finished["eos"].finish_reason == "eos"
    assert sched.finished["cap"].finish_reason == "capacity"
    assert len(sched.finished["cap"].output) == 3          # positions 29, 30, 31 were evaluated
    assert sched.finished["none"].output == [] and sched.finished["none"].finish_reason == "length"


def test_pages_run_out_waits_at_admission_never_preempts():
    cache = CacheManager([FULL], 16, 4, 4, 128)            # 4 pages = 64 tokens in all
    sched = Scheduler(SchedulerOptions(64, 4, 64), cache)
    sched.submit(Request("a", list(range(30)), 10))        # 39 tokens -> 3 pages
    sched.submit(Request("b", list(range(20)), 5))         # 24 tokens -> 2 pages: must wait
    sched.submit(Request("c", [1, 2], 2))                  # would fit, but keeps its place behind b
    sched.next_plan()
    assert list(sched.running) == ["a"] and [r.rid for r in sched.waiting] == ["b", "c"]
    assert sched.stats["deferred_admissions"] == 1
    cache.close("a"); del sched.running["a"]               # a ends -> b and c are admitted
    sched.next_plan()
    assert list(sched.running) == ["b", "c"]
    with pytest.raises(CacheError, match="can never run"):
        sched.submit(Request("huge", list(range(60)), 30))  # 89 tokens > the whole pool
    with pytest.raises(CacheError, match="positions"):
        Scheduler(SchedulerOptions(64, 4, 64), CacheManager([FULL], 16, 64, 4, 32)).submit(
            Request("long", list(range(40)), 1))
    with pytest.raises(ValueError, match="already in use"):
        sched.submit(Request("b", [1], 1))


def test_cancel_between_steps():
    cache = CacheManager([FULL], 16, 8, 2, 64)
    sched = Scheduler(SchedulerOptions(64, 2, 64), cache)
    sched.submit(Request("a", [1, 2, 3], 50))
    sched.submit(Request("w", [1, 2, 3], 50))
    sched.submit(Request("q", [1, 2, 3], 50))
    sched.next_plan()
    sched.cancel("a")
    sched.cancel("q")
    plan = sched.next_plan()
    assert "a" not in sched.running and sched.finished["a"].finish_reason == "cancelled"
    assert sched.finished["q"].finish_reason == "cancelled"
    assert [s.rid for s in plan.scheduled] == ["w"]
    cache.check()


def test_sampling_params_defaults():
    assert SamplingParams().greedy and SamplingParams(temperature=0.0).greedy
    assert not SamplingParams(temperature=0.8).greedy


def test_requests_that_arrive_together_compute_a_common_prefix_once():
    """Three requests with the same first two pages arrive at once: the first computes them,
    the others are passed over until the pages are in the prefix index and then take them
    from there; a fourth with another prompt does not wait behind them."""
    cache = CacheManager([FULL], 8, 64, 8, 128, share_prefixes=True)
    sched = Scheduler(SchedulerOptions(max_batched_tokens=64, max_lanes=8, prefill_chunk=8), cache)
    prefix = list(range(100, 116))                      # two full pages
    prompts = {"a": prefix + [1, 2, 3], "b": prefix + [4, 5, 6, 7, 8], "c": prefix + [9],
               "d": list(range(200, 212))}
    for rid, p in prompts.items():
        sched.submit(Request(rid=rid, prompt=p, max_new_tokens=2))
    computed = {rid: 0 for rid in prompts}
    admitted_at = {}
    step = 0
    while not sched.idle:
        step += 1
        assert step < 100
        plan = sched.next_plan()
        for rid in sched.running:
            admitted_at.setdefault(rid, step)
        for item in plan.scheduled:
            toks = sched.step_tokens(item)
            cache.reserve(item.rid, len(toks))
            cache.commit(item.rid, toks)
            if item.phase == "prefill":
                computed[item.rid] += len(toks)
        sched.complete(plan, {s.rid: 7 for s in plan.scheduled if sched.wants_logits(s)})
    # a and d start at once; b and c wait for a's two pages and then compute only their own tails
    assert admitted_at["a"] == 1 and admitted_at["d"] == 1
    assert admitted_at["b"] == admitted_at["c"] == 3
    assert computed == {"a": 19, "b": 5, "c": 1, "d": 12}
    assert cache.stats["prefix_hits"] == 4 and sched.stats["prefix_waits"] > 0
    cache.check()


def test_a_prefix_is_not_waited_for_when_its_producer_goes_away():
    cache = CacheManager([FULL], 8, 64, 8, 128, share_prefixes=True)
    sched = Scheduler(SchedulerOptions(max_batched_tokens=64, max_lanes=8, prefill_chunk=8), cache)
    prefix = list(range(100, 116))
    sched.submit(Request(rid="a", prompt=prefix + [1, 2, 3], max_new_tokens=2))
    sched.submit(Request(rid="b", prompt=prefix + [4], max_new_tokens=2))
    sched.next_plan()
    assert set(sched.running) == {"a"} and [r.rid for r in sched.waiting] == ["b"]
    sched.cancel("a")
    sched.next_plan()                                   # a ends; nobody computes the prefix now
    assert set(sched.running) == {"b"} and sched.running["b"].computed == 0
