"""The benchmark's workloads: decoding a fixed batch at a given context, one step of whole
prompts, and the mixed workload (many requests of unequal length, prompts in portions
beside decoding requests, a shared prefix, through the scheduler).

Timing: CUDA events on the launching stream around the device work of each step (from the
copy of the step's description to the kernel that chooses the tokens); wall-clock time
around the whole loop for the end-to-end figures, in which every step's token ids come from
pinned host memory and every step's chosen ids are read back to the host."""
from __future__ import annotations

import random
import statistics
import time

from .roofline import quantiles


def timed_decode(engine, batch, ctx_len, steps, warmup, vocab, seed, sampling=None):
    """Prefill ``batch`` requests and time ``steps`` decode steps of all of them together,
    ending near ``ctx_len`` tokens of context.  Requests whose prompts finish early decode
    while the others still prefill, so every request gets enough tokens to generate that
    none finishes inside the timed region; the mean context actually decoded at is
    measured.  Returns a dict: per-step device milliseconds, wall seconds, kernel launches,
    mean context, bytes copied to the device per step."""
    import torch
    from ..csrc import ops
    rng = random.Random(seed)
    extra = batch + 2                      # steps the first request may decode before the last one starts
    max_new = steps + warmup + extra + 1
    prompt_len = max(16, ctx_len - max_new)
    rids = [("bench", batch, ctx_len, seed, i) for i in range(batch)]
    for rid in rids:
        engine.submit(rid, [rng.randrange(vocab) for _ in range(prompt_len)], max_new, sampling)
    while any(r.phase != "decode" for r in engine.scheduler.running.values()) or \
            engine.scheduler.waiting:
        engine.step()
    assert len(engine.scheduler.running) == batch
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    assert len(engine.scheduler.running) == batch
    ctx_before = sum(len(r.prompt) + len(r.output) for r in engine.scheduler.running.values()) / batch
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    launches0 = ops.launch_count()
    engine.timing_events = (starts, ends)
    t0 = time.perf_counter()
    for k in range(steps):
        engine.step_index = k
        engine.step(ahead=True)            # the host reads step k's tokens during step k + 1
    engine.flush()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    engine.timing_events = None
    launches = ops.launch_count() - launches0
    assert len(engine.scheduler.running) == batch, "a request finished inside the timed region"
    ms = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    for rid in rids:
        engine.cancel(rid)
    while engine.scheduler.running:
        engine.step()
    for rid in rids:
        engine.scheduler.finished.pop(rid, None)
    return {"ms": ms, "wall_s": wall, "launches": launches, "mean_context": ctx_before + steps / 2.0,
            "h2d_bytes": engine.runner.last_h2d_bytes, "d2h_bytes": 4 * batch + 16}


def timed_prefill(lm, n_prompts, prompt_len, vocab, warmup=3, repeats=5, seed=11):
    """One step of ``n_prompts`` whole prompts of ``prompt_len`` tokens; device milliseconds
    of ``repeats`` timed steps after ``warmup`` untimed ones."""
    import torch
    from ..engine.batch import Entry
    rng = random.Random(seed)
    runner, cache = lm.runner, lm.cache
    out = []
    for it in range(warmup + repeats):
        entries = []
        for i in range(n_prompts):
            rid = ("prefill", it, i)
            cache.open(rid)
            entries.append(Entry(rid, [rng.randrange(vocab) for _ in range(prompt_len)],
                                 [prompt_len - 1]))
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        runner.start_event = s              # recorded where the step's device work begins
        runner.step(entries)
        runner.start_event = None
        e.record()
        torch.cuda.synchronize()
        if it >= warmup:
            out.append(s.elapsed_time(e))
        for en in entries:
            cache.close(en.rid)
    return out


def mixed_workload(engine, vocab, n_requests=64, max_new=128, shared_fraction=0.3,
                   shared_prefix=256, min_prompt=16, max_prompt=1024, seed=4,
                   max_events=4096):
    """Many requests at once through the scheduler: prompt lengths uniform in
    [min_prompt, max_prompt) from ``seed``, a fraction of them beginning with one common
    prefix (found again through the prefix index once the first of them has computed it),
    prompts cut into the engine's portions and run beside the decoding requests.  Reports the
    time to each request's first token, the device time of the steps by kind (decode only,
    or with prompt tokens) as min / median / p95 / max, tokens per second over the whole run,
    and the cache's and scheduler's counters."""
    import torch
    rng = random.Random(seed)
    positions = engine.lm.cache.max_positions
    prefix = [rng.randrange(vocab) for _ in range(shared_prefix)]
    prompts = []
    for i in range(n_requests):
        n = rng.randrange(min_prompt, min(max_prompt, positions))
        if rng.random() < shared_fraction and n > shared_prefix:
            prompts.append(prefix + [rng.randrange(vocab) for _ in range(n - shared_prefix)])
        else:
            prompts.append([rng.randrange(vocab) for _ in range(n)])
    # (made before the clock starts: thousands of events take milliseconds to create)
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(max_events)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(max_events)]
    first_token = {}
    t_submit = time.perf_counter()

    def on_token(rid, _tok):
        if rid not in first_token:
            first_token[rid] = time.perf_counter() - t_submit

    rids = [("mixed", seed, i) for i in range(n_requests)]
    for rid, p in zip(rids, prompts):
        engine.submit(rid, p, max_new, on_token=on_token)
    engine.timing_events = (starts, ends)
    kinds = []
    before = dict(engine.scheduler.stats), dict(engine.lm.cache.stats), dict(engine.runner.counters)
    k = 0
    while not engine.scheduler.idle and k < max_events:
        steps0 = engine.runner.counters["launched"]
        engine.step_index = k
        engine.step(ahead=True)
        if engine.launched_entries is not None and engine.runner.counters["launched"] > steps0:
            # a step was launched: decode only if every request brought one token
            entries = engine.launched_entries
            kinds.append("decode" if all(len(e.tokens) == 1 for e in entries) else "with_prompt")
            k += 1
    engine.flush()
    while not engine.scheduler.idle:        # (only if the event budget ran out)
        engine.timing_events = None
        engine.step()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t_submit
    engine.timing_events = None
    ms = [s.elapsed_time(e) for s, e in zip(starts[:k], ends[:k])]
    generated = sum(len(engine.scheduler.finished.pop(rid).output) for rid in rids)
    prompt_tokens = sum(len(p) for p in prompts)
    sched, cache, runner = engine.scheduler.stats, engine.lm.cache.stats, engine.runner.counters
    return {
        "requests": n_requests, "prompt_tokens": prompt_tokens, "generated_tokens": generated,
        "wall_s": round(wall, 4),
        "generated_tokens_per_s": generated / wall,
        "all_tokens_per_s": (generated + prompt_tokens) / wall,
        "ttft_ms": quantiles([1e3 * v for v in first_token.values()]),
        "decode_step_ms": quantiles([m for m, kind in zip(ms, kinds) if kind == "decode"]),
        "prompt_step_ms": quantiles([m for m, kind in zip(ms, kinds) if kind == "with_prompt"]),
        "steps": k,
        "prefix_hits": cache["prefix_hits"] - before[1]["prefix_hits"],
        "evicted_pages": cache["evicted"] - before[1]["evicted"],
        "cow_copies": runner["cow_copies"] - before[2]["cow_copies"],
        "deferred_admissions": sched["deferred_admissions"] - before[0]["deferred_admissions"],
        "pool_pages": engine.lm.cache.allocators[0].num_pages,
        "mean_prompt": statistics.mean(len(p) for p in prompts),
    }
