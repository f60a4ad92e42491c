#!/usr/bin/env python3
"""Benchmark: decode tokens/s (batch 8 by default) and prefill tokens/s at 2,048 tokens
for GPT-2 small with random weights, each with its fraction of the roofline.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

Prints ONE JSON line.  A "step" is one decode step of the whole batch.  ``value`` is
decoded tokens per second from device time (CUDA events around each step's kernels);
``e2e`` is the same through the engine's public step (token ids from pinned host memory
in, sampled ids read back to the host, every step).  ``prefill`` is one step of 2,048
prompt tokens (2 prompts x 1,024).  ``roofline`` divides the bytes a decode step has to
read (every weight once, and the cache of the live requests) by its time and by the
measured copy bandwidth.  Weights (247 MB) plus cache are larger than the 126 MB L2, so
no flush is needed between timed steps.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SMALL = dict(n_layer=12, n_embd=768, n_head=12, n_inner=3072, vocab_size=50257, n_positions=1024)
SIZES = {
    "small": SMALL,
    "medium": dict(n_layer=24, n_embd=1024, n_head=16, n_inner=4096, vocab_size=50257, n_positions=1024),
    "xl": dict(n_layer=48, n_embd=1600, n_head=25, n_inner=6400, vocab_size=50257, n_positions=1024),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as fh:
                raw = json.load(fh)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(raw.get(k), (int, float)):
                    out[k] = float(raw[k])
            out["source"] = "measured"
            return out
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self.index = index

    def _run(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                     "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) >= 6:
                    self.samples.append(float(parts[0]))
                    self.max_mhz = float(parts[1])
                    for name, val in zip(names, parts[2:6]):
                        if val.lower().startswith("active"):
                            self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def model_bytes(cfg, dtype_bytes=2):
    d, f, L, V = cfg["n_embd"], cfg["n_inner"], cfg["n_layer"], cfg["vocab_size"]
    per_layer = (d * 3 * d + d * d + d * f + f * d) * dtype_bytes + (3 * d + d + f + d + 4 * d) * 4
    return L * per_layer + V * d * dtype_bytes + 2 * d * 4


def kv_bytes_per_token(cfg, dtype_bytes=2):
    return 2 * cfg["n_layer"] * cfg["n_embd"] * dtype_bytes


def prefill_flops(cfg, n_prompts, prompt_len):
    d, f, L, V = cfg["n_embd"], cfg["n_inner"], cfg["n_layer"], cfg["vocab_size"]
    t = n_prompts * prompt_len
    gemm = 2 * t * (d * 3 * d + d * d + 2 * d * f) * L
    attn = L * n_prompts * 4 * d * (prompt_len * (prompt_len + 1) // 2)
    head = 2 * n_prompts * d * V
    return gemm + attn + head


def run_reference(args) -> int:
    print(json.dumps({
        "impl": "reference",
        "unavailable": "replikativ/pretrained-rstr is Clojure on the JVM computing through the "
                       "external Raster library; pip reports that its folder is not installable "
                       "(neither setup.py nor pyproject.toml found), and no JVM, Clojure or Raster "
                       "exists offline"}))
    return 0


def timed_decode(engine, lm, batch, ctx_len, steps, warmup, vocab, seed):
    """Prefill ``batch`` requests and time ``steps`` decode steps of all of them together,
    ending near ``ctx_len`` tokens of context.  Requests whose prompts finish early decode
    while the others still prefill, so every request gets enough tokens to generate that
    none finishes inside the timed region; the mean context actually decoded at is
    measured.  Returns per-step device milliseconds, wall seconds, launches, mean context,
    bytes copied to the device per step."""
    import random
    import torch
    from pretrained_rstr_b200.csrc import ops
    rng = random.Random(seed)
    extra = batch + 2                      # steps the first request may decode before the last one starts
    max_new = steps + warmup + extra + 1
    prompt_len = max(16, ctx_len - max_new)
    rids = [("bench", batch, i) for i in range(batch)]
    for rid in rids:
        engine.submit(rid, [rng.randrange(vocab) for _ in range(prompt_len)], max_new)
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
    mean_ctx = ctx_before + steps / 2.0
    for rid in rids:
        engine.cancel(rid)
    while engine.scheduler.running:
        engine.step()
    h2d = engine.runner.last_h2d_bytes
    return ms, wall, launches, mean_ctx, h2d


def profile_gemm(shape: str) -> int:
    """Small workload for ncu: the prompt-time GEMM at one shape, every tile width and every
    split of the reduction over a cluster that fits, timed as a CUDA graph of 20 launches,
    with cuBLAS (torch.mm) beside it."""
    import torch
    from pretrained_rstr_b200.csrc import ops
    m, n, k = (int(x) for x in shape.split(","))

    def timeit(f, reps=20):
        f()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(reps):
                f()
        g.replay()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        g.replay()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / reps * 1e3

    a = torch.randn(m, k, device="cuda").bfloat16()
    w = torch.randn(n, k, device="cuda").bfloat16()
    outb = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
    outf = torch.zeros(m, n, device="cuda")
    bias = torch.randn(n, device="cuda")
    res = {}
    for tn in (0, 32, 64, 96, 128, 160, 192, 224, 256):
        res[f"tile{tn}"] = {
            "bf16_plain_us": timeit(lambda: ops.gemm_bf16(outb, a, w, tile_n=tn)),
            "bf16_bias_gelu_us": timeit(lambda: ops.gemm_bf16(outb, a, w, bias=bias, act="gelu_new", tile_n=tn)),
            "f32_bias_resid_us": timeit(lambda: ops.gemm_bf16(outf, a, w, bias=bias, resid=outf, tile_n=tn)),
        }
    blocks = -(-k // 64)
    for tn in (64, 128):
        for sp in (2, 4, 8):
            if -(-blocks // sp) * (sp - 1) >= blocks or -(-m // 128) * -(-n // tn) * sp > 148:
                continue
            res[f"tile{tn}_split{sp}"] = {
                "bf16_plain_us": timeit(lambda: ops.gemm_bf16(outb, a, w, tile_n=tn, split_k=sp)),
                "bf16_bias_gelu_us": timeit(lambda: ops.gemm_bf16(outb, a, w, bias=bias, act="gelu_new", tile_n=tn, split_k=sp)),
                "f32_bias_resid_us": timeit(lambda: ops.gemm_bf16(outf, a, w, bias=bias, resid=outf, tile_n=tn, split_k=sp)),
            }
    res["cublas_us"] = timeit(lambda: torch.mm(a, w.t(), out=outb))
    res["gflop"] = 2 * m * n * k / 1e9
    print(json.dumps({"profile_gemm": shape, **res}))
    return 0


def profile_decode(batch: int, table: bool = False) -> int:
    """Small workload for ncu: the benchmark model, ``batch`` requests of 900 prompt tokens,
    then four decode steps launched kernel by kernel (no CUDA graph)."""
    import random
    import torch
    from pretrained_rstr_b200 import load_lm
    from pretrained_rstr_b200.config import GPT2Config
    from pretrained_rstr_b200.weights import make_random_model
    tmp = tempfile.mkdtemp(prefix="prb200_prof_")
    try:
        make_random_model(tmp, GPT2Config.from_dict(dict(SMALL)), seed=2, dtype=torch.bfloat16)
        m = load_lm(tmp, gpu=True, dtype="bfloat16", max_lanes=64, max_batched_tokens=2048,
                    prefill_chunk=1024, share_prefixes=False)
    finally:
        import shutil
        shutil.rmtree(tmp, ignore_errors=True)
    e = m.engine
    e.runner.use_graphs = False
    rng = random.Random(0)
    for i in range(batch):
        e.submit(i, [rng.randrange(SMALL["vocab_size"]) for _ in range(900)], 100)
    while any(r.phase != "decode" for r in e.scheduler.running.values()) or e.scheduler.waiting:
        e.step()
    if table:
        from torch.profiler import ProfilerActivity, profile
        e.step()
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(4):
                e.step()
            torch.cuda.synchronize()
        print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=12,
                                        max_name_column_width=70))
    else:
        for _ in range(4):
            e.step()
        torch.cuda.synchronize()
    print(json.dumps({"profile_decode": batch, "ok": True}))
    return 0


def profile_prompt(spec: str, table: bool = True) -> int:
    """One prompt alone: a step of N tokens (after AT tokens already in the cache) as the
    engine runs it (a CUDA graph from the third time on): device time of the step and the
    torch profiler's kernel table.  ``spec`` is "N" or "N,AT"."""
    import random
    import torch
    from torch.profiler import ProfilerActivity, profile
    from pretrained_rstr_b200 import load_lm
    from pretrained_rstr_b200.config import GPT2Config
    from pretrained_rstr_b200.engine.batch import Entry
    from pretrained_rstr_b200.weights import make_random_model
    parts = [int(x) for x in spec.split(",")]
    n, at = parts[0], (parts[1] if len(parts) > 1 else 0)
    tmp = tempfile.mkdtemp(prefix="prb200_prof_")
    try:
        make_random_model(tmp, GPT2Config.from_dict(dict(SMALL)), seed=2, dtype=torch.bfloat16)
        m = load_lm(tmp, gpu=True, dtype="bfloat16", max_lanes=8, max_batched_tokens=2048,
                    prefill_chunk=1024, share_prefixes=False)
    finally:
        import shutil
        shutil.rmtree(tmp, ignore_errors=True)
    runner, cache = m.loaded.runner, m.loaded.cache
    rng = random.Random(0)
    ids = [rng.randrange(SMALL["vocab_size"]) for _ in range(at + n)]

    def one(tag):
        cache.open(tag)
        if at:
            runner.step([Entry(tag, ids[:at], [])])
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        runner.start_event = start
        runner.step([Entry(tag, ids[at:], [n - 1])])
        end.record()
        torch.cuda.synchronize()
        runner.start_event = None
        cache.close(tag)
        return start.elapsed_time(end)

    for i in range(4):
        one(("warm", i))
    times = sorted(one(("timed", i)) for i in range(5))
    if table:
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for i in range(3):
                one(("table", i))
        print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=12,
                                        max_name_column_width=70))
    print(json.dumps({"profile_prompt": spec, "device_ms": [round(t, 4) for t in times]}))
    return 0


def profile_attention(spec: str) -> int:
    """The prompt attention kernels alone: PROMPTS prompts of LENGTH tokens, HEADS heads of
    64 ("HEADS,PROMPTS,LENGTH"), causal, over a paged cache, each timed as a CUDA graph of 10
    launches: the mma.sync kernel, the tcgen05 kernel with one CTA per tile, and with a tile's
    keys in parts of 1 to 32 blocks."""
    import torch
    from pretrained_rstr_b200.csrc import ops
    nh, nseq, length = (int(x) for x in spec.split(","))
    dh = ps = 64
    g = torch.Generator(device="cpu").manual_seed(0)
    pages_per = -(-length // ps)
    num_pages = nseq * pages_per + 3
    k = torch.randn(num_pages, nh, ps, dh, generator=g).bfloat16().cuda()
    v = torch.randn(num_pages, nh, ps, dh, generator=g).bfloat16().cuda()
    perm = torch.randperm(num_pages, generator=g).tolist()
    table = torch.full((nseq, pages_per + 1), -1, dtype=torch.int32)
    for b in range(nseq):
        for i in range(pages_per):
            table[b, i] = perm.pop()
    table = table.cuda()
    pos = torch.cat([torch.arange(length) for _ in range(nseq)]).int().cuda()
    q = torch.randn(nseq * length, nh * dh, generator=g).bfloat16().cuda()
    tiles = [(b, b * length + r0, min(128, length - r0)) for b in range(nseq)
             for r0 in range(0, length, 128)]
    tr, t0, tn = (torch.tensor([x[i] for x in tiles], dtype=torch.int32, device="cuda")
                  for i in range(3))
    status = torch.zeros(4, dtype=torch.int32, device="cuda")

    def timeit(f, reps=10):
        f()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(reps):
                f()
        graph.replay()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        graph.replay()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / reps * 1e3

    blocks = -(-length // 64)
    units = len(tiles) * nh
    cases = [("mma_sync", ops.attention_prefill, {}), ("tcgen05", ops.attention_prefill_tc, {})]
    for part in (1, 2, 4, 8, 16, 32):
        most = -(-blocks // part)
        if part < blocks and most <= ops.PREFILL_MAX_PARTS:
            ws = (torch.empty(units * most * 8192, device="cuda"),
                  torch.empty(units * most * 256, device="cuda"),
                  torch.zeros(units, dtype=torch.int32, device="cuda"))
            cases.append((f"tcgen05_parts_of_{part}", ops.attention_prefill_tc,
                          {"part_blocks": part, "max_parts": most, "parts": ws}))
    flops = 4 * nseq * nh * dh * length * (length + 1) / 2
    res, ref = {}, None
    for name, fn, kw in cases:
        out = torch.zeros_like(q)
        us = timeit(lambda: fn(out, q, k, v, table, pos, tr, t0, tn, None, len(tiles), nh, 0.125,
                               None, status, **kw))
        if ref is None:
            ref = out.clone()
        res[name] = {"us": round(us, 1), "tflops": round(flops / us / 1e6, 1),
                     "max_diff": float((out.float() - ref.float()).abs().max())}
    print(json.dumps({"profile_attention": spec, "status": status.tolist(), **res}))
    return 0


def profile_prefill(table: bool = True) -> int:
    """Small workload for a profiler: one step of 2 x 1,000 prompt tokens, launched kernel
    by kernel, with the torch profiler's kernel table printed (``table``; off under ncu)."""
    import random
    import torch
    from torch.profiler import ProfilerActivity, profile
    from pretrained_rstr_b200 import load_lm
    from pretrained_rstr_b200.config import GPT2Config
    from pretrained_rstr_b200.engine.batch import Entry
    from pretrained_rstr_b200.weights import make_random_model
    tmp = tempfile.mkdtemp(prefix="prb200_prof_")
    try:
        make_random_model(tmp, GPT2Config.from_dict(dict(SMALL)), seed=2, dtype=torch.bfloat16)
        m = load_lm(tmp, gpu=True, dtype="bfloat16", max_lanes=8, max_batched_tokens=2048,
                    prefill_chunk=1024, share_prefixes=False)
    finally:
        import shutil
        shutil.rmtree(tmp, ignore_errors=True)
    runner, cache = m.loaded.runner, m.loaded.cache
    runner.use_graphs = False
    rng = random.Random(0)

    def one_step(tag):
        entries = []
        for i in range(2):
            cache.open((tag, i))
            entries.append(Entry((tag, i), [rng.randrange(SMALL["vocab_size"]) for _ in range(1000)],
                                 [999]))
        runner.step(entries)
        torch.cuda.synchronize()
        for e in entries:
            cache.close(e.rid)

    one_step("warm")
    if not table:
        one_step("timed")
        print(json.dumps({"profile_prefill": True, "ok": True}))
        return 0
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        one_step("timed")
    print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=12,
                                    max_name_column_width=70))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--profile-prefill", action="store_true")
    ap.add_argument("--profile-gemm", default=None, metavar="M,N,K")
    ap.add_argument("--profile-prompt", default=None, metavar="N[,AT]",
                    help="one prompt step of N tokens after AT cached ones: device time, kernel table")
    ap.add_argument("--profile-attention", default=None, metavar="HEADS,PROMPTS,LENGTH",
                    help="the prompt attention kernels alone, every way of sharing a tile's keys")
    ap.add_argument("--profile-decode", type=int, default=None, metavar="BATCH")
    ap.add_argument("--kernel-table", action="store_true",
                    help="with --profile-decode: print the torch profiler's kernel table")
    ap.add_argument("--no-table", action="store_true",
                    help="with --profile-prefill: no torch profiler (for runs under ncu)")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers than the size has (named in the record)")
    ap.add_argument("--size", default="small", choices=sorted(SIZES),
                    help="layer sizes: GPT-2 small (the default record), medium or xl")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.profile_gemm:
        return profile_gemm(args.profile_gemm)
    if args.profile_decode:
        return profile_decode(args.profile_decode, args.kernel_table)
    if args.profile_prefill:
        return profile_prefill(not args.no_table)
    if args.profile_prompt:
        return profile_prompt(args.profile_prompt, not args.no_table)
    if args.profile_attention:
        return profile_attention(args.profile_attention)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from pretrained_rstr_b200 import load_lm
    from pretrained_rstr_b200.config import GPT2Config
    from pretrained_rstr_b200.engine.batch import Entry
    from pretrained_rstr_b200.weights import make_random_model

    raw = dict(SIZES[args.size])
    full_layers = raw["n_layer"]
    if args.layers:
        raw["n_layer"] = args.layers
    cfg = GPT2Config.from_dict(raw)
    pk = peaks()
    vocab = raw["vocab_size"]
    steps, warmup, ctx_len = args.steps, args.warmup, min(args.context, raw["n_positions"])
    steps = max(1, min(steps, ctx_len - warmup - 64 - 3 - 16))     # every request must fit its context
    tmp = tempfile.mkdtemp(prefix="prb200_bench_")
    try:
        make_random_model(tmp, cfg, seed=2, dtype=torch.bfloat16)
        m = load_lm(tmp, gpu=True, dtype="bfloat16", max_lanes=64, max_batched_tokens=2048,
                    prefill_chunk=1024, share_prefixes=False)
    finally:
        import shutil
        shutil.rmtree(tmp, ignore_errors=True)
    engine = m.engine

    # ---- prefill: one step of 2 x 1024 prompt tokens
    import random
    rng = random.Random(11)
    pre_ms = []
    for it in range(3 + 5):
        entries = []
        for i in range(2):
            rid = ("prefill", it, i)
            m.loaded.cache.open(rid)
            entries.append(Entry(rid, [rng.randrange(vocab) for _ in range(1024)], [1023]))
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        m.loaded.runner.start_event = s          # recorded where the step's device work begins
        m.loaded.runner.step(entries)
        m.loaded.runner.start_event = None
        e.record()
        torch.cuda.synchronize()
        if it >= 3:
            pre_ms.append(s.elapsed_time(e))
        for en in entries:
            m.loaded.cache.close(en.rid)
    pre = statistics.median(pre_ms)
    flops = prefill_flops(raw, 2, 1024)
    prefill = {"value": 2048 / (pre / 1e3), "tokens": 2048, "ms": pre,
               "frac": flops / (pre / 1e3) / (pk["bf16_tflops"] * 1e12)}

    # ---- decode
    points = {}
    clocks = ClockSampler()
    clocks.__enter__()
    for b in (1, 64):
        ms, wall, _l, _c, _h = timed_decode(engine, m.loaded, b, ctx_len, steps, warmup, vocab, b)
        points[f"decode_b{b}"] = b / (statistics.mean(ms) / 1e3)
        points[f"decode_b{b}_ms"] = [round(min(ms), 4), round(statistics.median(ms), 4),
                                     round(max(ms), 4)]
    ms, wall, launches, mean_ctx, h2d = timed_decode(engine, m.loaded, args.batch, ctx_len,
                                                    steps, warmup, vocab, 5)
    clocks.__exit__(None, None, None)
    step_ms = statistics.mean(ms)
    value = args.batch / (step_ms / 1e3)
    bytes_step = model_bytes(raw) + args.batch * mean_ctx * kv_bytes_per_token(raw)
    achieved = bytes_step / (step_ms / 1e3) / 1e9
    record = {
        "metric": f"decode tok/s (GPT-2 {args.size}, random weights)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"model": f"gpt2-{args.size}-random", "global_batch": args.batch, "seq_len": ctx_len,
                   "parallelism": "single-gpu", "n_layer": raw["n_layer"], "n_layer_full": full_layers,
                   "n_embd": raw["n_embd"], "n_head": raw["n_head"], "n_inner": raw["n_inner"],
                   "vocab_size": vocab, "n_positions": raw["n_positions"], "page_size": 64,
                   "mean_context": mean_ctx, "l2": "inputs_exceed_l2",
                   "peaks": pk["source"]},
        "e2e": {"value": args.batch * steps / wall, "unit": "tokens/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * args.batch + 16},
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"]},
        "points": points,
        "clocks": clocks.summary(),
    }
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    sys.exit(main())
