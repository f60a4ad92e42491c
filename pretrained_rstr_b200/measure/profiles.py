"""Small workloads of single kernels and single steps, for profiler captures and sweeps:
``bench.py --profile-gemm/-decode/-prompt/-attention/-prefill`` run them.  Each prints one
JSON line (and, where asked, the torch profiler's kernel table)."""
from __future__ import annotations

import json
import tempfile

from .roofline import SMALL

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
    for tn in (64, 128, 192, 256):
        res[f"pair{tn}"] = {
            "bf16_plain_us": timeit(lambda: ops.gemm_bf16(outb, a, w, tile_n=tn, pair=True)),
            "bf16_bias_gelu_us": timeit(lambda: ops.gemm_bf16(outb, a, w, bias=bias, act="gelu_new", tile_n=tn, pair=True)),
            "f32_bias_resid_us": timeit(lambda: ops.gemm_bf16(outf, a, w, bias=bias, resid=outf, tile_n=tn, pair=True)),
        }
    blocks = -(-k // 64)
    for tn in (64, 128, 192, 256):
        for sp in ((2, 4, 8) if tn <= 128 else (2,)):
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


def profile_host(batch: int) -> int:
    """The host's side of a decode step: the benchmark model with ONE layer (so that the
    device is never the bound), ``batch`` requests decoding through
    ``Engine.step(ahead=True)``; wall time a step over 300 steps, then the same under
    cProfile (its overhead about doubles the times; the shares are what it is for)."""
    import cProfile
    import pstats
    import random
    import time
    import torch
    from pretrained_rstr_b200 import load_lm
    from pretrained_rstr_b200.config import GPT2Config
    from pretrained_rstr_b200.weights import make_random_model
    raw = dict(SMALL)
    raw["n_layer"] = 1
    tmp = tempfile.mkdtemp(prefix="prb200_prof_")
    try:
        make_random_model(tmp, GPT2Config.from_dict(raw), seed=2, dtype=torch.bfloat16)
        m = load_lm(tmp, gpu=True, dtype="bfloat16", max_lanes=64, max_batched_tokens=2048,
                    prefill_chunk=1024, share_prefixes=False)
    finally:
        import shutil
        shutil.rmtree(tmp, ignore_errors=True)
    e = m.engine
    rng = random.Random(0)
    for i in range(batch):
        e.submit(i, [rng.randrange(raw["vocab_size"]) for _ in range(300)], 650)
    while any(r.phase != "decode" for r in e.scheduler.running.values()) or e.scheduler.waiting:
        e.step()
    for _ in range(30):
        e.step(ahead=True)
    e.flush()
    torch.cuda.synchronize()
    steps = 300
    t0 = time.perf_counter()
    for _ in range(steps):
        e.step(ahead=True)
    e.flush()
    torch.cuda.synchronize()
    wall_us = (time.perf_counter() - t0) / steps * 1e6
    prof = cProfile.Profile()
    prof.enable()
    for _ in range(200):
        e.step(ahead=True)
    e.flush()
    prof.disable()
    pstats.Stats(prof).sort_stats("tottime").print_stats(16)
    print(json.dumps({"profile_host": batch, "layers": 1, "wall_us_per_step": round(wall_us, 1)}))
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
    # the planner's work list: exactly the CTAs that have work, longest first, long tiles in parts
    import numpy as np
    from pretrained_rstr_b200.parts.attention import AttentionWork
    planner = AttentionWork()
    planner.note_mixer(nh, None, ops.sm_count())
    host = {name: np.full(cap, fill, dtype=np.int32)
            for name, (cap, fill) in planner.arrays(nseq * length, nseq).items()}
    got = planner.fill(host, [length] * nseq, [0] * nseq)
    dev = {name: torch.from_numpy(a).cuda() for name, a in host.items()}
    n_slots = planner.slot_cap()
    ws = (torch.empty(n_slots * nh * 8192, device="cuda"), torch.empty(n_slots * nh * 256, device="cuda"),
          torch.zeros(n_slots * nh, dtype=torch.int32, device="cuda"))
    cases.append((f"tcgen05_listed_{got['items']}_items_parts_of_{int(host['part_blocks'][0])}",
                  ops.attention_prefill_tc,
                  {"parts": ws, "items": (dev["item_tile"], dev["item_part"], dev["item_slot"], None,
                                          dev["part_blocks"], got["items"], n_slots)}))
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




def _graph_time_us(fn, reps=10):
    """Microseconds per call of ``fn``, timed as a CUDA graph of ``reps`` calls."""
    import torch
    fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(reps):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    best = None
    for _ in range(3):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        graph.replay()
        e.record()
        torch.cuda.synchronize()
        us = s.elapsed_time(e) / reps * 1e3
        best = us if best is None else min(best, us)
    return best


def profile_decode_attention(spec: str) -> int:
    """The decode attention kernel alone: REQUESTS single tokens at context CONTEXT, HEADS
    heads of 64 ("HEADS,REQUESTS,CONTEXT"), over a paged cache with shuffled pages, by split
    size; each a CUDA graph of 10 or more launches that go round several sets of requests,
    together larger than the L2.  Bytes = the keys and values read once."""
    import torch
    from ..csrc import ops
    nh, nreq, ctx = (int(x) for x in spec.split(","))
    dh = ps = 64
    g = torch.Generator(device="cpu").manual_seed(0)
    pages_per = -(-ctx // ps)
    nbytes = 2 * nreq * nh * ctx * dh * 2
    # as many sets of requests as together exceed the L2, one set per launch in turn: inside
    # a step no layer finds its keys and values in the L2 either
    sets = max(1, -(-int(300e6) // nbytes))
    num_pages = sets * nreq * pages_per + 3
    k = torch.randn(num_pages, nh, ps, dh, generator=g).bfloat16().cuda()
    v = torch.randn(num_pages, nh, ps, dh, generator=g).bfloat16().cuda()
    perm = torch.randperm(num_pages, generator=g).tolist()
    tables = []
    for _ in range(sets):
        table = torch.full((nreq, pages_per + 1), -1, dtype=torch.int32)
        for b in range(nreq):
            for i in range(pages_per):
                table[b, i] = perm.pop()
        tables.append(table.cuda())
    seq = torch.arange(nreq, dtype=torch.int32).cuda()
    pos = torch.full((nreq,), ctx - 1, dtype=torch.int32).cuda()
    q = torch.randn(nreq, nh * dh, generator=g).bfloat16().cuda()
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    res, ref = {}, None
    granule = ops.decode_split()
    chosen = None
    try:
        from ..parts.attention import decode_splits
        chosen = decode_splits(nreq * nh, -(-ctx // 256) * 256, ps)[0]
    except Exception:
        pass
    launches = max(10, sets)

    def timed(one):
        turn = [0]

        def run():
            one(tables[turn[0] % sets])
            turn[0] += 1
        return _graph_time_us(run, launches)

    for split in sorted({granule, 2 * granule, 3 * granule, 4 * granule, 8 * granule,
                         -(-ctx // granule) * granule} | ({chosen} if chosen else set())):
        splits = -(-ctx // split)
        ws = torch.zeros(nreq * nh * splits * (dh + 4), device="cuda")
        counters = torch.zeros(nreq * nh, dtype=torch.int32, device="cuda")
        out = torch.zeros_like(q)
        us = timed(lambda table: ops.attention_decode(out, q, k, v, table, seq, pos, None, None,
                                                      nreq, nh, 0.125, None, ws, counters,
                                                      splits, status, split_keys=split))
        if ref is None:
            ref = out.clone()
        res[f"split{split}"] = {"us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1),
                                "ctas": nreq * nh * splits,
                                "max_diff": float((out.float() - ref.float()).abs().max())}
    if ops.decode_ring_supports(dh, ps):
        ws = torch.zeros(ops.decode_ring_workspace(nreq, nh, dh), device="cuda")
        counters = torch.zeros(nreq * nh, dtype=torch.int32, device="cuda")
        for stages in (2, 3, 4):
            out = torch.zeros_like(q)
            us = timed(lambda table: ops.attention_decode_ring(
                out, q, k, v, table, seq, pos, None, None, nreq, nh, 0.125, None, ws, counters,
                status, new_keys=4, stages=stages, max_context=-(-ctx // 256) * 256))
            res[f"ring_stages{stages}"] = {"us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1),
                                           "max_diff": float((out.float() - ref.float()).abs().max())}
    print(json.dumps({"profile_decode_attention": spec, "mbytes": round(nbytes / 1e6, 2),
                      "sets": sets,
                      "engine_split": chosen, "status": status.tolist(), **res}))
    return 0


def profile_sample(spec: str) -> int:
    """The sampling kernel alone: ROWS rows of VOCAB float32 logits, top-k K ("ROWS,VOCAB,K"):
    greedy, and temperature 0.8 with top-p 1.0 and 0.9."""
    import torch
    from ..csrc import ops
    rows, vocab, k = (int(x) for x in spec.split(","))
    g = torch.Generator(device="cpu").manual_seed(0)
    logits = (torch.randn(rows, vocab, generator=g) * 0.6).cuda()
    out = torch.zeros(rows, dtype=torch.int32, device="cuda")
    temp = torch.full((rows,), 0.8, device="cuda")
    top_k = torch.full((rows,), k, dtype=torch.int32, device="cuda")
    seeds = torch.arange(rows, dtype=torch.int64, device="cuda")
    fresh = torch.ones(rows, dtype=torch.int32, device="cuda")
    slots = torch.arange(rows, dtype=torch.int32, device="cuda")
    states = torch.zeros(rows, dtype=torch.int64, device="cuda")
    res = {"greedy_us": round(_graph_time_us(lambda: ops.sample(out, logits, rows)), 2)}
    for p in (1.0, 0.9):
        top_p = torch.full((rows,), p, device="cuda")
        res[f"sampled_top_p_{p}_us"] = round(_graph_time_us(
            lambda: ops.sample(out, logits, rows, temperature=temp, top_k=top_k, top_p=top_p,
                               seeds=seeds, fresh=fresh, slots=slots, rng_states=states)), 2)
    if rows <= 64:
        # with a workspace every greedy row goes to several CTAs (what the engine's sampler runs)
        ws = torch.zeros(ops.sample_workspace_words(), dtype=torch.int32, device="cuda")
        res["several_ctas_greedy_us"] = round(_graph_time_us(
            lambda: ops.sample(out, logits, rows, workspace=ws)), 2)

    print(json.dumps({"profile_sample": spec, "mbytes": round(rows * vocab * 4 / 1e6, 2), **res}))
    return 0
