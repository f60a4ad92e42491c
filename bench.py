#!/usr/bin/env python3
"""Benchmark: decode tokens/s (batch 8 by default) and prefill tokens/s at 2,048 tokens
for GPT-2 small with random weights, each with its fraction of the roofline.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]
    python bench.py --workload mixed [--size medium] [--pool-fraction 0.4]

Prints ONE JSON line.  A "step" is one decode step of the whole batch.  ``value`` is
decoded tokens per second from device time (CUDA events around each step's kernels);
``e2e`` is the same through the engine's public step (token ids from pinned host memory
in, sampled ids read back to the host, every step).  ``prefill`` is one step of 2,048
prompt tokens (2 prompts x 1,024).  ``roofline`` divides the bytes a decode step has to
read (every weight once, and the cache of the live requests) by its time and by the
measured copy bandwidth.  ``points`` holds the other batch sizes (1 and 64) at the same
context and all three at a mean context of 256 (128-token prompts, 256 generated tokens),
each device-timed and end to end, and decoding with temperature sampling.  Weights (247 MB)
plus cache are larger than the 126 MB L2, so no flush is needed between timed steps.

``--workload mixed`` runs many requests of unequal length through the scheduler (prompts
uniform in [16, 1024), portions of 512 beside decoding requests, 30 % sharing a 256-token
prefix) and reports times to first token, step times by kind and the cache's counters.

The code that measures lives in ``pretrained_rstr_b200/measure/``; the ``--profile-*``
options run its small single-kernel workloads (for profiler captures).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from pretrained_rstr_b200.measure.roofline import (SIZES, ClockSampler, kv_bytes_per_token,  # noqa: E402
                                                   model_bytes, peaks, prefill_flops, quantiles)


def run_reference(args) -> int:
    print(json.dumps({
        "impl": "reference",
        "unavailable": "replikativ/pretrained-rstr is Clojure on the JVM computing through the "
                       "external Raster library; pip reports that its folder is not installable "
                       "(neither setup.py nor pyproject.toml found), and no JVM, Clojure or Raster "
                       "exists offline"}))
    return 0


def load_bench_model(size: str, layers, max_tokens=None, prefill_chunk=1024, share_prefixes=False):
    import tempfile
    import shutil
    import torch
    from pretrained_rstr_b200 import load_lm
    from pretrained_rstr_b200.config import GPT2Config
    from pretrained_rstr_b200.weights import make_random_model
    raw = dict(SIZES[size])
    full_layers = raw["n_layer"]
    if layers:
        raw["n_layer"] = layers
    cfg = GPT2Config.from_dict(raw)
    tmp = tempfile.mkdtemp(prefix="prb200_bench_")
    try:
        make_random_model(tmp, cfg, seed=2, dtype=torch.bfloat16)
        m = load_lm(tmp, gpu=True, dtype="bfloat16", max_lanes=64, max_batched_tokens=2048,
                    prefill_chunk=prefill_chunk, share_prefixes=share_prefixes,
                    max_tokens=max_tokens)
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    return m, raw, full_layers


def run_mixed(args) -> int:
    """The mixed workload: one JSON line."""
    # Every kernel instance is loaded when the library is (the driver's default loads an
    # instance at its first launch, a stall of milliseconds that a server meets once per
    # instance and this short run would meet inside its timed pass: 17.9 k to 21.4 k generated
    # tokens/s from run to run at GPT-2 medium sizes without this, 20.6 k to 21.4 k with it).
    # Must be set before the process's first CUDA call.
    os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")
    from pretrained_rstr_b200.measure.workloads import mixed_workload
    raw = dict(SIZES[args.size])
    per_request = -(-raw["n_positions"] // 64) * 64
    max_tokens = int(64 * per_request * args.pool_fraction)
    m, raw, full_layers = load_bench_model(args.size, args.layers, max_tokens=max_tokens,
                                           prefill_chunk=512, share_prefixes=True)
    with ClockSampler() as clocks:
        for _ in range(max(1, args.warmup // 3)):       # untimed passes: graphs, scratch, index
            mixed_workload(m.engine, raw["vocab_size"], n_requests=8, max_new=16, seed=99)
        # and one of the timed size with other prompts: a server has met its shapes before
        mixed_workload(m.engine, raw["vocab_size"], n_requests=args.requests,
                       max_new=args.max_new, seed=5)
        res = mixed_workload(m.engine, raw["vocab_size"], n_requests=args.requests,
                             max_new=args.max_new, seed=4)
    print(json.dumps({
        "metric": f"mixed workload (GPT-2 {args.size}, random weights)", "workload": "mixed",
        "value": res["generated_tokens_per_s"], "unit": "generated tokens/s", "n_gpus": 1,
        "dtype": "bf16", "data": "synthetic", "higher_is_better": True,
        "config": {"model": f"gpt2-{args.size}-random", "n_layer": raw["n_layer"],
                   "n_layer_full": full_layers, "n_embd": raw["n_embd"], "n_head": raw["n_head"],
                   "n_inner": raw["n_inner"], "vocab_size": raw["vocab_size"],
                   "requests": args.requests, "prompts": "uniform [16, 1024)", "prefill_chunk": 512,
                   "shared_prefix": 256, "shared_fraction": 0.3, "max_new": args.max_new,
                   "pool_fraction": args.pool_fraction, "page_size": 64,
                   "module_loading": os.environ.get("CUDA_MODULE_LOADING", "")},
        **res, "clocks": clocks.summary()}))
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
    ap.add_argument("--profile-host", type=int, default=None, metavar="BATCH",
                    help="the host's side of a decode step: wall time a step with a one-layer model, cProfile shares")
    ap.add_argument("--profile-decode-attention", default=None, metavar="HEADS,REQUESTS,CONTEXT",
                    help="the decode attention kernel alone, by split size")
    ap.add_argument("--profile-sample", default=None, metavar="ROWS,VOCAB,K",
                    help="the sampling kernel alone")
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
    ap.add_argument("--workload", default="decode", choices=["decode", "mixed"])
    ap.add_argument("--requests", type=int, default=64, help="mixed workload: requests")
    ap.add_argument("--max-new", type=int, default=128, help="mixed workload: tokens generated per request")
    ap.add_argument("--pool-fraction", type=float, default=1.0,
                    help="mixed workload: the page pool as a fraction of 64 full-length requests")
    ap.add_argument("--temperature", type=float, default=None,
                    help="decode with temperature sampling (top-k 40) instead of greedy")
    ap.add_argument("--quick", action="store_true", help="only the headline point and the prefill")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    from pretrained_rstr_b200.measure import profiles
    if args.profile_gemm:
        return profiles.profile_gemm(args.profile_gemm)
    if args.profile_host:
        return profiles.profile_host(args.profile_host)
    if args.profile_decode:
        return profiles.profile_decode(args.profile_decode, args.kernel_table)
    if args.profile_prefill:
        return profiles.profile_prefill(not args.no_table)
    if args.profile_prompt:
        return profiles.profile_prompt(args.profile_prompt, not args.no_table)
    if args.profile_attention:
        return profiles.profile_attention(args.profile_attention)
    if args.profile_decode_attention:
        return profiles.profile_decode_attention(args.profile_decode_attention)
    if args.profile_sample:
        return profiles.profile_sample(args.profile_sample)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.workload == "mixed":
        return run_mixed(args)

    from pretrained_rstr_b200.engine.scheduler import SamplingParams
    from pretrained_rstr_b200.measure.workloads import timed_decode, timed_prefill

    m, raw, full_layers = load_bench_model(args.size, args.layers)
    pk = peaks()
    vocab = raw["vocab_size"]
    steps, warmup, ctx_len = args.steps, args.warmup, min(args.context, raw["n_positions"])
    steps = max(1, min(steps, ctx_len - warmup - 64 - 3 - 16))     # every request must fit its context
    engine = m.engine
    sampling = None if args.temperature is None else \
        SamplingParams(temperature=args.temperature, seed=7)

    # ---- prefill: one step of 2 x 1024 prompt tokens
    pre = statistics.median(timed_prefill(m.loaded, 2, 1024, vocab))
    flops = prefill_flops(raw, 2, 1024)
    prefill = {"value": 2048 / (pre / 1e3), "tokens": 2048, "ms": pre,
               "frac": flops / (pre / 1e3) / (pk["bf16_tflops"] * 1e12)}

    def frac(batch, res):
        step_ms = statistics.mean(res["ms"])
        nbytes = model_bytes(raw) + batch * res["mean_context"] * kv_bytes_per_token(raw)
        return nbytes / (step_ms / 1e3) / 1e9 / pk["hbm_gbs"]

    # ---- decode
    points = {}
    clocks = ClockSampler()
    clocks.__enter__()
    if not args.quick:
        short = min(ctx_len, 256 + steps // 2)       # mean context 256: 128-token prompts, 256 generated
        for b, ctx, tag in [(1, ctx_len, ""), (64, ctx_len, ""), (1, short, "_ctx256"),
                            (8, short, "_ctx256"), (64, short, "_ctx256")]:
            if tag:
                # these contexts cross a boundary at which the step's graph changes (256
                # keys): an untimed pass of the same lengths first, so that the timed one
                # meets no shape for the first time, as in a server that has run for a while
                timed_decode(engine, b, ctx, steps, warmup, vocab, 999 * b + ctx, sampling)
            res = timed_decode(engine, b, ctx, steps, warmup, vocab, 1000 * b + ctx, sampling)
            name = f"decode_b{b}{tag}"
            points[name] = b / (statistics.mean(res["ms"]) / 1e3)
            points[name + "_ms"] = round(statistics.median(res["ms"]), 4)
            points[name + "_e2e"] = b * steps / res["wall_s"]
            points[name + "_hbm_frac"] = round(frac(b, res), 4)
        if sampling is None:
            res = timed_decode(engine, args.batch, ctx_len, steps, warmup, vocab, 77,
                               SamplingParams(temperature=0.8, seed=7))
            points[f"decode_b{args.batch}_sampled_t0.8_k40"] = args.batch / (statistics.mean(res["ms"]) / 1e3)
    res = timed_decode(engine, args.batch, ctx_len, steps, warmup, vocab, 5, sampling)
    clocks.__exit__(None, None, None)
    step_ms = statistics.mean(res["ms"])
    value = args.batch / (step_ms / 1e3)
    achieved = frac(args.batch, res) * pk["hbm_gbs"]
    record = {
        "metric": f"decode tok/s (GPT-2 {args.size}, random weights)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"model": f"gpt2-{args.size}-random", "global_batch": args.batch, "seq_len": ctx_len,
                   "parallelism": "single-gpu", "n_layer": raw["n_layer"], "n_layer_full": full_layers,
                   "n_embd": raw["n_embd"], "n_head": raw["n_head"], "n_inner": raw["n_inner"],
                   "vocab_size": vocab, "n_positions": raw["n_positions"], "page_size": 64,
                   "mean_context": res["mean_context"], "l2": "inputs_exceed_l2",
                   "peaks": pk["source"],
                   "sampling": "greedy" if sampling is None else f"temperature {args.temperature}"},
        "e2e": {"value": args.batch * steps / res["wall_s"], "unit": "tokens/s",
                "h2d_bytes_per_step": res["h2d_bytes"], "d2h_bytes_per_step": res["d2h_bytes"]},
        "gpu_launches": res["launches"],
        "step_ms": quantiles(res["ms"]),
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
