"""Trace replay: feeds given token ids through a model step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it loads the
model the way generation does and drives the same :class:`ModelRunner`, cache manager
and kernels.  Input: one JSON object a line on standard input,

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries``: for each request its next tokens and the places among them whose logits
are wanted; all entries of a step are one batch.  ``end``: requests that are finished
after this step; their pages and state slot are given back.  For a step in which
something is wanted, ``<out>/<step>.f32`` receives the logits ``[wanted, vocab]`` as
little-endian float32, in the order of the entries and of ``want``, and ``<out>/<step>.json``
names the rows: ``{"step": 0, "vocab": V, "rows": [[request, position], ...]}``.  After
every step ``done <step>`` is printed and flushed.

The model is a folder (``--model``) or, with ``--random SIZE --seed S``, a model of a named
size with seeded random weights, written to a temporary folder first and loaded from there
like any other.
"""
from __future__ import annotations

import argparse
import contextlib
import json
import os
import sys
from typing import List, Optional

import numpy as np


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", help="folder with config.json and model.safetensors")
    p.add_argument("--random", metavar="SIZE", help="instead of --model: a named size with random weights")
    p.add_argument("--seed", type=int, default=0, help="seed of --random")
    p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    p.add_argument("--out", required=True, help="folder for <step>.f32 files")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="most tokens live requests hold at any time (each rounded up to pages)")
    p.add_argument("--page-size", type=int, default=64)
    p.add_argument("--max-requests", type=int, default=4,
                   help="most requests that are live at a time (default 4)")
    p.add_argument("--device", default="cuda:0")
    return p


def main(argv: Optional[List[str]] = None) -> int:
    parser = build_parser()
    args = parser.parse_args(argv)
    if bool(args.model) == bool(args.random):
        parser.error("give exactly one of --model DIR and --random SIZE")
    if args.max_requests < 1:
        parser.error("--max-requests must be at least 1")
    from .batch import Entry
    from .loading import load_model, random_model_folder

    os.makedirs(args.out, exist_ok=True)
    page = args.page_size
    max_tokens = -(-args.max_tokens // page) * page
    with random_model_folder(args.random, args.seed, args.dtype) if args.random \
            else contextlib.nullcontext(args.model) as folder:
        lm = load_model(folder, dtype=args.dtype, device=args.device, page_size=page,
                        max_batched_tokens=max(max_tokens, page), max_requests=args.max_requests,
                        max_tokens=max_tokens)
    runner, cache = lm.runner, lm.cache
    vocab = lm.model.vocab
    live = {}                       # request -> tokens it holds
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries, rows = [], []
        for e in rec.get("entries", []):
            rid = e["id"]
            if rid not in live:
                if len(live) >= args.max_requests:
                    raise SystemExit(f"trace_run: step {step} brings request {rid!r} while "
                                     f"{len(live)} requests are live; --max-requests is "
                                     f"{args.max_requests}")
                cache.open(rid)
                live[rid] = 0
            entries.append(Entry(rid, [int(t) for t in e["tokens"]],
                                 [int(w) for w in e.get("want", [])]))
            rows.extend([rid, live[rid] + w] for w in entries[-1].want)
        if entries:
            logits = runner.step(entries)
            for e in entries:
                live[e.rid] += len(e.tokens)
            if logits.shape[0] > 0:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                tmp = os.path.join(args.out, f".{step}.f32.tmp")
                arr.tofile(tmp)
                os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
                tmp = os.path.join(args.out, f".{step}.json.tmp")
                with open(tmp, "w", encoding="utf-8") as fh:
                    json.dump({"step": step, "vocab": vocab, "rows": rows}, fh)
                os.replace(tmp, os.path.join(args.out, f"{step}.json"))
            runner.check_status()
        for rid in rec.get("end", []):
            if rid in live:
                cache.close(rid)
                del live[rid]
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
