"""Trace replay: feeds given token ids through a model step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it loads the
model the way generation does and drives the same :class:`ModelRunner`, cache manager
and kernels.  Input: one JSON object a line on standard input,

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries``: for each request its next tokens and the places among them whose logits
are wanted; all entries of a step are one batch.  ``end``: requests that are finished
after this step; their pages and state slot are given back.  For a step in which
something is wanted, ``<out>/<step>.f32`` receives the logits ``[wanted, vocab]`` as
little-endian float32, in the order of the entries and of ``want``.  After every step
``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Optional

import numpy as np


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    p.add_argument("--out", required=True, help="folder for <step>.f32 files")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="most tokens live requests hold at any time (each rounded up to pages)")
    p.add_argument("--page-size", type=int, default=64)
    p.add_argument("--device", default="cuda:0")
    return p


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    from .batch import Entry
    from .loading import load_model
    from ..config.registry import read_config

    os.makedirs(args.out, exist_ok=True)
    _arch, config = read_config(args.model)
    page = args.page_size
    max_tokens = -(-args.max_tokens // page) * page
    lm = load_model(args.model, dtype=args.dtype, device=args.device, page_size=page,
                    max_batched_tokens=max(max_tokens, page), max_requests=4,
                    max_tokens=max_tokens)
    runner, cache = lm.runner, lm.cache
    live = set()
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if rid not in live:
                cache.open(rid)
                live.add(rid)
            entries.append(Entry(rid, [int(t) for t in e["tokens"]],
                                 [int(w) for w in e.get("want", [])]))
        if entries:
            logits = runner.step(entries)
            if logits.shape[0] > 0:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                tmp = os.path.join(args.out, f".{step}.f32.tmp")
                arr.tofile(tmp)
                os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
            runner.check_status()
        for rid in rec.get("end", []):
            if rid in live:
                cache.close(rid)
                live.remove(rid)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
