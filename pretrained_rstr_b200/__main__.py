"""Command line: ``python -m pretrained_rstr_b200 <command> ...``; one JSON object on
standard output, like the reference's benchmark mains
(``dev/pretrained/laya_cpu_benchmark.clj:73-80``).

  generate  (--model DIR | --random SIZE [--weights-seed S]) --ids 5,17,3 --n 16
            [--temperature T --top-k K --top-p P --seed S]
  random    --out DIR (--config FILE.json | --size NAME) --seed S [--dtype float32|bfloat16]
  replay    (--model DIR | --random SIZE [--seed S]) --dtype D --out DIR --max-tokens N
            (the same program as bin/trace_run)
  bench     [--steps K --warmup W --size small|medium|xl --workload decode|mixed ...]
            (the benchmark beside the package, ``bench.py``; one JSON line)
"""
from __future__ import annotations

import argparse
import json
import sys

def _generate(args) -> int:
    from . import generate_ids, load_lm
    import contextlib
    from .engine.loading import random_model_folder
    if bool(args.model) == bool(args.random):
        raise SystemExit("generate: give exactly one of --model DIR and --random SIZE")
    ids = [int(t) for t in args.ids.replace(",", " ").split()]
    with random_model_folder(args.random, args.weights_seed, args.dtype) if args.random \
            else contextlib.nullcontext(args.model) as folder:
        m = load_lm(folder, gpu=args.gpu, dtype=args.dtype, device_id=args.device_id,
                    maxpos=args.maxpos, max_lanes=args.max_lanes)
    opts = {}
    if args.temperature is not None:
        opts = {"temperature": args.temperature, "top_k": args.top_k, "top_p": args.top_p,
                "seed": args.seed}
    out = generate_ids(m, ids, args.n, opts)
    print(json.dumps({"prompt": ids, "generated": out, "stats": m.stats()}))
    return 0


def _random(args) -> int:
    import torch
    from .config.registry import lookup, named_size
    from .weights import make_random_model
    if args.config:
        with open(args.config, "r", encoding="utf-8") as fh:
            raw = json.load(fh)
        cfg = lookup(raw).config_class.from_dict(raw)
    else:
        _arch, cfg = named_size(args.size)
    make_random_model(args.out, cfg, args.seed,
                      torch.bfloat16 if args.dtype == "bfloat16" else torch.float32)
    print(json.dumps({"out": args.out, "seed": args.seed, "config": cfg.to_dict()}))
    return 0


def _bench(argv) -> int:
    """Run ``bench.py`` (it lies beside the package folder) with the given arguments."""
    import os
    import runpy
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py")
    if not os.path.isfile(path):
        raise SystemExit(f"bench: {path} not found (the benchmark ships beside the package)")
    saved = sys.argv
    sys.argv = [path] + list(argv)
    try:
        runpy.run_path(path, run_name="__main__")
    except SystemExit as exc:
        return int(exc.code or 0)
    finally:
        sys.argv = saved
    return 0


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="pretrained_rstr_b200")
    sub = p.add_subparsers(dest="command", required=True)
    g = sub.add_parser("generate", help="generate token ids from prompt token ids")
    g.add_argument("--model", help="folder with config.json and model.safetensors")
    g.add_argument("--random", metavar="SIZE", help="instead of --model: a named size with random weights")
    g.add_argument("--weights-seed", type=int, default=0, help="seed of --random's weights")
    g.add_argument("--ids", required=True, help="prompt token ids, comma or space separated")
    g.add_argument("--n", type=int, default=16)
    g.add_argument("--temperature", type=float, default=None, help="absent or <= 0: greedy")
    g.add_argument("--top-k", type=int, default=None, help="default 40 when sampling")
    g.add_argument("--top-p", type=float, default=None, help="default 1.0")
    g.add_argument("--seed", type=int, default=None)
    g.add_argument("--gpu", action=argparse.BooleanOptionalAction, default=True)
    g.add_argument("--device-id", default="cuda:0")
    g.add_argument("--maxpos", type=int, default=None)
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    g.add_argument("--max-lanes", type=int, default=4)
    g.set_defaults(fn=_generate)
    r = sub.add_parser("random", help="write a model folder with seeded random weights")
    r.add_argument("--out", required=True)
    r.add_argument("--config")
    r.add_argument("--size", default="tiny-a", help="a named size (tiny-a, tiny-b, small, medium, xl)")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--dtype", default="float32", choices=["bfloat16", "float32"])
    r.set_defaults(fn=_random)
    t = sub.add_parser("replay", help="trace replay (see bin/trace_run)", add_help=False)
    t.set_defaults(fn=None)
    b = sub.add_parser("bench", help="the benchmark (bench.py beside the package)", add_help=False)
    b.set_defaults(fn=None)
    if argv is None:
        argv = sys.argv[1:]
    if argv and argv[0] == "replay":
        from .engine.trace import main as trace_main
        return trace_main(argv[1:])
    if argv and argv[0] == "bench":
        return _bench(argv[1:])
    args = p.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
