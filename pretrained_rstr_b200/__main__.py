"""Command line: ``python -m pretrained_rstr_b200 <command> ...``; one JSON object on
standard output, like the reference's benchmark mains
(``dev/pretrained/laya_cpu_benchmark.clj:73-80``).

  generate  --model DIR --ids 5,17,3 --n 16 [--temperature T --top-k K --top-p P --seed S]
  random    --out DIR (--config FILE.json | --size NAME) --seed S [--dtype float32|bfloat16]
  replay    --model DIR --dtype D --out DIR --max-tokens N      (same as bin/trace_run)
"""
from __future__ import annotations

import argparse
import json
import sys

SIZES = {
    "tiny-a": dict(n_layer=2, n_embd=64, n_head=4, n_inner=256, vocab_size=512, n_positions=128),
    "tiny-b": dict(n_layer=3, n_embd=96, n_head=3, n_inner=320, vocab_size=1000, n_positions=256,
                   layer_norm_epsilon=1e-6, activation_function="gelu",
                   scale_attn_by_inverse_layer_idx=True),
    "small": dict(n_layer=12, n_embd=768, n_head=12, n_inner=3072, vocab_size=50257,
                  n_positions=1024),
    "medium": dict(n_layer=24, n_embd=1024, n_head=16, n_inner=4096, vocab_size=50257,
                   n_positions=1024),
    "xl": dict(n_layer=48, n_embd=1600, n_head=25, n_inner=6400, vocab_size=50257,
               n_positions=1024),
}


def _generate(args) -> int:
    from . import generate_ids, load_lm
    ids = [int(t) for t in args.ids.replace(",", " ").split()]
    m = load_lm(args.model, gpu=args.gpu, dtype=args.dtype, device_id=args.device_id,
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
    from .config import GPT2Config
    from .config.registry import lookup
    from .weights import make_random_model
    if args.config:
        with open(args.config, "r", encoding="utf-8") as fh:
            raw = json.load(fh)
    else:
        raw = {"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2", **SIZES[args.size]}
    cfg = lookup(raw).config_class.from_dict(raw)
    make_random_model(args.out, cfg, args.seed,
                      torch.bfloat16 if args.dtype == "bfloat16" else torch.float32)
    print(json.dumps({"out": args.out, "seed": args.seed, "config": cfg.to_dict()}))
    return 0


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="pretrained_rstr_b200")
    sub = p.add_subparsers(dest="command", required=True)
    g = sub.add_parser("generate", help="generate token ids from prompt token ids")
    g.add_argument("--model", required=True)
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
    r.add_argument("--size", choices=sorted(SIZES), default="tiny-a")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--dtype", default="float32", choices=["bfloat16", "float32"])
    r.set_defaults(fn=_random)
    t = sub.add_parser("replay", help="trace replay (see bin/trace_run)", add_help=False)
    t.set_defaults(fn=None)
    if argv is None:
        argv = sys.argv[1:]
    if argv and argv[0] == "replay":
        from .engine.trace import main as trace_main
        return trace_main(argv[1:])
    args = p.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
