"""Shared by the tests: the two tiny configurations, model folders in temporary
directories, a replayer that drives the engine's step function the way bin/trace_run
does, and the comparison with the plain implementation."""
from __future__ import annotations

import os
import random
from typing import Dict, List, Sequence, Tuple

import torch

import plain_gpt2

# Two tiny GPT-2 configurations that differ in every size and option.
TINY_A = {
    "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2",
    "n_layer": 2, "n_embd": 64, "n_head": 4, "n_inner": 256, "vocab_size": 512,
    "n_positions": 128, "layer_norm_epsilon": 1e-5, "activation_function": "gelu_new",
    "scale_attn_weights": True, "scale_attn_by_inverse_layer_idx": False,
}
TINY_B = {
    "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2",
    "n_layer": 3, "n_embd": 96, "n_head": 3, "n_inner": 320, "vocab_size": 1000,
    "n_positions": 256, "layer_norm_epsilon": 1e-6, "activation_function": "gelu",
    "scale_attn_weights": True, "scale_attn_by_inverse_layer_idx": True,
}
# A third one with the head size (64) and widths (multiples of 64) that the tcgen05 prompt
# attention and the TMA decode product take, and contexts of several 128-query tiles.
TINY_C = {
    "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2",
    "n_layer": 2, "n_embd": 128, "n_head": 2, "n_inner": 448, "vocab_size": 700,
    "n_positions": 512, "layer_norm_epsilon": 1e-5, "activation_function": "gelu_new",
    "scale_attn_weights": True, "scale_attn_by_inverse_layer_idx": False,
}
TINY = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 2)}


def real_width(name: str) -> Dict:
    """The layer sizes of GPT-2 small, medium and XL (width, heads, inner width, vocabulary,
    positions) with two layers: fewer layers, not smaller ones, so that the engine runs the
    very kernel instances, tile widths and splits it runs at those sizes."""
    d, h = {"small": (768, 12), "medium": (1024, 16), "xl": (1600, 25)}[name]
    return {"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2", "n_layer": 2,
            "n_embd": d, "n_head": h, "n_inner": 4 * d, "vocab_size": 50257, "n_positions": 1024,
            "layer_norm_epsilon": 1e-5, "activation_function": "gelu_new",
            "scale_attn_weights": True, "scale_attn_by_inverse_layer_idx": False}


def bf16_atol(width: int) -> float:
    """bfloat16 tolerance on logits for a model of this width.  Between two products the
    activations are rounded to 8 bits of mantissa (relative error up to 2^-9); a logit is a sum
    over ``width`` such terms against table entries of standard deviation 0.02, so its error
    grows like sqrt(width), and the largest among ten thousands of logits is several standard
    deviations out.  6e-4 * sqrt(width): 4.8e-3 at 64, 1.7e-2 at 768, 2.4e-2 at 1,600 (the
    tiny configurations keep their fixed 1.5e-2)."""
    return 6e-4 * width ** 0.5

# Absolute tolerance on logits.  Random-weight logits are O(0.2); float32 differences
# come from summation order only; bfloat16 ones from rounding activations to 8 bits
# of mantissa between products.
ATOL = {"float32": 3e-5, "bfloat16": 1.5e-2}


def make_folder(path: str, raw: Dict, seed: int, dtype: str) -> str:
    from pretrained_rstr_b200.config import GPT2Config
    from pretrained_rstr_b200.weights import make_random_model
    cfg = GPT2Config.from_dict(raw)
    make_random_model(path, cfg, seed,
                      torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    return path


def random_tokens(n: int, vocab: int, seed: int) -> List[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


class Replayer:
    """Feeds steps to a loaded model like bin/trace_run and collects logits by
    (request, position)."""

    def __init__(self, folder: str, dtype: str, max_tokens: int, page_size: int = 64, **kw):
        from pretrained_rstr_b200.engine.loading import load_model
        max_tokens = -(-max_tokens // page_size) * page_size
        self.lm = load_model(folder, dtype=dtype, page_size=page_size,
                             max_batched_tokens=kw.pop("max_batched_tokens", max(max_tokens, 64)),
                             max_requests=kw.pop("max_requests", 4), max_tokens=max_tokens, **kw)
        self.pos: Dict[str, int] = {}
        self.rows: Dict[Tuple[str, int], torch.Tensor] = {}

    def step(self, entries: Sequence[Tuple[str, Sequence[int], Sequence[int]]], end=()):
        from pretrained_rstr_b200.engine.batch import Entry
        batch = []
        for rid, tokens, want in entries:
            if rid not in self.pos:
                self.lm.cache.open(rid)
                self.pos[rid] = 0
            batch.append(Entry(rid, list(tokens), list(want)))
        logits = self.lm.runner.step(batch).to("cpu")
        self.lm.runner.check_status()
        r = 0
        for rid, tokens, want in entries:
            for w in want:
                self.rows[(rid, self.pos[rid] + w)] = logits[r].clone()
                r += 1
            self.pos[rid] += len(tokens)
        for rid in end:
            self.lm.cache.close(rid)
            del self.pos[rid]
        self.lm.cache.check()


def compare(rows: Dict[Tuple[str, int], torch.Tensor], oracle: Dict[str, torch.Tensor],
            atol: float) -> float:
    """Every collected row against the plain implementation's row of the same
    (request, position); returns the largest difference and names the first bad token."""
    worst = 0.0
    for (rid, pos), row in sorted(rows.items()):
        ref = oracle[rid][pos]
        err = float((row - ref).abs().max())
        assert err == err, f"NaN at request {rid} position {pos}"
        assert err <= atol, (f"request {rid} position {pos}: max |difference| {err:.3e} > {atol:.1e} "
                             f"(page offset {pos % 64}, argmax {int(row.argmax())} vs "
                             f"{int(ref.argmax())})")
        worst = max(worst, err)
    return worst


def oracle_rows(folder: str, prompts: Dict[str, Sequence[int]],
                wanted: Dict[str, Sequence[int]]) -> Dict[str, Dict[int, torch.Tensor]]:
    """The plain implementation's logits at chosen positions only (large vocabularies): the
    whole sequence runs, the head is applied to the wanted rows."""
    model = plain_gpt2.PlainGPT2(folder)
    out = {}
    for rid, ids in prompts.items():
        hidden = plain_gpt2.forward(model, ids)
        pos = sorted(set(wanted[rid]))
        rows = plain_gpt2.logits(model, hidden[pos]).to(torch.float32)
        out[rid] = {p: rows[i] for i, p in enumerate(pos)}
    return out


def oracle_logits(folder: str, prompts: Dict[str, Sequence[int]]) -> Dict[str, torch.Tensor]:
    model = plain_gpt2.PlainGPT2(folder)
    return {rid: plain_gpt2.all_logits(model, ids) for rid, ids in prompts.items()}
