"""Plain, slow GPT-2: whole sequences, no cache, one function per part.

This file is the oracle of the test-suite.  It shares no code with the engine: it
reads ``config.json`` with :mod:`json` and ``model.safetensors`` with the
``safetensors`` package, and uses torch on the CPU only as an array library.

It rests on the formulas of the reference, not on running it: the reference's GPT-2
is ``dev/examples/gpt2.clj`` (Clojure on the JVM, computing through the external
Raster library); neither a JVM nor Raster exists on the machines this suite runs on,
so its model code cannot be imported or compiled here.  Each function cites the lines
it restates.  Where the reference delegates to an external op (layer norm, attention,
GELU), the cited lines are the reference's own in-repo statement of the same formula.

Arithmetic is float32 by default (``dtype=torch.float64`` gives a higher-precision
check of the oracle itself).
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch


# ----------------------------------------------------------------------------- model
class PlainGPT2:
    """A model folder read into a dict of arrays (``gpt2.clj:172-217``)."""

    def __init__(self, folder: str, dtype: torch.dtype = torch.float32):
        from safetensors.torch import load_file
        with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as fh:
            self.config = json.load(fh)
        raw = load_file(os.path.join(folder, "model.safetensors"))
        self.w: Dict[str, torch.Tensor] = {}
        for name, t in raw.items():
            if name.startswith("transformer."):
                name = name[len("transformer."):]
            self.w[name] = t.to(dtype) if t.dtype.is_floating_point else t
        c = self.config
        self.dtype = dtype
        self.n_embd = int(c["n_embd"])
        self.n_layer = int(c["n_layer"])
        self.n_head = int(c["n_head"])
        # n_inner null -> 4 * n_embd (gpt2.clj:179)
        self.n_inner = int(c["n_inner"]) if c.get("n_inner") is not None else 4 * self.n_embd
        self.vocab_size = int(c["vocab_size"])
        self.n_positions = int(c["n_positions"])
        # The reference hard-codes 1e-5 (gpt2.clj:152,160,240); the key is honoured here.
        self.eps = float(c.get("layer_norm_epsilon", 1e-5))
        self.activation = c.get("activation_function", "gelu_new")
        self.scale_attn_weights = bool(c.get("scale_attn_weights", True))
        self.scale_by_inverse_layer = bool(c.get("scale_attn_by_inverse_layer_idx", False))


# ------------------------------------------------------------------------------ parts
def embeddings(wte: torch.Tensor, wpe: torch.Tensor, ids: Sequence[int]) -> torch.Tensor:
    """out[i,:] = wte[id_i,:] + wpe[i,:]  (``gpt2.clj:49-62``, formula ``:65``)."""
    ids = torch.as_tensor(list(ids), dtype=torch.long)
    if len(ids) > wpe.shape[0]:
        raise ValueError("sequence longer than n_positions")
    return wte[ids] + wpe[torch.arange(len(ids))]


def layer_norm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor,
               eps: float) -> torch.Tensor:
    """Per row: mean-centred, biased variance, 1/sqrt(var+eps), then gain and bias
    (call: ``gpt2.clj:152,160,240``; formula: ``src/pretrained/asr/moonshine.clj:87-104``)."""
    d = x.shape[-1]
    mean = x.sum(dim=-1, keepdim=True) / d
    centred = x - mean
    var = (centred * centred).sum(dim=-1, keepdim=True) / d
    inv = 1.0 / torch.sqrt(var + eps)
    return centred * inv * gamma + beta


def linear_conv1d(x: torch.Tensor, w_in_out: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """y = x . W + b with W stored Conv1D-style [in, out]; the reference transposes it to
    [out, in] and calls a linear (``gpt2.clj:27-36, 162, 164``)."""
    return x @ w_in_out + b


def gelu_new(u: torch.Tensor) -> torch.Tensor:
    """0.5 u (1 + tanh(sqrt(2/pi) (u + 0.044715 u^3)))  (``gpt2.clj:163`` calls nn/gelu,
    the tanh form)."""
    return 0.5 * u * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (u + 0.044715 * u * u * u)))


def gelu_erf(u: torch.Tensor) -> torch.Tensor:
    """0.5 u (1 + erf(u / sqrt 2)): the "erf-exact" form
    (``src/pretrained/asr/moonshine.clj:106-108``)."""
    return 0.5 * u * (1.0 + torch.erf(u / math.sqrt(2.0)))


def activation(name: str, u: torch.Tensor) -> torch.Tensor:
    if name in ("gelu_new", "gelu_pytorch_tanh"):
        return gelu_new(u)
    if name == "gelu":
        return gelu_erf(u)
    if name == "relu":
        return torch.clamp(u, min=0.0)
    raise ValueError(name)


def attention_scale(model: PlainGPT2, layer: int) -> float:
    """1/sqrt(head_dim) (``src/pretrained/decoder.clj:56``), and 1/(layer+1) on top when
    the configuration asks for inverse-layer scaling."""
    s = 1.0
    if model.scale_attn_weights:
        s /= math.sqrt(model.n_embd // model.n_head)
    if model.scale_by_inverse_layer:
        s /= float(layer + 1)
    return s


def causal_attention(x_ln: torch.Tensor, c_attn_w: torch.Tensor, c_attn_b: torch.Tensor,
                     c_proj_w: torch.Tensor, c_proj_b: torch.Tensor, n_head: int,
                     scale: float, window: Optional[int] = None) -> torch.Tensor:
    """Causal multi-head attention with biases and the output projection
    (``gpt2.clj:154-156``; QKV split: columns [0,d) Q, [d,2d) K, [2d,3d) V of the fused
    matrix, ``gpt2.clj:186-194``; token i sees keys j <= i; softmax over the visible
    keys; masked keys contribute exactly 0)."""
    t, d = x_ln.shape
    dh = d // n_head
    qkv = linear_conv1d(x_ln, c_attn_w, c_attn_b)
    q, k, v = qkv[:, :d], qkv[:, d:2 * d], qkv[:, 2 * d:]
    out = torch.zeros_like(x_ln)
    i = torch.arange(t).unsqueeze(1)
    j = torch.arange(t).unsqueeze(0)
    visible = j <= i
    if window is not None:
        visible = visible & (j > i - window)
    for h in range(n_head):
        cols = slice(h * dh, (h + 1) * dh)
        scores = (q[:, cols] @ k[:, cols].T) * scale
        scores = scores.masked_fill(~visible, -math.inf)      # exp(-inf) == 0 exactly
        out[:, cols] = torch.softmax(scores, dim=1) @ v[:, cols]
    return linear_conv1d(out, c_proj_w, c_proj_b)


def mlp(x_ln: torch.Tensor, fc_w, fc_b, proj_w, proj_b, act: str) -> torch.Tensor:
    """up -> activation -> down (``gpt2.clj:160-164``)."""
    return linear_conv1d(activation(act, linear_conv1d(x_ln, fc_w, fc_b)), proj_w, proj_b)


def block(model: PlainGPT2, layer: int, x: torch.Tensor) -> torch.Tensor:
    """x -> LN -> attention -> add -> LN -> MLP -> add (``gpt2.clj:139-166``)."""
    w, p = model.w, f"h.{layer}."
    a = causal_attention(
        layer_norm(x, w[p + "ln_1.weight"], w[p + "ln_1.bias"], model.eps),
        w[p + "attn.c_attn.weight"], w[p + "attn.c_attn.bias"],
        w[p + "attn.c_proj.weight"], w[p + "attn.c_proj.bias"],
        model.n_head, attention_scale(model, layer))
    x1 = x + a
    m = mlp(layer_norm(x1, w[p + "ln_2.weight"], w[p + "ln_2.bias"], model.eps),
            w[p + "mlp.c_fc.weight"], w[p + "mlp.c_fc.bias"],
            w[p + "mlp.c_proj.weight"], w[p + "mlp.c_proj.bias"], model.activation)
    return x1 + m


def forward(model: PlainGPT2, ids: Sequence[int]) -> torch.Tensor:
    """Hidden states after the final norm, [T, d] (``gpt2.clj:219-240``)."""
    x = embeddings(model.w["wte.weight"], model.w["wpe.weight"], ids)
    for layer in range(model.n_layer):
        x = block(model, layer, x)
    return layer_norm(x, model.w["ln_f.weight"], model.w["ln_f.bias"], model.eps)


def logits(model: PlainGPT2, hidden: torch.Tensor) -> torch.Tensor:
    """logits[i, v] = sum_d hidden[i, d] * wte[v, d]: the output head is tied to the token
    table (``gpt2.clj:108-122``; the reference computes the last row only)."""
    return hidden @ model.w["wte.weight"].T


def all_logits(model: PlainGPT2, ids: Sequence[int]) -> torch.Tensor:
    """[T, V] logits of a whole sequence."""
    return logits(model, forward(model, ids)).to(torch.float32)


def argmax(row: torch.Tensor) -> int:
    """First strictly greater wins, so ties go to the lowest id (``gpt2.clj:264-270``)."""
    best, best_score = 0, float(row[0])
    for i in range(1, row.shape[0]):
        s = float(row[i])
        if s > best_score:
            best, best_score = i, s
    return best


def greedy_generate(model: PlainGPT2, ids: Sequence[int], n: int) -> List[int]:
    """Re-runs the whole sequence for every new token (``gpt2.clj:249-271``); returns the
    new tokens only."""
    ids = list(ids)
    out: List[int] = []
    for _ in range(n):
        if len(ids) > model.n_positions:      # a step runs while its position < n_positions (decoder_gpu.clj:1302)
            break
        row = all_logits(model, ids)[-1]
        tok = int(torch.argmax(row))          # torch.argmax returns the first maximum
        assert tok == argmax(row), "the tie rule of the scalar argmax differs from torch.argmax"
        ids.append(tok)
        out.append(tok)
    return out


# --------------------------------------------------------------------------- sampling
class JavaRandom:
    """``java.util.Random`` as its documentation specifies it: a 48-bit linear
    congruential generator; ``nextDouble`` = ((next(26) << 27) + next(27)) * 2^-53.
    The reference's sampler draws from ``java.util.Random(seed)``
    (``src/pretrained/sampling.clj:43, 61``)."""

    MULT = 0x5DEECE66D
    MASK = (1 << 48) - 1

    def __init__(self, seed: int):
        self.state = (int(seed) ^ self.MULT) & self.MASK

    def next(self, bits: int) -> int:
        self.state = (self.state * self.MULT + 0xB) & self.MASK
        return self.state >> (48 - bits)

    def next_double(self) -> float:
        return ((self.next(26) << 27) + self.next(27)) * (1.0 / (1 << 53))


def top_k_ids(row: torch.Tensor, k: int) -> List[int]:
    """Indices of the k largest logits in descending order; among equal logits the
    lower index comes first (bounded insertion, ``sampling.clj:14-29``)."""
    k = min(k, row.shape[0])
    ids = [0] * k
    vals = [-math.inf] * k
    for i in range(row.shape[0]):
        v = float(row[i])
        if v > vals[k - 1]:
            j = k - 1
            while j > 0 and vals[j - 1] < v:
                vals[j], ids[j] = vals[j - 1], ids[j - 1]
                j -= 1
            vals[j], ids[j] = v, i
    return ids


def sample(row: torch.Tensor, temperature: float, top_k: Optional[int], top_p: Optional[float],
           rng: Optional[JavaRandom]) -> int:
    """top-k -> softmax(logit / T) in double -> nucleus cut -> multinomial draw
    (``sampling.clj:31-64``).  temperature <= 0 is greedy (``:37-38``); top-k defaults to
    40 (``:41``), top-p to 1.0 (``:42``)."""
    if temperature is None or temperature <= 0.0:
        return argmax(row)
    k = 40 if top_k is None else int(top_k)
    p = 1.0 if top_p is None else float(top_p)
    kk = min(k, row.shape[0])
    ids = top_k_ids(row, kk)
    mx = float(row[ids[0]]) / temperature
    probs = [math.exp(float(row[i]) / temperature - mx) for i in ids]
    psum = 0.0
    for q in probs:
        psum += q
    cut, c = kk, 0.0
    for j in range(kk):
        c += probs[j] / psum
        if c >= p:
            cut = j + 1
            break
    tot = 0.0
    for j in range(cut):
        tot += probs[j]
    r = rng.next_double() * tot
    acc = 0.0
    for j in range(cut):
        acc += probs[j]
        if acc >= r or j == cut - 1:
            return ids[j]
    return ids[cut - 1]


def sample_generate(model: PlainGPT2, ids: Sequence[int], n: int, temperature: float,
                    top_k: Optional[int], top_p: Optional[float], seed: int) -> List[int]:
    rng = JavaRandom(seed)
    ids = list(ids)
    out: List[int] = []
    for _ in range(n):
        if len(ids) > model.n_positions:      # a step runs while its position < n_positions (decoder_gpu.clj:1302)
            break
        tok = sample(all_logits(model, ids)[-1], temperature, top_k, top_p, rng)
        ids.append(tok)
        out.append(tok)
    return out
