"""Each part alone against the plain implementation's function for that part, and the
generality of the assembly: a toy architecture defined here (a mixer with state of its
own in one layer, attention in another, a layer that runs twice and reads a cache
another run wrote) is registered, built and stepped without touching the framework."""
import math
import os
from dataclasses import dataclass
from typing import Dict

import pytest
import torch

import plain_gpt2
from helpers import ATOL, TINY, make_folder, random_tokens

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def loaded(tmp_path_factory):
    from pretrained_rstr_b200.engine.loading import load_model
    out = {}
    for name, (raw, seed) in TINY.items():
        for dtype in DTYPES:
            folder = make_folder(str(tmp_path_factory.mktemp(f"p{name}{dtype}")), raw, seed, dtype)
            out[(name, dtype)] = (load_model(folder, dtype=dtype, max_batched_tokens=256,
                                             max_requests=4, max_tokens=1024),
                                  plain_gpt2.PlainGPT2(folder))
    return out


def _ctx(lm, lengths, rid0=0):
    """A prepared step of whole prompts of the given lengths (reservation left pending)."""
    from pretrained_rstr_b200.engine.batch import Entry
    entries = []
    for i, n in enumerate(lengths):
        rid = f"part{rid0}_{i}"
        lm.cache.open(rid)
        entries.append(Entry(rid, random_tokens(n, lm.model.vocab, i), [n - 1]))
    ctx = lm.runner.prepare(entries)
    lm.runner.upload(ctx)                       # the step's arrays go to the device
    return ctx, entries


def _done(lm, entries):
    lm.runner.abort(entries)
    for e in entries:
        lm.cache.close(e.rid)


def _tol(dtype, scale=1.0):
    return (2e-5 if dtype == "float32" else 2e-2) * max(1.0, scale)


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_embedding_head_parts(loaded, name, dtype):
    lm, plain = loaded[(name, dtype)]
    ctx, entries = _ctx(lm, [7, 33])
    t, d = 40, lm.model.width
    act = lm.runtime.dtype
    x = torch.randn(t, d, device="cuda") * 2 + 0.3
    # norm
    out = torch.zeros(t, d, device="cuda", dtype=act)
    lm.model.blocks[1].mixer_norm.forward(ctx, x, out)
    ref = plain_gpt2.layer_norm(x.cpu(), plain.w["h.1.ln_1.weight"], plain.w["h.1.ln_1.bias"], plain.eps)
    assert float((out.float().cpu() - ref).abs().max()) <= _tol(dtype, float(ref.abs().max()))
    # embedding + learned positions
    emb = torch.zeros(t, d, device="cuda")
    lm.model.embedding.forward(ctx, lm.model.position, emb)
    toks = [tk for e in entries for tk in e.tokens]
    ref = torch.cat([plain_gpt2.embeddings(plain.w["wte.weight"], plain.w["wpe.weight"], e.tokens)
                     for e in entries])
    assert float((emb.cpu() - ref).abs().max()) <= 1e-6
    # tied head
    h = (torch.randn(5, d, device="cuda")).to(act)
    logits = torch.zeros(5, lm.model.vocab, device="cuda")
    lm.model.head.forward(ctx, h, logits)
    ref = h.float().cpu() @ plain.w["wte.weight"].T
    assert float((logits.cpu() - ref).abs().max()) <= _tol(dtype) * 0.5
    _done(lm, entries)


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens", [5, 100])        # decode-time and prompt-time products
def test_feed_forward_part(loaded, name, dtype, tokens):
    lm, plain = loaded[(name, dtype)]
    ctx, entries = _ctx(lm, [tokens], rid0=1)
    d = lm.model.width
    h = torch.randn(tokens, d, device="cuda").to(lm.runtime.dtype)
    x0 = torch.randn(tokens, d, device="cuda")
    x = x0.clone()
    lm.model.blocks[0].feed_forward.forward(ctx, h, x)
    w = plain.w
    ref = x0.cpu() + plain_gpt2.mlp(h.float().cpu(), w["h.0.mlp.c_fc.weight"], w["h.0.mlp.c_fc.bias"],
                                    w["h.0.mlp.c_proj.weight"], w["h.0.mlp.c_proj.bias"],
                                    plain.activation)
    assert float((x.cpu() - ref).abs().max()) <= _tol(dtype)
    _done(lm, entries)


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_mixer_part(loaded, name, dtype):
    """Whole prompts of two requests through the mixer alone: projections, cache append,
    attention over the pages, output projection, residual."""
    lm, plain = loaded[(name, dtype)]
    lengths = [70, 3]
    ctx, entries = _ctx(lm, lengths, rid0=2)
    d = lm.model.width
    layer = lm.model.config.n_layer - 1
    h = torch.randn(sum(lengths), d, device="cuda").to(lm.runtime.dtype)
    x = torch.zeros(sum(lengths), d, device="cuda")
    lm.model.blocks[layer].mixer.forward(ctx, h, x, lm.model._caches[layer])
    w, p = plain.w, f"h.{layer}."
    at = 0
    for n in lengths:
        ref = plain_gpt2.causal_attention(
            h[at:at + n].float().cpu(), w[p + "attn.c_attn.weight"], w[p + "attn.c_attn.bias"],
            w[p + "attn.c_proj.weight"], w[p + "attn.c_proj.bias"], plain.n_head,
            plain_gpt2.attention_scale(plain, layer))
        assert float((x[at:at + n].cpu() - ref).abs().max()) <= _tol(dtype)
        at += n
    _done(lm, entries)


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_part(loaded, dtype):
    lm, plain = loaded[("B", dtype)]
    ctx, entries = _ctx(lm, [50], rid0=3)
    x0 = torch.randn(50, lm.model.width, device="cuda")
    x = x0.clone()
    lm.model.blocks[1].forward(ctx, x, lm.model._caches[1])
    ref = plain_gpt2.block(plain, 1, x0.cpu())
    assert float((x.cpu() - ref).abs().max()) <= _tol(dtype, 2.0)
    _done(lm, entries)


# --------------------------------------------------------------------------- toy parts
def _register_toy():
    """A mixer that keeps a running state per request, and an architecture that uses it."""
    from pretrained_rstr_b200.config import (Architecture, ConfigError, LayerSpec, ModelConfig,
                                             PartSpec, RunEntry, register_architecture)
    from pretrained_rstr_b200.models.assembly import build_model
    from pretrained_rstr_b200.parts import Mixer, StateSpec, register_part
    from pretrained_rstr_b200.weights import TensorExpectation, normal

    class RunningStateMixer(Mixer):
        """s_t = decay * s_{t-1} + h_t (per request, kept in its state slot between steps);
        x_t += W s_t.  Written with array-library calls: toy parts need no kernels."""

        def __init__(self, params, store, runtime):
            self.w = store.get(params["weights"] + ".weight", torch.float32)
            self.decay = float(params["decay"])
            self.width = params["width"]

        def state_specs(self):
            return [StateSpec("running", (self.width,), torch.float32)]

        def forward(self, ctx, h, x, cache):
            state = cache.state["running"]
            host = ctx.host
            for b in range(len(host.rids)):
                slot = host.state_slot[b]
                s = torch.zeros(self.width, device=h.device) if host.fresh[b] else state[slot].clone()
                for t in range(host.q_start[b], host.q_start[b + 1]):
                    s = self.decay * s + h[t].float()
                    x[t] += self.w @ s
                state[slot] = s

    register_part("mixer", "toy_running_state", RunningStateMixer)

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        width: int
        heads: int
        inner: int
        vocab: int
        positions: int
        decay: float
        identifiers = ("ToyForTests",)

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["width"], raw["heads"], raw["inner"], raw["vocab"], raw["positions"],
                       raw["decay"])

        def to_dict(self):
            return {"architectures": ["ToyForTests"], "width": self.width, "heads": self.heads,
                    "inner": self.inner, "vocab": self.vocab, "positions": self.positions,
                    "decay": self.decay}

        def _mlp(self, p):
            return PartSpec("dense_mlp", {"weights": {"up": p + "up", "down": p + "down"},
                                          "width": self.width, "inner": self.inner,
                                          "activation": "relu", "bias": True,
                                          "weight_layout": "out_in"})

        def _norm(self, name):
            return PartSpec("layer_norm", {"weights": name, "size": self.width, "eps": 1e-5})

        def layer_specs(self):
            toy = PartSpec("toy_running_state", {"weights": "l0.mix", "decay": self.decay,
                                                 "width": self.width})
            attn = PartSpec("causal_attention", {
                "weights": {"qkv": "l1.qkv", "out": "l1.out"}, "width": self.width,
                "n_head": self.heads, "n_kv_head": self.heads, "head_dim": self.width // self.heads,
                "scale": 1.0 / math.sqrt(self.width // self.heads), "window": None, "bias": False,
                "weight_layout": "out_in"})
            return [LayerSpec("l0.", "pre_norm", toy, self._mlp("l0."),
                              {"mixer": self._norm("l0.n1"), "feed_forward": self._norm("l0.n2")},
                              self.width),
                    LayerSpec("l1.", "pre_norm", attn, self._mlp("l1."),
                              {"mixer": self._norm("l1.n1"), "feed_forward": self._norm("l1.n2")},
                              self.width)]

        def run_order(self):
            # layer 1 runs twice; its second run reads the cache its first run wrote
            return [RunEntry(0, 0, True), RunEntry(1, 1, True), RunEntry(1, 1, False)]

        def embedding_spec(self):
            return PartSpec("token_embedding", {"weights": "emb", "vocab": self.vocab,
                                                "width": self.width})

        def position_spec(self):
            return PartSpec("learned_absolute", {"weights": "pos", "positions": self.positions,
                                                 "width": self.width})

        def final_norm_spec(self):
            return self._norm("nf")

        def head_spec(self):
            return PartSpec("tied_head", {"weights": "emb", "vocab": self.vocab, "width": self.width})

        @property
        def max_positions(self):
            return self.positions

    def expected(cfg):
        d, f = cfg.width, cfg.inner
        e = {"emb.weight": (cfg.vocab, d), "pos.weight": (cfg.positions, d),
             "nf.weight": (d,), "nf.bias": (d,), "l0.mix.weight": (d, d),
             "l1.qkv.weight": (3 * d, d), "l1.out.weight": (d, d)}
        for l in ("l0.", "l1."):
            e.update({l + "n1.weight": (d,), l + "n1.bias": (d,), l + "n2.weight": (d,),
                      l + "n2.bias": (d,), l + "up.weight": (f, d), l + "up.bias": (f,),
                      l + "down.weight": (d, f), l + "down.bias": (d,)})
        return {k: TensorExpectation(v) for k, v in e.items()}

    def random_tensors(cfg, seed):
        out = {}
        for name, exp in expected(cfg).items():
            is_gain = name.split(".")[-2] in ("n1", "n2", "nf") and name.endswith("weight")
            out[name] = normal(seed, name, exp.shape, 0.05, mean=1.0 if is_gain else 0.0)
        return out

    register_architecture(ToyConfig.identifiers, Architecture(
        "toy", ToyConfig, lambda cfg, store, rt: build_model(cfg, store, rt), expected,
        random_tensors))
    return ToyConfig


def _toy_plain(w: Dict[str, torch.Tensor], cfg, ids):
    """The toy model, whole sequence, plain."""
    d, nh = cfg.width, cfg.heads
    dh = d // nh
    ln = lambda x, n: plain_gpt2.layer_norm(x, w[n + ".weight"], w[n + ".bias"], 1e-5)
    mlp = lambda x, l: torch.relu(x @ w[l + "up.weight"].T + w[l + "up.bias"]) @ w[l + "down.weight"].T \
        + w[l + "down.bias"]
    x = w["emb.weight"][torch.tensor(ids)] + w["pos.weight"][:len(ids)]
    h = ln(x, "l0.n1")
    s = torch.zeros(d)
    mixed = []
    for t in range(len(ids)):
        s = cfg.decay * s + h[t]
        mixed.append(w["l0.mix.weight"] @ s)
    x = x + torch.stack(mixed)
    x = x + mlp(ln(x, "l0.n2"), "l0.")
    kv = None
    for run in range(2):
        qkv = ln(x, "l1.n1") @ w["l1.qkv.weight"].T
        q = qkv[:, :d]
        if run == 0:
            kv = (qkv[:, d:2 * d], qkv[:, 2 * d:])         # the second run reads these again
        k, v = kv
        mask = torch.tril(torch.ones(len(ids), len(ids), dtype=torch.bool))
        o = torch.zeros_like(x)
        for hh in range(nh):
            c = slice(hh * dh, (hh + 1) * dh)
            sc = (q[:, c] @ k[:, c].T) / math.sqrt(dh)
            o[:, c] = torch.softmax(sc.masked_fill(~mask, -math.inf), 1) @ v[:, c]
        x = x + o @ w["l1.out.weight"].T
        x = x + mlp(ln(x, "l1.n2"), "l1.")
    return ln(x, "nf") @ w["emb.weight"].T


@pytest.mark.parametrize("dtype", DTYPES)
def test_toy_architecture_with_state_and_repeated_layer(tmp_path, dtype):
    from pretrained_rstr_b200.engine.batch import Entry
    from pretrained_rstr_b200.engine.loading import load_model
    from pretrained_rstr_b200.weights import load_file, make_random_model
    ToyConfig = _register_toy()
    cfg = ToyConfig(width=48, heads=3, inner=80, vocab=200, positions=160, decay=0.7)
    folder = str(tmp_path / "toy")
    make_random_model(folder, cfg, seed=5,
                      dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    lm = load_model(folder, dtype=dtype, max_batched_tokens=256, max_requests=2, max_tokens=512)
    assert lm.model.graph_safe is False                       # toy parts are not replayed as graphs
    assert (0, "running") in lm.model.state_specs and len(lm.model.group_specs) == 1
    assert lm.model.group_specs[0].layers == (1,)
    w = {k: v.float() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    prompts = {r: random_tokens(n, 200, i) for i, (r, n) in enumerate([("a", 90), ("b", 41), ("c", 70)])}
    oracle = {r: _toy_plain(w, cfg, ids) for r, ids in prompts.items()}
    got = {}

    def run(batch, end=()):
        entries = []
        for rid, lo, hi in batch:
            if rid not in lm.cache.requests:
                lm.cache.open(rid)
            entries.append(Entry(rid, prompts[rid][lo:hi], list(range(hi - lo))))
        logits = lm.runner.step(entries).cpu()
        lm.runner.check_status()
        r = 0
        for rid, lo, hi in batch:
            for p in range(lo, hi):
                got[(rid, p)] = logits[r].clone()
                r += 1
        for rid in end:
            lm.cache.close(rid)

    run([("a", 0, 30)])
    run([("a", 30, 31), ("b", 0, 41)])                        # decode beside a whole prompt
    run([("a", 31, 90), ("b", 41, 41)][:1], end=["a"])
    run([("c", 0, 2)], end=[])                                # c takes the slot a gave back:
    run([("c", 2, 70)], end=["c", "b"])                       # its state must start from zero
    tol = ATOL[dtype]
    for (rid, p), row in got.items():
        err = float((row - oracle[rid][p]).abs().max())
        assert err <= tol, f"request {rid} position {p}: {err:.3e}"
    assert lm.cache.slots.free_count == 2


@pytest.mark.parametrize("dtype", DTYPES)
def test_state_keeping_toy_through_the_entry_point_and_forked(tmp_path, dtype):
    """The same toy model through ``load_lm``, whose default shares prompt prefixes: for a
    model that keeps per-request state the sharing is switched off (a request that took over
    cached pages would never run the state updates of their tokens), so two requests with a
    common 64-token prefix both give the plain tokens.  A fork copies the state row."""
    from pretrained_rstr_b200 import generate_batch, load_lm
    from pretrained_rstr_b200.cache import CacheError
    from pretrained_rstr_b200.engine.batch import Entry
    from pretrained_rstr_b200.weights import load_file, make_random_model
    ToyConfig = _register_toy()
    cfg = ToyConfig(width=48, heads=3, inner=80, vocab=200, positions=160, decay=0.7)
    folder = str(tmp_path / "toy")
    make_random_model(folder, cfg, seed=5,
                      dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    w = {k: v.float() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    m = load_lm(folder, gpu=True, dtype=dtype, max_lanes=3, max_batched_tokens=128,
                prefill_chunk=32, page_size=16)
    cache = m.loaded.cache
    assert cache.has_state and cache.share_prefixes is False
    prefix = random_tokens(64, 200, 1)
    prompts = [prefix + random_tokens(n, 200, 2 + n) for n in (5, 9)]
    first = generate_batch(m, prompts[:1], 5)[0]
    outs = generate_batch(m, prompts, 5)                  # the prefix is in the cache by now
    assert m.stats()["cache"]["prefix_hits"] == 0 and outs[0] == first
    for p, got in zip(prompts, outs):
        ids = list(p)
        for i, tok in enumerate(got):
            row = _toy_plain(w, cfg, ids)[-1]
            want = int(row.argmax())
            if tok != want:
                assert dtype == "bfloat16" and abs(float(row[tok] - row[want])) < 3e-2, \
                    f"token {i}: {tok}, plain says {want}"
            ids.append(tok)
    # fork at a page edge: the child goes on from the parent's pages AND the parent's state
    runner = m.loaded.runner
    base, tails = random_tokens(32, 200, 30), {"root": random_tokens(9, 200, 31),
                                               "kid": random_tokens(12, 200, 32)}
    cache.open("root")
    runner.step([Entry("root", base, [])])
    with pytest.raises(CacheError, match="present length"):
        cache.fork("root", "kid", 16)
    cache.fork("root", "kid")
    logits = runner.step([Entry("root", tails["root"], list(range(9))),
                          Entry("kid", tails["kid"], list(range(12)))]).cpu()
    runner.check_status()
    want = torch.cat([_toy_plain(w, cfg, base + tails["root"])[32:],
                      _toy_plain(w, cfg, base + tails["kid"])[32:]])
    assert float((logits - want).abs().max()) <= ATOL[dtype]
    cache.close("root")
    cache.close("kid")
    cache.check()


# ------------------------------------------------- groups: a windowed layer, grouped heads
def _register_windowed():
    """A second toy architecture out of the framework's own parts: layer 0 attends over all
    keys with grouped key/value heads, layer 1 over a window of 40 keys.  The two layers
    need different caches, so they get page pools and block tables of their own, and the
    windowed one gives pages back while a request is still running."""
    from pretrained_rstr_b200.config import (Architecture, LayerSpec, ModelConfig, PartSpec,
                                             register_architecture)
    from pretrained_rstr_b200.models.assembly import build_model
    from pretrained_rstr_b200.weights import TensorExpectation, normal

    @dataclass(frozen=True)
    class WindowedConfig(ModelConfig):
        width: int
        heads: int
        kv_heads: int
        inner: int
        vocab: int
        positions: int
        window: int
        identifiers = ("WindowedToyForTests",)

        @classmethod
        def from_dict(cls, raw):
            return cls(*(raw[k] for k in ("width", "heads", "kv_heads", "inner", "vocab",
                                          "positions", "window")))

        def to_dict(self):
            return {"architectures": ["WindowedToyForTests"], "width": self.width,
                    "heads": self.heads, "kv_heads": self.kv_heads, "inner": self.inner,
                    "vocab": self.vocab, "positions": self.positions, "window": self.window}

        def _norm(self, name):
            return PartSpec("layer_norm", {"weights": name, "size": self.width, "eps": 1e-5})

        def layer_specs(self):
            dh = self.width // self.heads
            specs = []
            for i, (kv, window) in enumerate([(self.kv_heads, None), (self.heads, self.window)]):
                p = f"l{i}."
                specs.append(LayerSpec(
                    p, "pre_norm",
                    PartSpec("causal_attention", {
                        "weights": {"qkv": p + "qkv", "out": p + "out"}, "width": self.width,
                        "n_head": self.heads, "n_kv_head": kv, "head_dim": dh,
                        "scale": 1.0 / math.sqrt(dh), "window": window, "bias": True,
                        "weight_layout": "out_in"}),
                    PartSpec("dense_mlp", {"weights": {"up": p + "up", "down": p + "down"},
                                           "width": self.width, "inner": self.inner,
                                           "activation": "gelu_new", "bias": True,
                                           "weight_layout": "out_in"}),
                    {"mixer": self._norm(p + "n1"), "feed_forward": self._norm(p + "n2")},
                    self.width))
            return specs

        def embedding_spec(self):
            return PartSpec("token_embedding", {"weights": "emb", "vocab": self.vocab,
                                                "width": self.width})

        def position_spec(self):
            return PartSpec("learned_absolute", {"weights": "pos", "positions": self.positions,
                                                 "width": self.width})

        def final_norm_spec(self):
            return self._norm("nf")

        def head_spec(self):
            return PartSpec("tied_head", {"weights": "emb", "vocab": self.vocab, "width": self.width})

        @property
        def max_positions(self):
            return self.positions

    def expected(cfg):
        d, f, dh = cfg.width, cfg.inner, cfg.width // cfg.heads
        e = {"emb.weight": (cfg.vocab, d), "pos.weight": (cfg.positions, d),
             "nf.weight": (d,), "nf.bias": (d,)}
        for i, kv in enumerate([cfg.kv_heads, cfg.heads]):
            l = f"l{i}."
            n_qkv = (cfg.heads + 2 * kv) * dh
            e.update({l + "qkv.weight": (n_qkv, d), l + "qkv.bias": (n_qkv,),
                      l + "out.weight": (d, d), l + "out.bias": (d,),
                      l + "n1.weight": (d,), l + "n1.bias": (d,), l + "n2.weight": (d,),
                      l + "n2.bias": (d,), l + "up.weight": (f, d), l + "up.bias": (f,),
                      l + "down.weight": (d, f), l + "down.bias": (d,)})
        return {k: TensorExpectation(v) for k, v in e.items()}

    def random_tensors(cfg, seed):
        out = {}
        for name, exp in expected(cfg).items():
            gain = name.split(".")[-2] in ("n1", "n2", "nf") and name.endswith("weight")
            std = 0.12 if "qkv.weight" in name else 0.05       # fairly peaked attention: edges matter
            out[name] = normal(seed, name, exp.shape, std, mean=1.0 if gain else 0.0)
        return out

    register_architecture(WindowedConfig.identifiers, Architecture(
        "windowed-toy", WindowedConfig, lambda cfg, store, rt: build_model(cfg, store, rt),
        expected, random_tensors))
    return WindowedConfig


def _windowed_plain(w, cfg, ids):
    d, nh, dh = cfg.width, cfg.heads, cfg.width // cfg.heads
    ln = lambda x, n: plain_gpt2.layer_norm(x, w[n + ".weight"], w[n + ".bias"], 1e-5)
    x = w["emb.weight"][torch.tensor(ids)] + w["pos.weight"][:len(ids)]
    t = len(ids)
    i, j = torch.arange(t).unsqueeze(1), torch.arange(t).unsqueeze(0)
    for li, (kv, window) in enumerate([(cfg.kv_heads, None), (cfg.heads, cfg.window)]):
        l = f"l{li}."
        qkv = ln(x, l + "n1") @ w[l + "qkv.weight"].T + w[l + "qkv.bias"]
        q, k, v = qkv[:, :nh * dh], qkv[:, nh * dh:(nh + kv) * dh], qkv[:, (nh + kv) * dh:]
        vis = j <= i
        if window is not None:
            vis = vis & (j > i - window)
        o = torch.zeros(t, d)
        for h in range(nh):
            hk = h // (nh // kv)
            sc = (q[:, h * dh:(h + 1) * dh] @ k[:, hk * dh:(hk + 1) * dh].T) / math.sqrt(dh)
            o[:, h * dh:(h + 1) * dh] = torch.softmax(sc.masked_fill(~vis, -math.inf), 1) @ \
                v[:, hk * dh:(hk + 1) * dh]
        x = x + o @ w[l + "out.weight"].T + w[l + "out.bias"]
        hmid = plain_gpt2.gelu_new(ln(x, l + "n2") @ w[l + "up.weight"].T + w[l + "up.bias"])
        x = x + hmid @ w[l + "down.weight"].T + w[l + "down.bias"]
    return ln(x, "nf") @ w["emb.weight"].T


@pytest.mark.parametrize("dtype", DTYPES)
def test_windowed_and_grouped_layers_have_pools_of_their_own(tmp_path, dtype):
    from pretrained_rstr_b200.engine.batch import Entry
    from pretrained_rstr_b200.engine.loading import load_model
    from pretrained_rstr_b200.weights import load_file, make_random_model
    Cfg = _register_windowed()
    cfg = Cfg(width=64, heads=4, kv_heads=2, inner=96, vocab=300, positions=200, window=40)
    folder = str(tmp_path / "win")
    make_random_model(folder, cfg, seed=9,
                      dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    lm = load_model(folder, dtype=dtype, page_size=16, max_batched_tokens=256, max_requests=3,
                    max_tokens=3 * 208)
    groups = lm.model.group_specs
    assert len(groups) == 2 and {g.window for g in groups} == {None, 40}
    assert {g.kv_heads for g in groups} == {2, 4}
    win = [i for i, g in enumerate(groups) if g.window == 40][0]
    w = {k: v.float() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    prompts = {"a": random_tokens(190, 300, 1), "b": random_tokens(75, 300, 2)}
    oracle = {r: _windowed_plain(w, cfg, ids) for r, ids in prompts.items()}
    got, at = {}, {"a": 0, "b": 0}
    for r in prompts:
        lm.cache.open(r)
    cuts = {"a": [50, 1, 1, 30, 2, 64, 1, 41], "b": [3, 40, 1, 1, 30]}
    k = 0
    most_window_pages = 0
    while any(at[r] < len(prompts[r]) for r in prompts):
        entries = []
        for r in prompts:
            if at[r] < len(prompts[r]):
                n = min(cuts[r][k % len(cuts[r])], len(prompts[r]) - at[r])
                entries.append(Entry(r, prompts[r][at[r]:at[r] + n], list(range(n))))
        logits = lm.runner.step(entries).cpu()
        lm.runner.check_status()
        row = 0
        for e in entries:
            for p in range(len(e.tokens)):
                got[(e.rid, at[e.rid] + p)] = logits[row].clone()
                row += 1
            at[e.rid] += len(e.tokens)
        k += 1
        lm.cache.check()
        held = sum(1 for p in lm.cache.block_table("a", win) if p >= 0)
        most_window_pages = max(most_window_pages, held)
    # the windowed group never held more than the window plus the longest portion needs
    assert most_window_pages <= -(-(40 + 64) // 16) + 1
    assert lm.cache.stats["window_released"] > 0
    assert sum(1 for p in lm.cache.block_table("a", 1 - win) if p >= 0) == -(-190 // 16)
    tol = ATOL[dtype] * (3.0 if dtype == "bfloat16" else 2.0)      # peaked attention
    for (rid, p), rowv in sorted(got.items()):
        err = float((rowv - oracle[rid][p]).abs().max())
        assert err <= tol, f"request {rid} position {p}: {err:.3e}"
    for r in prompts:
        lm.cache.close(r)
    assert all(a.free_count == a.num_pages for a in lm.cache.allocators)


# ------------------------- a position encoding and a routed feed-forward defined in the test
def _register_routed():
    """A third toy architecture: no position table but a rotation of queries and keys by
    their position (a position encoding defined here), and in the last layer a feed-forward
    that routes every token to two of three small experts (also defined here), in a block
    arrangement of its own: mixer and feed-forward side by side behind ONE norm."""
    from pretrained_rstr_b200.config import (Architecture, LayerSpec, ModelConfig, PartSpec,
                                             register_architecture)
    from pretrained_rstr_b200.models.assembly import build_model
    from pretrained_rstr_b200.parts import Block, FeedForward, PositionEncoding, register_part
    from pretrained_rstr_b200.weights import TensorExpectation, normal

    class ToyRotation(PositionEncoding):
        """Pairs (i, i + half) of every head turn by position * theta^(-i / half), in 32-bit."""

        def __init__(self, params, store, runtime):
            self.head_dim, self.theta = params["head_dim"], float(params["theta"])

        def rotate(self, ctx, q, k):
            t, half = q.shape[0], self.head_dim // 2
            pos = ctx.positions[:t].float()
            inv = self.theta ** (-torch.arange(half, device=q.device, dtype=torch.float32) / half)
            ang = pos[:, None, None] * inv[None, None, :]
            cos, sin = torch.cos(ang), torch.sin(ang)
            for x in (q, k):
                v = x.float().view(t, -1, self.head_dim)
                a, b = v[..., :half], v[..., half:]
                turned = torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)
                x.copy_(turned.view(t, -1).to(x.dtype))

    class ToyRoutedExperts(FeedForward):
        """x += sum over the token's top two experts of softmax weight * expert(h); router
        logits and weights in 32-bit.  Array-library calls: toy parts need no kernels."""

        def __init__(self, params, store, runtime):
            name = params["weights"]
            self.router = store.get(name + ".router.weight", torch.float32)
            self.up = store.get(name + ".experts.up", torch.float32)        # [E, inner, width]
            self.down = store.get(name + ".experts.down", torch.float32)    # [E, width, inner]
            self.top = int(params["top"])

        def forward(self, ctx, h, x):
            hf = h.tensor().float() if hasattr(h, "tensor") else h.float()
            logits = hf @ self.router.T
            top, which = torch.topk(logits, self.top, dim=1)
            weight = torch.softmax(top, dim=1)
            for e in range(self.router.shape[0]):
                share = (weight * (which == e)).sum(1, keepdim=True)          # 0 where not routed
                x += share * (torch.relu(hf @ self.up[e].T) @ self.down[e].T)

    class ToyParallelBlock(Block):
        """x += mixer(n(x)) + feed_forward(n(x)): both branches read the same normed input."""

        def __init__(self, mixer, feed_forward, norms, width, runtime):
            assert sorted(norms) == ["shared"]
            self.mixer, self.feed_forward, self.norms = mixer, feed_forward, dict(norms)
            self.width, self.runtime = width, runtime

        def forward(self, ctx, x, cache):
            h = ctx.scratch("toy_parallel_normed", (ctx.token_capacity, self.width),
                            self.runtime.dtype)[:x.shape[0]]
            self.norms["shared"].forward(ctx, x, h)
            self.mixer.forward(ctx, h, x, cache)        # x changes, h does not
            self.feed_forward.forward(ctx, h, x)

    register_part("arrangement", "toy_parallel", ToyParallelBlock)
    register_part("position", "toy_rotation", ToyRotation)
    register_part("feed_forward", "toy_routed_experts", ToyRoutedExperts)

    @dataclass(frozen=True)
    class RoutedConfig(ModelConfig):
        width: int
        heads: int
        inner: int
        experts: int
        vocab: int
        positions: int
        theta: float
        identifiers = ("RoutedToyForTests",)
        _keys = ("width", "heads", "inner", "experts", "vocab", "positions", "theta")

        @classmethod
        def from_dict(cls, raw):
            return cls(*(raw[k] for k in cls._keys))

        def to_dict(self):
            return {"architectures": ["RoutedToyForTests"], **{k: getattr(self, k) for k in self._keys}}

        def _norm(self, name):
            return PartSpec("layer_norm", {"weights": name, "size": self.width, "eps": 1e-5})

        def layer_specs(self):
            dh = self.width // self.heads
            specs = []
            for i in range(2):
                p = f"l{i}."
                attn = PartSpec("causal_attention", {
                    "weights": {"qkv": p + "qkv", "out": p + "out"}, "width": self.width,
                    "n_head": self.heads, "n_kv_head": self.heads, "head_dim": dh,
                    "scale": 1.0 / math.sqrt(dh), "window": None, "bias": False,
                    "weight_layout": "out_in"})
                if i == 0:
                    ff = PartSpec("dense_mlp", {"weights": {"up": p + "up", "down": p + "down"},
                                                "width": self.width, "inner": self.inner,
                                                "activation": "relu", "bias": False,
                                                "weight_layout": "out_in"})
                else:
                    ff = PartSpec("toy_routed_experts", {"weights": p + "moe", "top": 2})
                if i == 0:
                    specs.append(LayerSpec(p, "pre_norm", attn, ff,
                                           {"mixer": self._norm(p + "n1"),
                                            "feed_forward": self._norm(p + "n2")}, self.width))
                else:
                    specs.append(LayerSpec(p, "toy_parallel", attn, ff,
                                           {"shared": self._norm(p + "n1")}, self.width))
            return specs

        def embedding_spec(self):
            return PartSpec("token_embedding", {"weights": "emb", "vocab": self.vocab,
                                                "width": self.width})

        def position_spec(self):
            return PartSpec("toy_rotation", {"head_dim": self.width // self.heads,
                                             "theta": self.theta})

        def final_norm_spec(self):
            return self._norm("nf")

        def head_spec(self):
            return PartSpec("tied_head", {"weights": "emb", "vocab": self.vocab, "width": self.width})

        @property
        def max_positions(self):
            return self.positions

    def expected(cfg):
        d, f, n = cfg.width, cfg.inner, cfg.experts
        e = {"emb.weight": (cfg.vocab, d), "nf.weight": (d,), "nf.bias": (d,),
             "l0.up.weight": (f, d), "l0.down.weight": (d, f),
             "l1.moe.router.weight": (n, d), "l1.moe.experts.up": (n, f, d),
             "l1.moe.experts.down": (n, d, f)}
        for l in ("l0.", "l1."):
            e.update({l + "qkv.weight": (3 * d, d), l + "out.weight": (d, d),
                      l + "n1.weight": (d,), l + "n1.bias": (d,)})
        e.update({"l0.n2.weight": (d,), "l0.n2.bias": (d,)})      # the parallel block has one norm
        return {k: TensorExpectation(v) for k, v in e.items()}

    def random_tensors(cfg, seed):
        out = {}
        for name, exp in expected(cfg).items():
            gain = name.split(".")[-2] in ("n1", "n2", "nf") and name.endswith("weight")
            std = 0.5 if "router" in name else 0.15 if "qkv" in name else 0.05
            out[name] = normal(seed, name, exp.shape, std, mean=1.0 if gain else 0.0)
        return out

    register_architecture(RoutedConfig.identifiers, Architecture(
        "routed-toy", RoutedConfig, lambda cfg, store, rt: build_model(cfg, store, rt),
        expected, random_tensors))
    return RoutedConfig


def _routed_plain(w, cfg, ids):
    """The routed toy model, whole sequence, plain.  Also returns, per position, how far the
    router's second choice is ahead of its third."""
    d, nh, dh = cfg.width, cfg.heads, cfg.width // cfg.heads
    half, t = dh // 2, len(ids)
    ln = lambda x, n: plain_gpt2.layer_norm(x, w[n + ".weight"], w[n + ".bias"], 1e-5)
    inv = cfg.theta ** (-torch.arange(half, dtype=torch.float32) / half)
    ang = torch.arange(t, dtype=torch.float32)[:, None] * inv[None, :]
    cos, sin = torch.cos(ang), torch.sin(ang)

    def turn(m):                                   # [t, dh] of one head
        a, b = m[:, :half], m[:, half:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=1)

    mask = torch.tril(torch.ones(t, t, dtype=torch.bool))
    x = w["emb.weight"][torch.tensor(ids)]
    margin = None
    for l in ("l0.", "l1."):
        qkv = ln(x, l + "n1") @ w[l + "qkv.weight"].T
        o = torch.zeros(t, d)
        for h in range(nh):
            c = slice(h * dh, (h + 1) * dh)
            q, k, v = turn(qkv[:, c]), turn(qkv[:, d:2 * d][:, c]), qkv[:, 2 * d:][:, c]
            sc = (q @ k.T) / math.sqrt(dh)
            o[:, c] = torch.softmax(sc.masked_fill(~mask, -math.inf), 1) @ v
        if l == "l0.":
            x = x + o @ w[l + "out.weight"].T
            hn = ln(x, l + "n2")
            x = x + torch.relu(hn @ w["l0.up.weight"].T) @ w["l0.down.weight"].T
        else:
            hn = ln(x, l + "n1")                   # the parallel block: one norm feeds both branches
            x = x + o @ w[l + "out.weight"].T
            logits = hn @ w["l1.moe.router.weight"].T
            ranked, order = torch.sort(logits, dim=1, descending=True)
            margin = ranked[:, 1] - ranked[:, 2]
            weight = torch.softmax(ranked[:, :2], dim=1)
            y = torch.zeros(t, d)
            for pos in range(t):
                for slot in range(2):
                    e = int(order[pos, slot])
                    y[pos] += weight[pos, slot] * (torch.relu(hn[pos] @ w["l1.moe.experts.up"][e].T)
                                                   @ w["l1.moe.experts.down"][e].T)
            x = x + y
    return ln(x, "nf") @ w["emb.weight"].T, margin


@pytest.mark.parametrize("dtype", DTYPES)
def test_position_encoding_and_routed_feed_forward_defined_in_the_test(tmp_path, dtype):
    from pretrained_rstr_b200.engine.batch import Entry
    from pretrained_rstr_b200.engine.loading import load_model
    from pretrained_rstr_b200.weights import load_file, make_random_model
    Cfg = _register_routed()
    cfg = Cfg(width=64, heads=4, inner=40, experts=3, vocab=150, positions=200, theta=50.0)
    folder = str(tmp_path / "routed")
    make_random_model(folder, cfg, seed=11,
                      dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    lm = load_model(folder, dtype=dtype, page_size=16, max_batched_tokens=256, max_requests=2,
                    max_tokens=2 * 208)
    assert lm.model.graph_safe is False
    w = {k: v.float() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    prompts = {"a": random_tokens(150, 150, 3), "b": random_tokens(67, 150, 4)}
    oracle = {r: _routed_plain(w, cfg, ids) for r, ids in prompts.items()}
    got, at = {}, {"a": 0, "b": 0}
    for r in prompts:
        lm.cache.open(r)
    cuts = {"a": [70, 1, 1, 2, 33, 1], "b": [5, 1, 40, 1, 1]}
    k = 0
    while any(at[r] < len(prompts[r]) for r in prompts):
        entries = []
        for r in prompts:
            if at[r] < len(prompts[r]):
                n = min(cuts[r][k % len(cuts[r])], len(prompts[r]) - at[r])
                entries.append(Entry(r, prompts[r][at[r]:at[r] + n], list(range(n))))
        logits = lm.runner.step(entries).cpu()
        lm.runner.check_status()
        row = 0
        for e in entries:
            for p in range(len(e.tokens)):
                got[(e.rid, at[e.rid] + p)] = logits[row].clone()
                row += 1
            at[e.rid] += len(e.tokens)
        k += 1
    # where the router's second and third choices lie closer than rounding can move them the
    # engine may rightly choose otherwise; the routed layer is the last, so only that
    # position's logits would differ
    near = 1e-4 if dtype == "float32" else 5e-2
    # (bfloat16: the rotation defined above rounds queries and keys a second time)
    tol, checked = ATOL[dtype] * (1.0 if dtype == "float32" else 2.0), 0
    for (rid, p), rowv in sorted(got.items()):
        ref, margin = oracle[rid]
        if float(margin[p]) < near:
            continue
        checked += 1
        err = float((rowv - ref[p]).abs().max())
        assert err <= tol, f"request {rid} position {p}: {err:.3e}"
    assert checked >= 0.8 * len(got)
    for r in prompts:
        lm.cache.close(r)
    lm.cache.check()
