"""The scheduler on the device: more requests than lanes and than pages, prompts in
portions beside decoding requests, shared prefixes, eviction of cached pages, greedy and
seeded sampling side by side, in 32-bit (token for token) and in bfloat16 (token for token
up to near-ties of the plain implementation's own numbers)."""
import math

import pytest
import torch

import plain_gpt2
from helpers import TINY, make_folder, random_tokens

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {(name, dtype): make_folder(str(tmp_path_factory.mktemp(f"s{name}{dtype}")), raw, seed,
                                       dtype)
            for name, (raw, seed) in TINY.items() for dtype in DTYPES}


def check_tokens(plain, prompt, got, opts, dtype, what):
    """``got`` against the plain implementation, token by token along the sequence that was
    really generated.  float32: every token equal.  bfloat16: a token may differ only where the
    plain numbers nearly tie: two logits within 3e-2 (for a greedy choice, or for two candidates
    of a sampled one, which may then swap places in the sorted list); or, for a sampled one, the
    draw within 0.02 (in probability) of the boundaries between the two candidates."""
    greedy = not opts or opts.get("temperature", 0.0) <= 0.0
    rng = None if greedy else plain_gpt2.JavaRandom(opts["seed"])
    ids = list(prompt)
    for i, tok in enumerate(got):
        row = plain_gpt2.all_logits(plain, ids)[-1]
        if greedy:
            want = plain_gpt2.argmax(row)
            if tok != want:
                assert dtype == "bfloat16", f"{what}: token {i} is {tok}, plain says {want}"
                gap = abs(float(row[tok] - row[want]))
                assert gap < 3e-2, f"{what}: token {i} is {tok}, plain says {want}, gap {gap:.3g}"
        else:
            t, k, p = opts["temperature"], opts.get("top_k") or 40, opts.get("top_p") or 1.0
            cand = plain_gpt2.top_k_ids(row, k)
            mx = float(row[cand[0]]) / t
            probs = [math.exp(float(row[c]) / t - mx) for c in cand]
            total = sum(probs)
            cut, c = len(cand), 0.0
            for j, q in enumerate(probs):
                c += q / total
                if c >= p:
                    cut = j + 1
                    break
            tot = sum(probs[:cut])
            r = rng.next_double() * tot
            acc, want, edges = 0.0, cand[cut - 1], []
            for j in range(cut):
                acc += probs[j]
                edges.append(acc)
            for j in range(cut):
                if edges[j] >= r or j == cut - 1:
                    want = cand[j]
                    break
            if tok != want:
                assert dtype == "bfloat16", f"{what}: sampled token {i} is {tok}, plain says {want}"
                # two candidates whose logits nearly tie may swap places in the sorted list, and
                # the same draw then lands on the other one
                if abs(float(row[tok] - row[want])) >= 3e-2:
                    assert tok in cand[:cut], f"{what}: token {i} ({tok}) outside the candidates"
                    jt, jw = cand.index(tok), cand.index(want)
                    lo, hi = min(jt, jw), max(jt, jw)
                    # else the draw lies within a whisker of every boundary between the two
                    assert all(abs(edges[j] - r) / tot < 0.02 for j in range(lo, hi)), \
                        f"{what}: sampled token {i} is {tok}, plain says {want}, no near-tie"
        ids.append(tok)


@pytest.mark.parametrize("dtype", DTYPES)
def test_tiny_b_workload_as_written(folders, dtype):
    """Five requests with prompts of 1, 9, 33, 64 and 130 tokens, cut into portions of 32 and
    mixed with decoding requests, 24 new tokens each at temperature 0.8 with seed 7, on four
    lanes (so the fifth waits for a lane)."""
    from pretrained_rstr_b200 import generate_batch, load_lm
    raw, seed = TINY["B"]
    folder = folders[("B", dtype)]
    plain = plain_gpt2.PlainGPT2(folder)
    m = load_lm(folder, gpu=True, dtype=dtype, max_lanes=4, max_batched_tokens=64, prefill_chunk=32)
    prompts = [random_tokens(n, raw["vocab_size"], 40 + i) for i, n in enumerate([1, 9, 33, 64, 130])]
    opts = {"temperature": 0.8, "seed": 7}
    outs = generate_batch(m, prompts, 24, opts)
    for p, got in zip(prompts, outs):
        assert len(got) == 24
        if dtype == "float32":
            assert got == plain_gpt2.sample_generate(plain, p, 24, 0.8, None, None, 7)
        check_tokens(plain, p, got, opts, dtype, f"prompt of {len(p)}")
    stats = m.stats()
    assert stats["scheduler"]["iterations"] > 24 and not m.loaded.cache.requests
    m.loaded.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_more_requests_than_pages(folders, dtype):
    """Eight requests, pages for about three: admissions wait for pages, finished requests'
    pages are cached by the prefix index, taken over by later requests with the same prefix,
    and evicted when a stranger needs room.  Greedy and sampling requests side by side."""
    from pretrained_rstr_b200 import load_lm
    from pretrained_rstr_b200.engine.scheduler import SamplingParams
    raw, seed = TINY["B"]
    folder = folders[("B", dtype)]
    plain = plain_gpt2.PlainGPT2(folder)
    page = 16
    m = load_lm(folder, gpu=True, dtype=dtype, max_lanes=4, max_batched_tokens=96,
                prefill_chunk=32, page_size=page, max_tokens=24 * page, share_prefixes=True)
    eng = m.engine
    prefix = random_tokens(70, raw["vocab_size"], 77)             # four full pages and a bit
    tails = [3, 40, 1, 25, 60]
    prompts = [prefix + random_tokens(n, raw["vocab_size"], 80 + n) for n in tails]
    prompts += [random_tokens(n, raw["vocab_size"], 90 + n) for n in (120, 9, 150)]
    n_new = 14
    opts = [None if i % 2 == 0 else {"temperature": 0.9, "top_k": 12, "seed": 100 + i}
            for i in range(len(prompts))]
    order = [0, 5, 1, 6, 2, 7, 3, 4]
    for i in order:
        sp = SamplingParams() if opts[i] is None else SamplingParams(
            temperature=opts[i]["temperature"], top_k=opts[i]["top_k"], seed=opts[i]["seed"])
        eng.submit(i, prompts[i], n_new, sp)
    eng.run()
    outs = {i: eng.scheduler.finished.pop(i).output for i in order}
    stats = eng.stats()
    assert stats["scheduler"]["deferred_admissions"] > 0, "every admission found its pages at once"
    assert stats["cache"]["prefix_hits"] >= 4, "no request took over cached pages of the shared prefix"
    assert stats["cache"]["evicted"] > 0, "no cached page had to make room"
    cache = m.loaded.cache
    assert not cache.requests
    cache.check()
    assert cache.free_pages(0) + len(cache._index) == cache.allocators[0].num_pages
    for i in order:
        assert len(outs[i]) == n_new
        check_tokens(plain, prompts[i], outs[i], opts[i], dtype, f"request {i}")
