"""Whole-model comparisons at the layer sizes the engine is measured at: GPT-2 small,
medium and XL widths, head counts, inner widths and the 50,257-token vocabulary, with two
layers (fewer layers, not smaller ones).  The kernels choose instances, tile widths and
splits from these sizes, so only models of these sizes run what the benchmark runs: the
tensor-memory product at 96 to 256 columns and with the reduction split over a cluster,
the cluster split-K product at widths 768 to 1,600, the key and value scatter at 12, 16
and 25 heads, the head over a vocabulary whose row pitch is odd, prompt attention with key
parts, and decode attention with one split per (token, head) at 64 live requests.

Every way of cutting the work, in 32-bit and in bfloat16, against the plain implementation
at chosen positions (first tokens, the edges of pages and of 128-query tiles, the tail).
"""
import random

import pytest
import torch

from helpers import ATOL, Replayer, bf16_atol, compare, make_folder, oracle_rows, random_tokens, \
    real_width

pytestmark = pytest.mark.gpu

SIZES = ["small", "medium", "xl"]
LENGTHS = {"small": [1000, 260, 70], "medium": [900, 131, 66], "xl": [1024, 200, 40]}


def _tol(dtype, width):
    return ATOL["float32"] if dtype == "float32" else bf16_atol(width)


def _wanted(n):
    """Positions whose logits are compared: the first tokens, both sides of every page and
    tile edge up to 256 and of the last page edge, and the last 33."""
    picks = {0, 1, 2, 62, 63, 64, 65, 127, 128, 129, 255, 256, 257}
    edge = (n - 1) // 64 * 64
    picks |= {edge - 1, edge, edge + 1}
    picks |= set(range(n - 33, n))
    return sorted(p for p in picks if 0 <= p < n)


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """Folder, prompts and plain logits per (size, element type), made when first asked for."""
    made = {}

    def get(size, dtype):
        key = (size, dtype)
        if key not in made:
            raw = real_width(size)
            folder = make_folder(str(tmp_path_factory.mktemp(f"real_{size}_{dtype}")), raw,
                                 {"small": 2, "medium": 3, "xl": 4}[size], dtype)
            prompts = {f"w{i}": random_tokens(n, raw["vocab_size"], 71 * i + len(size))
                       for i, n in enumerate(LENGTHS[size])}
            wanted = {rid: _wanted(len(ids)) for rid, ids in prompts.items()}
            made[key] = (folder, raw, prompts, wanted, oracle_rows(folder, prompts, wanted))
        return made[key]
    return get


def _want_in(wanted, lo, hi):
    return [p - lo for p in wanted if lo <= p < hi]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("size", SIZES)
def test_whole_and_last_tokens_one_by_one(models, size, dtype):
    """Each request alone and whole; then most of it in one step and the last 32 tokens one
    by one."""
    folder, raw, prompts, wanted, oracle = models(size, dtype)
    rp = Replayer(folder, dtype, max_tokens=1024, max_batched_tokens=1024)
    for rid, ids in prompts.items():
        rp.step([(rid, ids, wanted[rid])], end=[rid])
    whole = compare(rp.rows, oracle, _tol(dtype, raw["n_embd"]))
    rp.rows.clear()
    for rid, ids in prompts.items():
        head = len(ids) - 32
        rp.step([(rid, ids[:head], _want_in(wanted[rid], 0, head))])
        for i in range(head, len(ids)):
            rp.step([(rid, ids[i:i + 1], [0])], end=[rid] if i == len(ids) - 1 else [])
    tail = compare(rp.rows, oracle, _tol(dtype, raw["n_embd"]))
    print(f"{size} {dtype}: largest difference whole {whole:.2e}, decoded tail {tail:.2e}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("size", SIZES)
def test_portions_and_mixed_with_page_reuse(models, size, dtype):
    """Portions of changing size, down to two tokens; then the requests mixed, portions of
    some beside decoded tokens of others, in a pool too small for all of them."""
    folder, raw, prompts, wanted, oracle = models(size, dtype)
    tol = _tol(dtype, raw["n_embd"])
    rp = Replayer(folder, dtype, max_tokens=1024, max_batched_tokens=1024)
    sizes = [7, 2, 190, 2, 65, 64, 3, 300, 31, 129]
    for rid, ids in prompts.items():
        at = k = 0
        while at < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - at)
            k += 1
            rp.step([(rid, ids[at:at + n], _want_in(wanted[rid], at, at + n))],
                    end=[rid] if at + n >= len(ids) else [])
            at += n
    portions = compare(rp.rows, oracle, tol)
    # mixed: every request twice (the second time under another name), two pages short of
    # holding all at once, so that pages of finished requests are handed out again
    lengths = sorted((len(v) for v in prompts.values()), reverse=True)
    rounded = [-(-n // 64) * 64 for n in lengths]
    pool = rounded[0] + rounded[1] + rounded[2]
    rp = Replayer(folder, dtype, max_tokens=pool, max_batched_tokens=1024)
    jobs = [(f"{rid}/{rep}", rid) for rep in range(2) for rid in prompts]
    rng = random.Random(9)
    live, waiting = {}, list(jobs)
    while waiting or live:
        while waiting and len(live) < 3 and \
                sum(-(-len(prompts[src]) // 64) for _, src in live.values()) + \
                -(-len(prompts[waiting[0][1]]) // 64) <= pool // 64:
            name, src = waiting.pop(0)
            live[name] = (0, src)
        entries, end = [], []
        for name in list(live):
            at, src = live[name]
            ids = prompts[src]
            left = len(ids) - at
            if left > 20:
                n = min(left - 8, rng.choice([2, 3, 64, 70, 200, 400]))
            else:
                n = 1
            entries.append((name, ids[at:at + n], _want_in(wanted[src], at, at + n)))
            live[name] = (at + n, src)
            if at + n == len(ids):
                end.append(name)
                del live[name]
        rp.step(entries, end=end)
    assert rp.lm.cache.stats["allocated"] > rp.lm.cache.allocators[0].num_pages
    assert rp.lm.cache.free_pages(0) == rp.lm.cache.allocators[0].num_pages
    rows = {(name.split("/")[0], pos): row for (name, pos), row in rp.rows.items()}
    mixed = compare(rows, oracle, tol)
    print(f"{size} {dtype}: largest difference portions {portions:.2e}, mixed {mixed:.2e}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sixty_four_requests_decoding_together(models, tmp_path, dtype):
    """Prompts of unequal length, several to a step; then all 64 requests decode together,
    one token each a step: the products of 17 to 64 rows, decode attention with one split per
    (token, head) (64 x 12 pairs), and the steps' graphs at 64 requests."""
    folder, raw, _p, _w, _o = models("small", dtype)
    rng = random.Random(3)
    decode_steps = 12
    prompts = {f"q{i}": random_tokens(rng.choice([3, 17, 64, 65, 130, 200, 333]) + decode_steps,
                                      raw["vocab_size"], 500 + i) for i in range(64)}
    wanted = {rid: list(range(len(ids) - decode_steps - 1, len(ids))) for rid, ids in prompts.items()}
    oracle = oracle_rows(folder, prompts, wanted)
    total = sum(-(-len(ids) // 64) * 64 for ids in prompts.values())
    rp = Replayer(folder, dtype, max_tokens=total, max_batched_tokens=2048, max_requests=64)
    batch, tokens = [], 0
    for rid, ids in prompts.items():
        n = len(ids) - decode_steps
        if tokens + n > 2048:
            rp.step(batch)
            batch, tokens = [], 0
        batch.append((rid, ids[:n], [n - 1]))
        tokens += n
    rp.step(batch)
    for k in range(decode_steps, 0, -1):
        rp.step([(rid, ids[len(ids) - k:len(ids) - k + 1], [0]) for rid, ids in prompts.items()],
                end=list(prompts) if k == 1 else [])
    assert len(rp.rows) == 64 * (decode_steps + 1)
    worst = compare(rp.rows, oracle, _tol(dtype, raw["n_embd"]))
    print(f"64 requests {dtype}: largest difference {worst:.2e}")


@pytest.mark.parametrize("ring", [False, True])
def test_either_decode_attention_kernel_forced(models, monkeypatch, ring):
    """The engine picks the decode attention kernel by the size of the launch; here each of
    the two runs everything: single tokens of one request, of three requests of unequal
    length side by side, and portions of two to four tokens beside them."""
    from pretrained_rstr_b200.settings import SETTINGS
    monkeypatch.setattr(SETTINGS, "decode_ring", ring)
    folder, raw, prompts, wanted, oracle = models("small", "bfloat16")
    rp = Replayer(folder, "bfloat16", max_tokens=2048, max_batched_tokens=1024)
    tail = 12
    for rid, ids in prompts.items():
        head = len(ids) - tail
        rp.step([(rid, ids[:head], _want_in(wanted[rid], 0, head))])
    first = next(iter(prompts))
    done = {rid: len(ids) - tail for rid, ids in prompts.items()}
    for i in range(4):                                     # one request alone
        at = done[first]
        rp.step([(first, prompts[first][at:at + 1], [0])])
        done[first] += 1
    cuts = [1, 3, 2, 1, 4, 1]
    step = 0
    while any(done[rid] < len(ids) for rid, ids in prompts.items()):
        batch, ended = [], []
        for j, (rid, ids) in enumerate(prompts.items()):
            if done[rid] >= len(ids):
                continue
            n = min(cuts[(step + j) % len(cuts)], len(ids) - done[rid])
            batch.append((rid, ids[done[rid]:done[rid] + n], list(range(n))))
            done[rid] += n
            if done[rid] == len(ids):
                ended.append(rid)
        rp.step(batch, end=ended)
        step += 1
    worst = compare(rp.rows, oracle, _tol("bfloat16", raw["n_embd"]))
    print(f"ring {ring}: largest difference {worst:.2e}")
