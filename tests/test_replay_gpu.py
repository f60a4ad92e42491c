"""Whole-model comparisons with the plain implementation under every way of cutting
and batching the work, in 32-bit and in bfloat16, for both tiny configurations."""
import pytest
import torch

from helpers import ATOL, TINY, Replayer, compare, make_folder, oracle_logits, random_tokens

pytestmark = pytest.mark.gpu

CASES = [(name, dtype) for name in ("A", "B", "C") for dtype in ("float32", "bfloat16")]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, (raw, seed) in TINY.items():
        for dtype in ("float32", "bfloat16"):
            out[(name, dtype)] = make_folder(
                str(tmp_path_factory.mktemp(f"tiny{name}_{dtype}")), raw, seed, dtype)
    return out


def _prompts(name):
    raw, seed = TINY[name]
    lengths = {"A": [5, 17, 40, 100], "B": [1, 9, 33, 64, 130, 250], "C": [3, 64, 129, 300, 500]}[name]
    return {f"r{i}": random_tokens(n, raw["vocab_size"], 100 * seed + i)
            for i, n in enumerate(lengths)}


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole(folders, name, dtype):
    """Each request alone and whole, every position's logits."""
    folder = folders[(name, dtype)]
    prompts = _prompts(name)
    oracle = oracle_logits(folder, prompts)
    rp = Replayer(folder, dtype, max_tokens=512)
    for rid, ids in prompts.items():
        rp.step([(rid, ids, list(range(len(ids))))], end=[rid])
    compare(rp.rows, oracle, ATOL[dtype])


@pytest.mark.parametrize("name,dtype", CASES)
def test_prefill_then_decode(folders, name, dtype):
    """Most of it in one step and the last 32 tokens one by one."""
    folder = folders[(name, dtype)]
    prompts = {k: v for k, v in _prompts(name).items() if len(v) > 33}
    oracle = oracle_logits(folder, prompts)
    rp = Replayer(folder, dtype, max_tokens=512)
    for rid, ids in prompts.items():
        head = len(ids) - 32
        rp.step([(rid, ids[:head], [head - 1])])
        for i in range(head, len(ids)):
            rp.step([(rid, ids[i:i + 1], [0])], end=[rid] if i == len(ids) - 1 else [])
    compare(rp.rows, oracle, ATOL[dtype])


@pytest.mark.parametrize("name,dtype", CASES)
def test_portions(folders, name, dtype):
    """Portions of changing size, down to two tokens."""
    folder = folders[(name, dtype)]
    prompts = _prompts(name)
    oracle = oracle_logits(folder, prompts)
    rp = Replayer(folder, dtype, max_tokens=512)
    sizes = [7, 2, 19, 2, 5, 64, 3, 2, 31, 66, 130]
    for rid, ids in prompts.items():
        at, k = 0, 0
        while at < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - at)
            k += 1
            last = at + n >= len(ids)
            rp.step([(rid, ids[at:at + n], list(range(n)))], end=[rid] if last else [])
            at += n
    compare(rp.rows, oracle, ATOL[dtype])


@pytest.mark.parametrize("name,dtype", CASES)
def test_mixed_with_page_reuse(folders, name, dtype):
    """Up to four live requests, portions of some beside decoded tokens of others, in a
    pool so small that pages of finished requests are used again."""
    folder = folders[(name, dtype)]
    raw, seed = TINY[name]
    n_pos = raw["n_positions"]
    lengths = {"A": [40, 100, 17, 70, 128, 5, 90, 33], "B": [130, 64, 250, 9, 33, 200, 1, 120],
               "C": [300, 130, 500, 64, 257, 9, 400, 128]}[name]
    prompts = {f"m{i}": random_tokens(n, raw["vocab_size"], 977 * seed + i)
               for i, n in enumerate(lengths)}
    oracle = oracle_logits(folder, prompts)
    # room for the four largest at once, not for all eight
    biggest = sorted((-(-n // 64) * 64 for n in lengths), reverse=True)
    max_tokens = sum(biggest[:4])
    assert max_tokens < sum(-(-n // 64) * 64 for n in lengths)
    rp = Replayer(folder, dtype, max_tokens=max_tokens)
    import random
    rng = random.Random(5)
    waiting = list(prompts)
    live = {}
    while waiting or live:
        while waiting and len(live) < 4:
            live[waiting.pop(0)] = 0
        entries, end = [], []
        for rid in list(live):
            ids = prompts[rid]
            at = live[rid]
            left = len(ids) - at
            if at == 0 and rng.random() < 0.3 and len(live) > 1:
                continue                                   # left out of this step
            if left > 34 and at < len(ids) - 16:
                n = min(left - 16, rng.choice([2, 3, 8, 21, 64, 70, 140]))
            else:
                n = 1                                      # decode the tail token by token
            entries.append((rid, ids[at:at + n], list(range(n))))
            live[rid] = at + n
            if live[rid] == len(ids):
                end.append(rid)
                del live[rid]
        if entries:
            rp.step(entries, end=end)
    assert rp.lm.cache.stats["allocated"] > rp.lm.cache.allocators[0].num_pages, \
        "the pool was large enough that no page was used twice"
    assert rp.lm.cache.free_pages(0) == rp.lm.cache.allocators[0].num_pages
    compare(rp.rows, oracle, ATOL[dtype])
