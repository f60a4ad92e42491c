"""Generation through the Python entry point against the plain implementation:
greedy and seeded temperature sampling, one request and several at once."""
import pytest
import torch

import plain_gpt2
from helpers import TINY, make_folder, random_tokens

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {(name, dtype): make_folder(str(tmp_path_factory.mktemp(f"g{name}{dtype}")), raw, seed,
                                       dtype)
            for name, (raw, seed) in TINY.items() for dtype in ("float32", "bfloat16")}


def _agree(plain, prompt, got, want, dtype, what):
    """Token lists must be equal; in bfloat16 the first difference may only be a near-tie
    of the plain logits (after it the sequences legitimately diverge)."""
    if got == want:
        return
    assert dtype == "bfloat16", f"{what}: {got} != {want}"
    for i, (a, b) in enumerate(zip(got, want)):
        if a != b:
            row = plain_gpt2.all_logits(plain, list(prompt) + want[:i])[-1]
            gap = abs(float(row[a] - row[b]))
            assert gap < 3e-2, f"{what}: token {i} is {a}, plain says {b}, logit gap {gap:.3g}"
            return
    assert len(got) == len(want), f"{what}: lengths differ"


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_entry_point(folders, name, dtype):
    from pretrained_rstr_b200 import generate_batch, generate_ids, load_lm
    raw, seed = TINY[name]
    folder = folders[(name, dtype)]
    plain = plain_gpt2.PlainGPT2(folder)
    m = load_lm(folder, gpu=True, dtype=dtype, max_lanes=4, max_batched_tokens=128,
                prefill_chunk=32)
    lengths = [5, 17, 40] if name == "A" else [1, 9, 33, 64, 130]
    prompts = [random_tokens(n, raw["vocab_size"], 31 * seed + i) for i, n in enumerate(lengths)]
    n_new = 16 if name == "A" else 24
    for p in prompts[:2]:
        _agree(plain, p, generate_ids(m, p, n_new), plain_gpt2.greedy_generate(plain, p, n_new),
               dtype, f"alone len {len(p)}")
    outs = generate_batch(m, prompts, n_new)          # more prompts than lanes: queueing too
    for p, got in zip(prompts, outs):
        _agree(plain, p, got, plain_gpt2.greedy_generate(plain, p, n_new), dtype,
               f"batched len {len(p)}")
    cache = m.engine.lm.cache
    assert not cache.requests
    # every page is either free or held by the prefix index alone: none is lost
    assert cache.free_pages(0) + len(cache._index) == cache.allocators[0].num_pages
    m.engine.lm.cache.check()


@pytest.mark.parametrize("name", ["A", "B"])
def test_temperature_sampling_matches_plain(folders, name):
    """float32 logits, same top-k / softmax / nucleus / generator: same tokens."""
    from pretrained_rstr_b200 import generate_batch, generate_ids, load_lm
    raw, seed = TINY[name]
    folder = folders[(name, "float32")]
    plain = plain_gpt2.PlainGPT2(folder)
    m = load_lm(folder, gpu=True, dtype="float32", max_lanes=4, max_batched_tokens=128,
                prefill_chunk=32)
    prompts = [random_tokens(n, raw["vocab_size"], 7 * seed + i) for i, n in enumerate([9, 33, 3])]
    for opts in ({"temperature": 0.8, "seed": 7}, {"temperature": 1.3, "top_k": 5, "seed": 1},
                 {"temperature": 0.7, "top_k": 50, "top_p": 0.6, "seed": 123456789}):
        want = [plain_gpt2.sample_generate(plain, p, 12, opts["temperature"], opts.get("top_k"),
                                           opts.get("top_p"), opts["seed"]) for p in prompts]
        assert generate_ids(m, prompts[0], 12, opts) == want[0]
        assert generate_batch(m, prompts, 12, opts) == want


def test_stop_token_and_capacity(folders):
    from pretrained_rstr_b200 import generate_ids, load_lm
    raw, seed = TINY["A"]
    folder = folders[("A", "float32")]
    plain = plain_gpt2.PlainGPT2(folder)
    m = load_lm(folder, gpu=True, dtype="float32", max_lanes=2, max_batched_tokens=128)
    p = random_tokens(6, raw["vocab_size"], 3)
    free = plain_gpt2.greedy_generate(plain, p, 10)
    m.eos_ids = (free[3],)
    stop_at = free.index(free[3])
    assert generate_ids(m, p, 10) == free[:stop_at + 1]       # the stop token is kept
    m.eos_ids = ()
    long_prompt = random_tokens(raw["n_positions"] - 3, raw["vocab_size"], 4)
    out = generate_ids(m, long_prompt, 10)
    assert len(out) == 4                                       # positions are used up
    assert out == plain_gpt2.greedy_generate(plain, long_prompt, 10)[:4]


def test_stop_token_inside_a_batch(folders):
    """The engine launches the next step before this one's tokens have reached the host,
    assuming nobody stops on a stop token.  One of three requests does stop: its row in the
    step already in flight is dropped, the others go on unchanged, and no page is lost."""
    from pretrained_rstr_b200 import generate_batch, load_lm
    raw, seed = TINY["B"]
    folder = folders[("B", "float32")]
    plain = plain_gpt2.PlainGPT2(folder)
    m = load_lm(folder, gpu=True, dtype="float32", max_lanes=4, max_batched_tokens=128)
    prompts = [random_tokens(n, raw["vocab_size"], 50 + i) for i, n in enumerate([7, 12, 3])]
    opts = {"temperature": 1.2, "seed": 11}           # greedy output of random weights repeats
    free = [plain_gpt2.sample_generate(plain, p, 20, 1.2, None, None, 11) for p in prompts]
    stop = next(t for t in free[1][4:]
                if t not in free[0] and t not in free[2] and t not in free[1][:4])
    want = [free[0], free[1][:free[1].index(stop) + 1], free[2]]
    assert 4 < len(want[1]) < 20
    m.eos_ids = (stop,)
    assert generate_batch(m, prompts, 20, opts) == want
    ahead = m.engine.stats()["prepared_ahead"]
    # the step after the stop token was already in flight: its row for that request is dropped
    assert ahead["used"] > 10 and ahead["dead_rows"] >= 1
    m.engine.lm.cache.check()
    assert not m.engine.lm.cache.requests


def test_arrivals_cancels_and_mixed_sampling_with_steps_in_flight(folders):
    """The host runs one step behind the GPU (``step(ahead=True)``): requests with
    different sampling options side by side, one arriving and one cancelled while steps
    are in flight; every output equals the plain implementation's (a prefix of it for the
    cancelled request)."""
    from pretrained_rstr_b200 import load_lm
    from pretrained_rstr_b200.engine.scheduler import SamplingParams
    raw, seed = TINY["C"]
    folder = folders[("C", "float32")]
    plain = plain_gpt2.PlainGPT2(folder)
    m = load_lm(folder, gpu=True, dtype="float32", max_lanes=4, max_batched_tokens=256)
    eng = m.engine
    prompts = [random_tokens(n, raw["vocab_size"], 900 + i) for i, n in enumerate([11, 70, 5, 33])]
    opts = [SamplingParams(), SamplingParams(temperature=0.9, top_k=20, seed=5),
            SamplingParams(temperature=1.4, top_k=7, top_p=0.8, seed=6), SamplingParams()]
    n_new = [30, 25, 40, 12]
    want = []
    for p, o, n in zip(prompts, opts, n_new):
        want.append(plain_gpt2.greedy_generate(plain, p, n) if o.greedy else
                    plain_gpt2.sample_generate(plain, p, n, o.temperature, o.top_k, o.top_p, o.seed))
    for i in (0, 1):
        eng.submit(i, prompts[i], n_new[i], opts[i])
    finished, calls = {}, 0
    while not eng.scheduler.idle or calls < 8:
        if calls == 6:
            eng.submit(2, prompts[2], n_new[2], opts[2])      # arrives while steps are in flight
            eng.submit(3, prompts[3], n_new[3], opts[3])
        if calls == 14:
            eng.cancel(0)
        for r in eng.step(ahead=True):
            finished[r.rid] = r
        calls += 1
        assert calls < 400
    for r in eng.flush():
        finished[r.rid] = r
    assert sorted(finished) == [1, 2, 3]               # a cancelled request is not reported as done
    finished[0] = eng.scheduler.finished[0]
    assert finished[0].finish_reason == "cancelled"
    assert 3 < len(finished[0].output) < n_new[0] and finished[0].output == want[0][:len(finished[0].output)]
    for i in (1, 2, 3):
        assert finished[i].output == want[i], f"request {i}"
    stats = eng.stats()
    assert stats["prepared_ahead"]["used"] > 20
    m.engine.lm.cache.check()
    assert not m.engine.lm.cache.requests


def test_step_words_through_the_copy_engine(folders, monkeypatch):
    """Where kernels cannot reach the pinned buffers (here: switched off), the step's
    description and its result go through the copy engine and token feedback through a kernel
    of its own; the tokens are the same."""
    from pretrained_rstr_b200 import generate_batch, load_lm
    from pretrained_rstr_b200.settings import SETTINGS
    raw, seed = TINY["A"]
    folder = folders[("A", "float32")]
    prompts = [random_tokens(n, raw["vocab_size"], 40 + n) for n in (3, 9, 17)]
    by_kernel = load_lm(folder, gpu=True, dtype="float32")
    assert all(by_kernel.engine.runner._host_addresses) and all(by_kernel.engine.runner._result_addresses)
    want = generate_batch(by_kernel, prompts, 12)
    monkeypatch.setattr(SETTINGS, "step_words_by_kernel", False)
    by_copy = load_lm(folder, gpu=True, dtype="float32")
    assert not any(by_copy.engine.runner._host_addresses) and not any(by_copy.engine.runner._result_addresses)
    assert generate_batch(by_copy, prompts, 12) == want
    assert by_copy.engine.ahead["used"] > 0                # steps were launched ahead (feedback)


def test_more_lanes_than_the_several_cta_token_choice_takes(folders):
    """100 requests through 128 lanes (steps of up to 100 rows: one CTA a row chooses and
    publishes) give what they give through 8 lanes, greedy and sampled."""
    from pretrained_rstr_b200 import generate_batch, load_lm
    raw, seed = TINY["A"]
    folder = folders[("A", "float32")]
    few = load_lm(folder, gpu=True, dtype="float32", max_lanes=8)
    many = load_lm(folder, gpu=True, dtype="float32", max_lanes=128, max_batched_tokens=1024)
    prompts = [random_tokens(3 + i % 17, raw["vocab_size"], 100 + i) for i in range(100)]
    assert generate_batch(many, prompts, 10) == generate_batch(few, prompts, 10)
    assert many.engine.ahead["used"] > 0
    sampling = {"temperature": 0.8, "top_k": 20, "seed": 3}
    assert generate_batch(many, prompts, 10, sampling) == generate_batch(few, prompts, 10, sampling)
