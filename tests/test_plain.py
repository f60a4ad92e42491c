"""The plain implementation itself: each part against an independent statement of its
formula, and the oracle against a float64 run of itself."""
import math

import pytest
import torch

import plain_gpt2
from helpers import TINY, make_folder, random_tokens


def test_layer_norm_and_gelu():
    torch.manual_seed(0)
    x, g, b = torch.randn(5, 96), torch.randn(96), torch.randn(96)
    ours = plain_gpt2.layer_norm(x, g, b, 1e-6)
    assert torch.allclose(ours, torch.nn.functional.layer_norm(x, (96,), g, b, 1e-6), atol=1e-5)
    u = torch.linspace(-4, 4, 41)
    assert torch.allclose(plain_gpt2.gelu_new(u), torch.nn.functional.gelu(u, approximate="tanh"),
                          atol=1e-6)
    assert torch.allclose(plain_gpt2.gelu_erf(u), torch.nn.functional.gelu(u), atol=1e-6)


def test_attention_is_causal_and_windowed():
    torch.manual_seed(1)
    d, h = 32, 2
    x = torch.randn(9, d)
    w, b = torch.randn(d, 3 * d) * 0.2, torch.randn(3 * d) * 0.1
    wo, bo = torch.randn(d, d) * 0.2, torch.randn(d) * 0.1
    full = plain_gpt2.causal_attention(x, w, b, wo, bo, h, 0.25)
    short = plain_gpt2.causal_attention(x[:5], w, b, wo, bo, h, 0.25)
    assert torch.allclose(full[:5], short, atol=1e-6)            # the future is invisible
    win = plain_gpt2.causal_attention(x, w, b, wo, bo, h, 0.25, window=3)
    tail = plain_gpt2.causal_attention(x[6:], w, b, wo, bo, h, 0.25)
    assert torch.allclose(win[8], tail[2], atol=1e-6)            # token 8 sees 6, 7, 8 only
    assert not torch.allclose(win[8], full[8], atol=1e-4)


def test_sampler_pieces():
    row = torch.tensor([0.1, 2.0, 2.0, -1.0, 3.0])
    assert plain_gpt2.argmax(torch.tensor([1.0, 5.0, 5.0])) == 1     # ties -> lowest id
    assert plain_gpt2.top_k_ids(row, 3) == [4, 1, 2]
    r = plain_gpt2.JavaRandom(42)
    # java.util.Random(42).nextDouble() per its documented recurrence
    assert r.next_double() == pytest.approx(0.7275636800328681, abs=1e-15)
    assert plain_gpt2.sample(row, 0.0, None, None, None) == 4
    picks = {plain_gpt2.sample(row, 1.0, 2, None, plain_gpt2.JavaRandom(s)) for s in range(40)}
    assert picks == {4, 1}                                          # only the top two
    assert plain_gpt2.sample(row, 1.0, 5, 0.1, plain_gpt2.JavaRandom(3)) == 4   # nucleus of one


@pytest.mark.parametrize("name", ["A", "B"])
def test_oracle_against_float64_and_greedy(tmp_path, name):
    raw, seed = TINY[name]
    folder = make_folder(str(tmp_path / name), raw, seed, "float32")
    ids = random_tokens(raw["n_positions"], raw["vocab_size"], 9)
    m32 = plain_gpt2.PlainGPT2(folder)
    m64 = plain_gpt2.PlainGPT2(folder, dtype=torch.float64)
    a, b = plain_gpt2.all_logits(m32, ids), plain_gpt2.all_logits(m64, ids)
    assert float((a.double() - b.double()).abs().max()) < 5e-6
    # prefix property: logits of a prefix equal the first rows of the whole
    assert torch.allclose(plain_gpt2.all_logits(m32, ids[:11]), a[:11], atol=2e-6)
    out = plain_gpt2.greedy_generate(m32, ids[:4], 3)
    assert len(out) == 3 and out[0] == int(plain_gpt2.all_logits(m32, ids[:4])[-1].argmax())
    with pytest.raises(ValueError, match="n_positions"):
        plain_gpt2.all_logits(m32, ids + [0])
