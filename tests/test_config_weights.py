"""Configuration, registry and weight loading (no GPU)."""
import json
import os

import pytest
import torch

from helpers import TINY_A, TINY_B, make_folder
from pretrained_rstr_b200.config import (ConfigError, GPT2Config, lookup, read_config, registered)
from pretrained_rstr_b200.models import gpt2 as gpt2_arch
from pretrained_rstr_b200.weights import (SafetensorsFile, WeightError, load_file, load_weights,
                                          save_file)


def test_config_reads_every_key():
    a, b = GPT2Config.from_dict(TINY_A), GPT2Config.from_dict(TINY_B)
    assert (a.n_layer, a.n_embd, a.n_head, a.n_inner, a.vocab_size, a.n_positions) == \
        (2, 64, 4, 256, 512, 128)
    assert a.head_dim == 16 and b.head_dim == 32
    assert b.layer_norm_epsilon == 1e-6 and b.activation_function == "gelu"
    assert a.attention_scale(1) == pytest.approx(0.25)
    assert b.attention_scale(2) == pytest.approx(1 / (32 ** 0.5) / 3)
    assert GPT2Config.from_dict({**TINY_A, "scale_attn_weights": False}).attention_scale(0) == 1.0


def test_config_defaults_and_errors():
    raw = {k: v for k, v in TINY_A.items()
           if k not in ("n_inner", "layer_norm_epsilon", "activation_function")}
    c = GPT2Config.from_dict(raw)
    assert c.n_inner == 4 * c.n_embd and c.layer_norm_epsilon == 1e-5
    assert c.activation_function == "gelu_new"
    assert GPT2Config.from_dict({**TINY_A, "n_inner": None}).n_inner == 256
    with pytest.raises(ConfigError, match="n_head"):
        GPT2Config.from_dict({**TINY_A, "n_head": 5})
    with pytest.raises(ConfigError, match="missing required key 'n_layer'"):
        GPT2Config.from_dict({k: v for k, v in TINY_A.items() if k != "n_layer"})
    with pytest.raises(ConfigError, match="activation"):
        GPT2Config.from_dict({**TINY_A, "activation_function": "swish"})
    with pytest.raises(ConfigError, match="integer"):
        GPT2Config.from_dict({**TINY_A, "vocab_size": "512"})
    assert GPT2Config.from_dict(c.to_dict()) == c


def test_layer_specs_are_data():
    c = GPT2Config.from_dict(TINY_B)
    specs = c.layer_specs()
    assert len(specs) == 3
    assert specs[2].mixer.kind == "causal_attention" and specs[2].feed_forward.kind == "dense_mlp"
    assert specs[2].mixer.params["scale"] == pytest.approx(c.attention_scale(2))
    assert specs[0].feed_forward.params["inner"] == 320
    assert [(e.layer, e.cache_layer, e.writes_cache) for e in c.run_order()] == \
        [(0, 0, True), (1, 1, True), (2, 2, True)]


def test_registry_lookup_order_and_miss(tmp_path):
    assert set(registered()) >= {"GPT2LMHeadModel", "gpt2"}
    assert lookup({"architectures": ["Nope", "GPT2LMHeadModel"]}).name == "GPT-2"
    assert lookup({"model_type": "gpt2"}).name == "GPT-2"
    with pytest.raises(ConfigError, match="known: .*GPT2LMHeadModel"):
        lookup({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})
    folder = make_folder(str(tmp_path / "m"), TINY_A, 0, "float32")
    arch, cfg = read_config(folder)
    assert arch.name == "GPT-2" and cfg.n_embd == 64
    with pytest.raises(ConfigError, match="no config.json"):
        read_config(str(tmp_path))


def test_safetensors_roundtrip(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
         "c": torch.arange(6, dtype=torch.int64).view(2, 3), "d": torch.zeros(0, 4)}
    path = str(tmp_path / "x.safetensors")
    save_file(t, path)
    back = load_file(path)
    for k in t:
        assert back[k].dtype == t[k].dtype and torch.equal(back[k], t[k])
    from safetensors.torch import load_file as theirs        # the format, not just our reader
    other = theirs(path)
    assert all(torch.equal(other[k], t[k]) for k in t)
    f = SafetensorsFile(path)
    with pytest.raises(ValueError, match="tensor not found"):
        f.tensor("zzz")


def test_random_model_is_seeded_and_storage_precision_kept(tmp_path):
    f1 = make_folder(str(tmp_path / "a"), TINY_A, 0, "float32")
    f2 = make_folder(str(tmp_path / "b"), TINY_A, 0, "float32")
    f3 = make_folder(str(tmp_path / "c"), TINY_A, 1, "float32")
    a, b, c = (load_file(os.path.join(f, "model.safetensors")) for f in (f1, f2, f3))
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["wte.weight"], c["wte.weight"])
    assert abs(float(a["h.0.ln_1.weight"].mean()) - 1.0) < 0.02
    assert float(a["h.0.attn.c_proj.weight"].std()) == pytest.approx(0.02 / 2.0, rel=0.15)
    cfg = GPT2Config.from_dict(TINY_A)
    store = load_weights(f1, gpt2_arch.expected_tensors(cfg), "cpu")
    assert store.get("wte.weight").dtype == torch.float32          # stored 32-bit stays 32-bit
    fb = make_folder(str(tmp_path / "d"), TINY_A, 0, "bfloat16")
    store = load_weights(fb, gpt2_arch.expected_tensors(cfg), "cpu")
    assert store.get("wte.weight").dtype == torch.bfloat16
    assert store.get("h.1.mlp.c_fc.weight").shape == (64, 256)
    # a float16 checkpoint is kept as it is until a part converts it to the runtime's type:
    # widened to float32 it loses no bits (it is not rounded to bfloat16 on the way)
    from pretrained_rstr_b200.weights import save_file
    half = {k: v.to(torch.float16) for k, v in a.items()}
    os.makedirs(tmp_path / "h")
    cfg.save(str(tmp_path / "h"))
    save_file(half, str(tmp_path / "h" / "model.safetensors"))
    store = load_weights(str(tmp_path / "h"), gpt2_arch.expected_tensors(cfg), "cpu")
    assert store.get("wte.weight").dtype == torch.float16
    assert torch.equal(store.get("wte.weight", torch.float32), half["wte.weight"].float())


def test_weight_errors_list_everything_at_once(tmp_path):
    cfg = GPT2Config.from_dict(TINY_A)
    folder = make_folder(str(tmp_path / "m"), TINY_A, 0, "float32")
    path = os.path.join(folder, "model.safetensors")
    t = load_file(path)
    del t["h.1.ln_2.bias"], t["wpe.weight"]
    t["h.0.attn.c_attn.weight"] = torch.zeros(64, 128)
    t["extra.weight"] = torch.zeros(2)
    t["h.0.attn.bias"] = torch.ones(1, 1, 8, 8)                   # a mask buffer: ignorable
    t["lm_head.weight"] = t["wte.weight"].clone()                 # tied copy: ignorable
    t["ln_f.bias"] = torch.zeros(64, dtype=torch.int32)
    save_file(t, path)
    with pytest.raises(WeightError) as err:
        load_weights(folder, gpt2_arch.expected_tensors(cfg), "cpu",
                     strip_prefixes=gpt2_arch.STRIP_PREFIXES, ignorable=gpt2_arch.ignorable)
    e = err.value
    assert e.missing == ["h.1.ln_2.bias", "wpe.weight"]
    assert e.unexpected == ["extra.weight"]
    assert len(e.wrong) == 2 and "expected [64, 192], found [64, 128]" in e.wrong[0]
    msg = str(e)
    assert "missing (2)" in msg and "unexpected (1)" in msg and "wrong shape or type (2)" in msg


def test_transformer_prefix_is_stripped(tmp_path):
    cfg = GPT2Config.from_dict(TINY_A)
    folder = make_folder(str(tmp_path / "m"), TINY_A, 0, "float32")
    path = os.path.join(folder, "model.safetensors")
    save_file({"transformer." + k: v for k, v in load_file(path).items()}, path)
    store = load_weights(folder, gpt2_arch.expected_tensors(cfg), "cpu",
                         strip_prefixes=gpt2_arch.STRIP_PREFIXES)
    assert "wte.weight" in store
    with pytest.raises(WeightError, match="file does not exist"):
        load_weights(str(tmp_path), gpt2_arch.expected_tensors(cfg), "cpu")
