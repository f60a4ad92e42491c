"""The plain implementation against a second one written apart from it: tests/scalar_gpt2.cpp,
scalar C++ in double precision with its own readers of config.json and model.safetensors.

The reference's own model code cannot run here (Clojure on the JVM over an external library),
and model code of installed packages is not a source for this suite, so the anchor is
agreement of two independent statements of the reference's formulas: every logit of the
tiny configurations, and of variants that flip one option each (no score scale, n_inner
left null, ReLU), must agree with the plain implementation's float64 run to 1e-9."""
import json
import os
import shutil
import subprocess

import numpy as np
import pytest
import torch

import plain_gpt2
from helpers import TINY, make_folder, random_tokens

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def scalar(tmp_path_factory):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++ to build the scalar implementation with")
    exe = str(tmp_path_factory.mktemp("scalar") / "scalar_gpt2")
    subprocess.run([gxx, "-O2", "-std=c++17", "-o", exe, os.path.join(HERE, "scalar_gpt2.cpp")],
                   check=True, capture_output=True, text=True)
    return exe


VARIANTS = {
    "A": {}, "B": {}, "C": {},
    "A-unscaled": {"scale_attn_weights": False},
    "B-inner-null": {"n_inner": None, "activation_function": "relu"},
    "A-bfloat16-weights": {},
}


@pytest.mark.parametrize("variant", sorted(VARIANTS))
def test_every_logit_agrees_with_the_scalar_implementation(tmp_path, scalar, variant):
    name = variant[0]
    raw, seed = TINY[name]
    raw = dict(raw, **VARIANTS[variant])
    n = {"A": 70, "B": 90, "C": 150}[name]
    if raw.get("n_inner", 0) is None:
        # the configuration class fills the default in; write the null back so that both
        # implementations have to apply it themselves
        folder = make_folder(str(tmp_path / "m"), dict(raw, n_inner=4 * raw["n_embd"]), seed, "float32")
        with open(os.path.join(folder, "config.json")) as fh:
            cfg = json.load(fh)
        cfg["n_inner"] = None
        with open(os.path.join(folder, "config.json"), "w") as fh:
            json.dump(cfg, fh)
    else:
        folder = make_folder(str(tmp_path / "m"), raw, seed,
                             "bfloat16" if "bfloat16" in variant else "float32")
    ids = random_tokens(n, raw["vocab_size"], 17)
    out = str(tmp_path / "logits.f64")
    proc = subprocess.run([scalar, folder, out] + [str(t) for t in ids], capture_output=True,
                          text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr
    got = torch.from_numpy(np.fromfile(out, dtype="<f8").reshape(n, raw["vocab_size"]))
    m64 = plain_gpt2.PlainGPT2(folder, dtype=torch.float64)
    want = plain_gpt2.logits(m64, plain_gpt2.forward(m64, ids))
    assert want.dtype == torch.float64
    assert float((got - want).abs().max()) <= 1e-9
    # and the float32 oracle the engine is compared with stays within rounding of both
    m32 = plain_gpt2.PlainGPT2(folder)
    assert float((plain_gpt2.all_logits(m32, ids).double() - got).abs().max()) <= 1e-5
