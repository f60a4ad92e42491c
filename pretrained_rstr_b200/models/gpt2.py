"""GPT-2 as data for the engine: tensor names and shapes, random initialisation, and
registration under its Hugging Face identifiers.

The model itself is not written here: :func:`pretrained_rstr_b200.models.assembly.build_model`
puts it together from the parts that ``GPT2Config.layer_specs()`` names.  Tensor names
are the bare Hugging Face ones the reference reads (``dev/examples/gpt2.clj:183-210``):
``wte.weight``, ``wpe.weight``, ``h.{i}.ln_1.*``, ``h.{i}.attn.c_attn.*``,
``h.{i}.attn.c_proj.*``, ``h.{i}.ln_2.*``, ``h.{i}.mlp.c_fc.*``, ``h.{i}.mlp.c_proj.*``,
``ln_f.*``; linear weights are in Conv1D ``[in, out]`` layout (``gpt2.clj:27-36``).
"""
from __future__ import annotations

import math
import re
from typing import Dict

import torch

from ..config.gpt2 import GPT2Config
from ..config.registry import Architecture, register_architecture
from ..weights.loader import TensorExpectation, normal

STRIP_PREFIXES = ("transformer.",)

_BUFFER_RE = re.compile(r"^h\.\d+\.attn\.(bias|masked_bias)$")


def ignorable(name: str) -> bool:
    """Tensors a GPT-2 checkpoint may carry that are not parameters: the causal-mask
    buffers and a stored copy of the tied output head."""
    return bool(_BUFFER_RE.match(name)) or name == "lm_head.weight"


def expected_tensors(cfg: GPT2Config) -> Dict[str, TensorExpectation]:
    d, f = cfg.n_embd, cfg.n_inner
    exp: Dict[str, TensorExpectation] = {
        "wte.weight": TensorExpectation((cfg.vocab_size, d)),
        "wpe.weight": TensorExpectation((cfg.n_positions, d)),
        "ln_f.weight": TensorExpectation((d,)),
        "ln_f.bias": TensorExpectation((d,)),
    }
    for i in range(cfg.n_layer):
        p = f"h.{i}."
        exp.update({
            p + "ln_1.weight": TensorExpectation((d,)),
            p + "ln_1.bias": TensorExpectation((d,)),
            p + "attn.c_attn.weight": TensorExpectation((d, 3 * d)),
            p + "attn.c_attn.bias": TensorExpectation((3 * d,)),
            p + "attn.c_proj.weight": TensorExpectation((d, d)),
            p + "attn.c_proj.bias": TensorExpectation((d,)),
            p + "ln_2.weight": TensorExpectation((d,)),
            p + "ln_2.bias": TensorExpectation((d,)),
            p + "mlp.c_fc.weight": TensorExpectation((d, f)),
            p + "mlp.c_fc.bias": TensorExpectation((f,)),
            p + "mlp.c_proj.weight": TensorExpectation((f, d)),
            p + "mlp.c_proj.bias": TensorExpectation((d,)),
        })
    return exp


def random_tensors(cfg: GPT2Config, seed: int) -> Dict[str, torch.Tensor]:
    """Seeded initialisation: matrices and tables N(0, 0.02); both ``c_proj`` matrices
    N(0, 0.02/sqrt(2 L)); biases N(0, 0.02); norm gains 1 + N(0, 0.02), norm biases
    N(0, 0.02).  Every tensor has a generator of its own, keyed by (seed, name)."""
    out: Dict[str, torch.Tensor] = {}
    proj_std = 0.02 / math.sqrt(2.0 * cfg.n_layer)
    for name, exp in expected_tensors(cfg).items():
        if re.search(r"ln_(1|2|f)\.weight$", name):
            out[name] = normal(seed, name, exp.shape, 0.02, mean=1.0)
        elif name.endswith("c_proj.weight"):
            out[name] = normal(seed, name, exp.shape, proj_std)
        else:
            out[name] = normal(seed, name, exp.shape, 0.02)
    return out


_IDS = {"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2"}
#: Sizes a random-weight model can be asked for by name: the two tiny test configurations
#: and the layer sizes of GPT-2 small, medium and XL.
NAMED_SIZES = {
    "tiny-a": dict(_IDS, n_layer=2, n_embd=64, n_head=4, n_inner=256, vocab_size=512,
                   n_positions=128),
    "tiny-b": dict(_IDS, n_layer=3, n_embd=96, n_head=3, n_inner=320, vocab_size=1000,
                   n_positions=256, layer_norm_epsilon=1e-6, activation_function="gelu",
                   scale_attn_by_inverse_layer_idx=True),
    "small": dict(_IDS, n_layer=12, n_embd=768, n_head=12, n_inner=3072, vocab_size=50257,
                  n_positions=1024),
    "medium": dict(_IDS, n_layer=24, n_embd=1024, n_head=16, n_inner=4096, vocab_size=50257,
                   n_positions=1024),
    "xl": dict(_IDS, n_layer=48, n_embd=1600, n_head=25, n_inner=6400, vocab_size=50257,
               n_positions=1024),
}


def build(cfg: GPT2Config, store, runtime):
    from .assembly import build_model
    return build_model(cfg, store, runtime)


ARCHITECTURE = Architecture(
    name="GPT-2",
    config_class=GPT2Config,
    build=build,
    expected_tensors=expected_tensors,
    random_tensors=random_tensors,
    strip_prefixes=STRIP_PREFIXES,
    ignorable=ignorable,
    named_sizes=NAMED_SIZES,
)
register_architecture(GPT2Config.identifiers, ARCHITECTURE)
