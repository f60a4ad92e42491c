"""GPT-2 configuration: the keys of a GPT-2 ``config.json`` as a typed object.

The reference reads ``n_embd``, ``n_inner`` (null -> 4*n_embd), ``n_layer``, ``n_head``,
``vocab_size`` and ``n_positions`` (``dev/examples/gpt2.clj:176-217``) and fixes the
LayerNorm epsilon at 1e-5 in code (``gpt2.clj:152,160,240``).  Here every one of them,
and the remaining GPT-2 keys that change arithmetic (``layer_norm_epsilon``,
``activation_function``, ``scale_attn_weights``, ``scale_attn_by_inverse_layer_idx``),
is read from the file.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List

from .base import (ConfigError, LayerSpec, ModelConfig, PartSpec, _require_bool,
                   _require_float, _require_int)

_ACTIVATIONS = ("gelu_new", "gelu", "gelu_pytorch_tanh", "relu")


@dataclass(frozen=True)
class GPT2Config(ModelConfig):
    n_layer: int
    n_embd: int
    n_head: int
    n_inner: int
    vocab_size: int
    n_positions: int
    layer_norm_epsilon: float = 1e-5
    activation_function: str = "gelu_new"
    scale_attn_weights: bool = True
    scale_attn_by_inverse_layer_idx: bool = False

    identifiers = ("GPT2LMHeadModel", "gpt2")

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "GPT2Config":
        n_embd = _require_int(raw, "n_embd")
        n_inner = raw.get("n_inner")
        if n_inner is None:                      # gpt2.clj:179
            n_inner = 4 * n_embd
        else:
            n_inner = _require_int(raw, "n_inner")
        act = raw.get("activation_function", "gelu_new")
        if act not in _ACTIVATIONS:
            raise ConfigError(
                f"config.json: unknown activation_function {act!r}; known: {list(_ACTIVATIONS)}")
        if raw.get("tie_word_embeddings", True) is not True:
            raise ConfigError("config.json: GPT-2 ties lm_head to wte; "
                              "tie_word_embeddings=false is not supported")
        cfg = cls(
            n_layer=_require_int(raw, "n_layer"),
            n_embd=n_embd,
            n_head=_require_int(raw, "n_head"),
            n_inner=n_inner,
            vocab_size=_require_int(raw, "vocab_size"),
            n_positions=_require_int(raw, "n_positions"),
            layer_norm_epsilon=_require_float(raw, "layer_norm_epsilon", 1e-5),
            activation_function=act,
            scale_attn_weights=_require_bool(raw, "scale_attn_weights", True),
            scale_attn_by_inverse_layer_idx=_require_bool(
                raw, "scale_attn_by_inverse_layer_idx", False),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.n_embd % self.n_head != 0:
            raise ConfigError(
                f"config.json: n_embd={self.n_embd} is not divisible by n_head={self.n_head}")
        if self.layer_norm_epsilon <= 0.0:
            raise ConfigError("config.json: layer_norm_epsilon must be positive")

    def to_dict(self) -> Dict[str, Any]:
        return {
            "architectures": ["GPT2LMHeadModel"],
            "model_type": "gpt2",
            "n_layer": self.n_layer,
            "n_embd": self.n_embd,
            "n_head": self.n_head,
            "n_inner": self.n_inner,
            "vocab_size": self.vocab_size,
            "n_positions": self.n_positions,
            "layer_norm_epsilon": self.layer_norm_epsilon,
            "activation_function": self.activation_function,
            "scale_attn_weights": self.scale_attn_weights,
            "scale_attn_by_inverse_layer_idx": self.scale_attn_by_inverse_layer_idx,
            "tie_word_embeddings": True,
        }

    # ------------------------------------------------------------------ derived
    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    def attention_scale(self, layer: int) -> float:
        """Score multiplier of ``layer``: 1/sqrt(head size) when ``scale_attn_weights``
        (the reference's decoders use 1/sqrt(head_dim): ``src/pretrained/decoder.clj:56``),
        divided by (layer+1) when ``scale_attn_by_inverse_layer_idx``."""
        scale = 1.0
        if self.scale_attn_weights:
            scale /= float(self.head_dim) ** 0.5
        if self.scale_attn_by_inverse_layer_idx:
            scale /= float(layer + 1)
        return scale

    # ---------------------------------------------------------------- structure
    def layer_specs(self) -> List[LayerSpec]:
        """Pre-LN blocks: LN -> causal MHA -> add -> LN -> MLP -> add
        (``dev/examples/gpt2.clj:149-166``)."""
        specs = []
        for i in range(self.n_layer):
            p = f"h.{i}."
            norm = {"size": self.n_embd, "eps": self.layer_norm_epsilon}
            specs.append(LayerSpec(
                prefix=p,
                arrangement="pre_norm",
                mixer=PartSpec("causal_attention", {
                    "weights": {"qkv": p + "attn.c_attn", "out": p + "attn.c_proj"},
                    "width": self.n_embd,
                    "n_head": self.n_head,
                    "n_kv_head": self.n_head,
                    "head_dim": self.head_dim,
                    "scale": self.attention_scale(i),
                    "window": None,
                    "bias": True,
                    "weight_layout": "in_out",
                }),
                feed_forward=PartSpec("dense_mlp", {
                    "weights": {"up": p + "mlp.c_fc", "down": p + "mlp.c_proj"},
                    "width": self.n_embd,
                    "inner": self.n_inner,
                    "activation": self.activation_function,
                    "bias": True,
                    "weight_layout": "in_out",
                }),
                norms={"mixer": PartSpec("layer_norm", {"weights": p + "ln_1", **norm}),
                       "feed_forward": PartSpec("layer_norm", {"weights": p + "ln_2", **norm})},
                width=self.n_embd,
            ))
        return specs

    def embedding_spec(self) -> PartSpec:
        return PartSpec("token_embedding", {
            "weights": "wte", "vocab": self.vocab_size, "width": self.n_embd})

    def position_spec(self) -> PartSpec:
        return PartSpec("learned_absolute", {
            "weights": "wpe", "positions": self.n_positions, "width": self.n_embd})

    def final_norm_spec(self) -> PartSpec:
        return PartSpec("layer_norm", {
            "weights": "ln_f", "size": self.n_embd, "eps": self.layer_norm_epsilon})

    def head_spec(self) -> PartSpec:
        return PartSpec("tied_head", {
            "weights": "wte", "vocab": self.vocab_size, "width": self.n_embd})

    @property
    def max_positions(self) -> int:
        return self.n_positions
