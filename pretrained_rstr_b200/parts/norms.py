"""Norms.  ``layer_norm``: mean-centred, biased variance, gain and bias, statistics in
32-bit (call sites ``dev/examples/gpt2.clj:152,160,240``; formula
``src/pretrained/asr/moonshine.clj:87-104``).  Size and eps are parameters."""
from __future__ import annotations

import torch

from ..csrc import ops
from .interfaces import Norm
from .registry import register_part


class LayerNorm(Norm):
    graph_safe = True
    kind = "layer_norm"
    def __init__(self, gamma: torch.Tensor, beta, eps: float, size: int):
        if gamma.numel() != size or (beta is not None and beta.numel() != size):
            raise ValueError(f"layer_norm: gain/bias size differs from {size}")
        self.gamma = gamma.to(torch.float32).contiguous()
        self.beta = None if beta is None else beta.to(torch.float32).contiguous()
        self.eps = float(eps)
        self.size = size

    def forward(self, ctx, x, out, rows=None) -> None:
        ops.layernorm(out, x, self.gamma, self.beta, self.eps, rows=rows, status=ctx.status)


def _layer_norm(params, store, runtime) -> LayerNorm:
    name = params["weights"]
    beta = store.get(name + ".bias") if params.get("bias", True) else None
    return LayerNorm(store.get(name + ".weight"), beta, params["eps"], params["size"])


register_part("norm", "layer_norm", _layer_norm)
