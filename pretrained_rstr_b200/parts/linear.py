"""A linear map y = act(a . W^T + b) (+ residual): the building block of mixers,
feed-forwards and the head.

Weights are kept ``[out, in]`` with the input dimension contiguous, whatever layout
the checkpoint uses (GPT-2 stores Conv1D ``[in, out]``; the reference transposes it at
load time too, ``dev/examples/gpt2.clj:27-36``), in the runtime's element type.
Biases stay float32: they are added to the 32-bit accumulator.

float32 runtime: the true 32-bit FMA kernel.  bfloat16 runtime: the tensor-core
kernel with its fused epilogue.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops


class Linear:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor], runtime):
        if weight.dim() != 2:
            raise ValueError("Linear weight must be [out, in]")
        self.weight = weight.to(runtime.dtype).contiguous()
        self.bias = None if bias is None else bias.to(torch.float32).contiguous()
        self.n_out, self.n_in = self.weight.shape
        self.runtime = runtime

    @classmethod
    def from_store(cls, store, name: str, layout: str, n_in: int, n_out: int, bias: bool,
                   runtime) -> "Linear":
        w = store.get(name + ".weight")
        if layout == "in_out":
            if tuple(w.shape) != (n_in, n_out):
                raise ValueError(f"{name}.weight: expected [{n_in}, {n_out}], found {list(w.shape)}")
            w = w.to(runtime.dtype).t().contiguous()
        elif layout == "out_in":
            if tuple(w.shape) != (n_out, n_in):
                raise ValueError(f"{name}.weight: expected [{n_out}, {n_in}], found {list(w.shape)}")
        else:
            raise ValueError(f"unknown weight layout {layout!r}")
        b = store.get(name + ".bias") if bias else None
        return cls(w, b, runtime)

    def forward(self, ctx, a: torch.Tensor, out: torch.Tensor, act: Optional[str] = None,
                resid: Optional[torch.Tensor] = None) -> None:
        """out = act(a . W^T + bias) (+ resid).  ``out`` may be float32 (then ``resid`` may
        alias it) or the activation type."""
        if self.runtime.dtype == torch.float32:
            ops.gemm_f32(out, a, self.weight, self.bias, resid, act)
            return
        gemm_bf16(ctx, out, a, self.weight, self.bias, resid, act)


def gemm_bf16(ctx, out, a, weight, bias, resid, act) -> None:
    """bfloat16 operands, float32 accumulation in tensor memory, epilogue in float32."""
    ops.gemm_bf16(out, a, weight, bias, resid, act, status=ctx.status)
