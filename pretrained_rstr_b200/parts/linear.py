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
        if runtime.dtype != torch.float32 and self.n_in % 8 != 0:
            # the tensor-core kernels read rows in 16-byte pieces; said here, when the model
            # is built, rather than by the first step
            raise ValueError(f"a {str(runtime.dtype).replace('torch.', '')} product needs an input "
                             f"width that is a multiple of 8; this one has {self.n_in} "
                             f"(float32 takes any width)")

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

    def forward(self, ctx, a, out: torch.Tensor, act: Optional[str] = None,
                resid: Optional[torch.Tensor] = None, kv_scatter=None) -> bool:
        """out = act(a . W^T + bias) (+ resid).  ``out`` may be float32 (then ``resid`` may
        alias it) or the activation type.  ``a`` is a tensor, or a :class:`LazyNorm`: a
        norm that has not run yet, which the decode-time kernel computes in its prologue
        and every other kernel asks to run first.  ``kv_scatter`` = (k_pages, v_pages, slots,
        q_width[, only_cache]) offers the kernel the chance to write the key and value columns of a fused
        QKV product straight to the cache; returns True when it did."""
        m = out.shape[0]
        if self.runtime.dtype == torch.float32:
            ops.gemm_f32(out, _tensor(a), self.weight, self.bias, resid, act)
            return False
        # Which kernel (measured on GPT-2 small and XL shapes): up to 16 rows
        # the weight-streaming kernel with the norm fused into it; 17 to 64 rows the cluster
        # split-K kernel for narrow outputs and long reductions, the tensor-memory kernel for
        # wide outputs (the register-streaming kernel where K is no multiple of 64); beyond
        # 64 rows the tensor-memory kernel.
        max_rows, max_norm = ops.smallm_limits()
        if 16 < m <= 64 and (self.n_out <= 2048 or self.n_in >= 4 * self.n_out) and \
                ops.midm_supports(m, self.n_out, self.n_in):
            # narrow outputs or long reductions at a few dozen rows: the reduction split over
            # a thread-block cluster (measured against the other two kernels)
            ops.gemm_midm(out, _tensor(a), self.weight, self.bias, resid, act, status=ctx.status)
            return False
        if m <= max_rows and self.n_in % 8 == 0 and (m <= 16 or self.n_out <= 1024):
            if kv_scatter is not None and kv_scatter[0].dtype != out.dtype:
                kv_scatter = None
            if m <= 16 and isinstance(a, LazyNorm) and a.fusable and self.n_in <= max_norm:
                ops.gemm_smallm(out, self.weight, norm_input=a.x, gamma=a.norm.gamma,
                                beta=a.norm.beta, eps=a.norm.eps, bias=self.bias, resid=resid,
                                act=act, kv_scatter=kv_scatter, status=ctx.status,
                                norm_rows=a.rows)
            else:
                ops.gemm_smallm(out, self.weight, a=_tensor(a), bias=self.bias, resid=resid,
                                act=act, kv_scatter=kv_scatter, status=ctx.status)
            return kv_scatter is not None
        if kv_scatter is not None and (kv_scatter[0].dtype != out.dtype or resid is not None or
                                       kv_scatter[0].shape[3] % 8 != 0 or kv_scatter[3] % 8 != 0):
            kv_scatter = None
        ops.gemm_bf16(out, _tensor(a), self.weight, self.bias, resid, act, status=ctx.status,
                      kv_scatter=kv_scatter)
        return kv_scatter is not None


class LazyNorm:
    """A norm of ``x`` (of its rows ``rows``, if given: an int32 tensor of row indices) that
    runs when its result is first needed.  A consumer that can compute the norm itself
    (``fusable``: a plain layer norm) reads ``x``, ``rows`` and ``norm`` instead and the norm
    never runs as a kernel of its own."""

    def __init__(self, ctx, norm, x: torch.Tensor, out: torch.Tensor, rows=None):
        self.ctx, self.norm, self.x, self._out, self.rows = ctx, norm, x, out, rows
        self._done = False
        self.fusable = all(hasattr(norm, f) for f in ("gamma", "beta", "eps")) and \
            getattr(norm, "kind", "") == "layer_norm"
        self.shape = out.shape

    def tensor(self) -> torch.Tensor:
        if not self._done:
            if self.rows is None:
                self.norm.forward(self.ctx, self.x, self._out)
            else:
                self.norm.forward(self.ctx, self.x, self._out, rows=self.rows)
            self._done = True
        return self._out


def _tensor(a) -> torch.Tensor:
    return a.tensor() if isinstance(a, LazyNorm) else a
