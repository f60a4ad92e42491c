"""Python face of the CUDA library: loads it (building it on first use) and wraps each
exported C function in a call that takes torch tensors.

There is no fallback: if the library cannot be built or loaded, or no CUDA device is
present, :func:`lib` raises :class:`ExtensionError`.  Wrappers check devices, element
types and contiguity, pass raw pointers and the current torch stream, and turn a
non-zero return code into an exception that names the refused argument.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_long, c_void_p
from typing import Optional

import torch

from . import build as _build

F32, BF16 = 0, 1
ACT_CODES = {None: 0, "none": 0, "gelu_new": 1, "gelu_pytorch_tanh": 1, "gelu": 2, "relu": 3}

_ERRORS = {
    -2: "unknown element type",
    -3: "a size this kernel does not take",
    -4: "a pointer or stride that is not aligned as the kernel requires",
    -5: "bad argument",
    -6: "the device or driver lacks a feature the kernel needs",
}
STATUS_TEXT = {
    1: "token id outside the vocabulary (token index, id, vocabulary size)",
    2: "position outside the position table or the cache (token index, position, limit)",
    3: "cache slot outside the pool (token index, slot, pages)",
    4: "block-table entry missing or outside the pool (token index, position, page)",
    5: "a bounded wait inside a kernel gave up (kernel id, block, stage)",
    6: "row index outside its tensor (row, index, rows)",
}


class ExtensionError(RuntimeError):
    pass


class KernelArgumentError(ValueError):
    pass


_LIB = None


def lib() -> ctypes.CDLL:
    """The loaded library; builds it at the first call."""
    global _LIB
    if _LIB is None:
        try:
            path = _build.build()
            handle = ctypes.CDLL(path)
        except (OSError, _build.BuildError) as exc:
            raise ExtensionError(
                f"the CUDA extension of pretrained_rstr_b200 is not available: {exc}") from exc
        _declare(handle)
        _LIB = handle
    return _LIB


def library_path() -> str:
    return _build.build()


def require_cuda() -> None:
    if not torch.cuda.is_available():
        raise ExtensionError("pretrained_rstr_b200 runs on a CUDA device only (sm_100a); "
                             "torch.cuda.is_available() is False and there is no CPU path")


def _declare(h: ctypes.CDLL) -> None:
    P, I, L, F = c_void_p, c_int, c_long, c_float
    h.prb_embed.argtypes = [P, P, P, P, P, I, I, I, I, I, P, P]
    h.prb_layernorm.argtypes = [P, P, P, P, P, I, I, I, F, I, P, P]
    h.prb_bias_act.argtypes = [P, P, P, P, I, I, I, I, I, P]
    h.prb_kv_append.argtypes = [P, P, P, P, L, P, I, I, I, I, I, I, P, P]
    h.prb_copy_pages.argtypes = [P, P, I, L, I, I, P, P]
    h.prb_resolve_tokens.argtypes = [P, I, P, I, P, P]
    h.prb_host_device_address.argtypes = [P]
    h.prb_host_device_address.restype = c_void_p
    h.prb_fetch_step.argtypes = [P, P, I, I, I, P, I, P, P]
    h.prb_publish_result.argtypes = [P, P, I, P]
    h.prb_gemm_f32.argtypes = [P, P, P, P, P, I, I, I, L, L, L, I, P]
    h.prb_gemm_bf16.argtypes = [P, P, P, P, P, I, I, I, L, L, L, I, I, I, P, P]
    h.prb_gemm_bf16_scatter.argtypes = [P, P, P, P, I, I, I, L, L, L, I, I, P, P, P, I, I, I, I, I,
                                        I, P, P]
    h.prb_gemm_midm.argtypes = [P, P, P, P, P, I, I, I, L, L, L, I, I, P, P]
    h.prb_gemm_midm_supports.argtypes = [I, I, I]
    h.prb_gemm_smallm.argtypes = [P, P, P, P, I, P, P, F, P, P, P, I, I, I, L, L, L, I, I,
                                  P, P, P, I, I, I, I, I, P, P]
    h.prb_gemm_smallm_max_rows.argtypes = []
    h.prb_gemm_smallm_max_norm_width.argtypes = []
    h.prb_attention_generic.argtypes = [P, L, P, L, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I,
                                        I, P, P]
    h.prb_attention_decode.argtypes = [P, L, P, L, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I,
                                       P, P, I, I, P, P]
    h.prb_attention_decode_ring.argtypes = [P, L, P, L, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F,
                                            I, I, P, P, L, P, P, I, I, P, P]
    h.prb_attention_decode_ring_tune.argtypes = [I, I]
    h.prb_attention_decode_ring_tune.restype = c_int
    h.prb_attention_decode_ring.restype = c_int
    h.prb_attention_decode_ring_supports.argtypes = [I, I]
    h.prb_attention_decode_ring_supports.restype = c_int
    h.prb_attention_decode_ring_prefers.argtypes = [I, I, I]
    h.prb_attention_decode_ring_prefers.restype = c_int
    h.prb_attention_decode_ring_max_list.argtypes = []
    h.prb_attention_decode_ring_max_list.restype = c_int
    h.prb_attention_decode_ring_workspace.argtypes = [I, I, I]
    h.prb_attention_decode_ring_workspace.restype = L
    h.prb_attention_prefill.argtypes = [P, L, P, L, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F,
                                        I, P, P]
    h.prb_attention_prefill_supports.argtypes = [I]
    h.prb_attention_prefill_tile.argtypes = []
    h.prb_attention_prefill_tc.argtypes = [P, L, P, L, I, P, P, P, P, P, P, P, P, I, I, I, I, I, I,
                                           I, F, I, I, I, P, P, P, P, P, P, P, P, I, P, P]
    h.prb_attention_prefill_tc_supports.argtypes = [I, I]
    h.prb_attention_prefill_tc_tile.argtypes = []
    h.prb_attention_decode_split.argtypes = []
    h.prb_attention_decode_max_split_pages.argtypes = []
    h.prb_attention_decode_max_split_pages.restype = c_int
    h.prb_device_sm_count.argtypes = []
    h.prb_device_sm_count.restype = c_int
    h.prb_attention_decode_set_stream.argtypes = [I]
    h.prb_attention_decode_set_stream.restype = None
    h.prb_set_pdl.argtypes = [I]
    h.prb_set_pdl.restype = None
    h.prb_sample.argtypes = [P, P, L, I, P, P, P, P, P, P, P, I, P, P, I, P, P]
    h.prb_sample_max_top_k.argtypes = []
    h.prb_sample_workspace_words.argtypes = []
    h.prb_sample_workspace_words.restype = c_int
    for name in ("prb_resolve_tokens", "prb_fetch_step", "prb_publish_result", "prb_embed", "prb_layernorm", "prb_bias_act", "prb_kv_append", "prb_copy_pages",
                 "prb_gemm_f32", "prb_gemm_bf16", "prb_gemm_bf16_scatter", "prb_gemm_midm",
                 "prb_gemm_midm_supports", "prb_gemm_smallm", "prb_gemm_smallm_max_rows",
                 "prb_gemm_smallm_max_norm_width", "prb_attention_generic", "prb_attention_decode",
                 "prb_attention_prefill", "prb_attention_prefill_supports",
                 "prb_attention_prefill_tile", "prb_attention_prefill_tc",
                 "prb_attention_prefill_tc_supports", "prb_attention_prefill_tc_tile",
                 "prb_attention_decode_split", "prb_sample", "prb_sample_max_top_k"):
        getattr(h, name).restype = c_int


# ------------------------------------------------------------------------- helpers
def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelArgumentError(f"element type {dtype} is not supported (float32 or bfloat16)")


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


_LAUNCHES = 0


def launch_count() -> int:
    """Kernels of this library launched so far through these wrappers."""
    return _LAUNCHES


def add_launches(n: int) -> None:
    """Account for kernels launched by replaying a CUDA graph that holds ``n`` of them."""
    global _LAUNCHES
    _LAUNCHES += int(n)


def _check(code: int, what: str) -> None:
    global _LAUNCHES
    if code == 0:
        _LAUNCHES += 1
        return
    if code < 0:
        raise KernelArgumentError(f"{what}: {_ERRORS.get(code, 'error')} (code {code})")
    raise ExtensionError(f"{what}: CUDA error {code} at launch")


def _need(t: torch.Tensor, dtype, name: str, what: str) -> None:
    if not t.is_cuda:
        raise KernelArgumentError(f"{what}: {name} is not on a CUDA device")
    if dtype is not None and t.dtype != dtype:
        raise KernelArgumentError(f"{what}: {name} must be {dtype}, is {t.dtype}")
    if not t.is_contiguous():
        raise KernelArgumentError(f"{what}: {name} must be contiguous")


_PDL = True


def set_pdl(on: bool) -> None:
    """Switch programmatic dependent launch of the decode-chain kernels on or off."""
    global _PDL
    _PDL = bool(on)
    lib().prb_set_pdl(1 if on else 0)


class plain_launch:
    """``with plain_launch(cond):`` kernels launched inside start only when their predecessor
    has ended (no programmatic dependent launch), if ``cond``; the setting outside is kept."""

    def __init__(self, cond: bool = True):
        self.cond = bool(cond) and _PDL

    def __enter__(self):
        if self.cond:
            lib().prb_set_pdl(0)
        return self

    def __exit__(self, *exc):
        if self.cond:
            lib().prb_set_pdl(1)
        return False


# ------------------------------------------------------------------------ kernels
def embed(out, tokens, positions, wte, wpe, status) -> None:
    """out[t,:] = wte[tokens[t],:] (+ wpe[positions[t],:]); out float32 [T, width]."""
    what = "embed"
    _need(out, torch.float32, "out", what)
    _need(tokens, torch.int32, "tokens", what)
    _need(positions, torch.int32, "positions", what)
    _need(wte, None, "wte", what)
    n, width = out.shape
    if wte.shape[1] != width or (wpe is not None and (wpe.shape[1] != width or wpe.dtype != wte.dtype)):
        raise KernelArgumentError(f"{what}: table widths or types differ from the output's")
    if tokens.numel() < n or positions.numel() < n:
        raise KernelArgumentError(f"{what}: fewer token ids or positions than output rows")
    _check(lib().prb_embed(_p(out), _p(tokens), _p(positions), _p(wte), _p(wpe), n, width,
                           wte.shape[0], 0 if wpe is None else wpe.shape[0],
                           dtype_code(wte.dtype), _p(status), _stream()), what)


def layernorm(out, x, gamma, beta, eps: float, rows=None, status=None) -> None:
    """out[r,:] = LayerNorm(x[rows[r],:] or x[r,:]); x float32, out float32 or bfloat16."""
    what = "layernorm"
    _need(x, torch.float32, "x", what)
    _need(out, None, "out", what)
    _need(gamma, torch.float32, "gamma", what)
    if beta is not None:
        _need(beta, torch.float32, "beta", what)
    n_rows, width = out.shape
    if x.shape[1] != width or gamma.numel() != width:
        raise KernelArgumentError(f"{what}: widths differ")
    if rows is None and x.shape[0] < n_rows:
        raise KernelArgumentError(f"{what}: fewer input rows than output rows")
    if rows is not None:
        _need(rows, torch.int32, "rows", what)
    _check(lib().prb_layernorm(_p(out), _p(x), _p(gamma), _p(beta), _p(rows), n_rows, x.shape[0],
                               width, float(eps), dtype_code(out.dtype), _p(status), _stream()),
           what)


def bias_act(out, inp, bias, resid, act) -> None:
    """out = act(inp + bias) (+ resid), sums in float32."""
    what = "bias_act"
    _need(out, None, "out", what)
    _need(inp, None, "inp", what)
    m, n = inp.shape
    if out.shape != inp.shape:
        raise KernelArgumentError(f"{what}: shapes differ")
    if bias is not None:
        _need(bias, torch.float32, "bias", what)
    if resid is not None:
        _need(resid, torch.float32, "resid", what)
    _check(lib().prb_bias_act(_p(out), _p(inp), _p(bias), _p(resid), m, n, ACT_CODES[act],
                              dtype_code(inp.dtype), dtype_code(out.dtype), _stream()), what)


def kv_append(k_pages, v_pages, k_src, v_src, slots, n_tokens, status) -> None:
    """Write the step's keys and values to their cache slots.  k_pages/v_pages:
    [pages, kv_heads, page_size, head_dim]; k_src/v_src: [T, kv_heads*head_dim] views that
    may be column slices of one wider row-major tensor."""
    what = "kv_append"
    num_pages, kv_heads, page_size, head_dim = k_pages.shape
    _need(k_pages, None, "k_pages", what)
    _need(v_pages, k_pages.dtype, "v_pages", what)
    _need(slots, torch.int32, "slots", what)
    for name, s in (("k_src", k_src), ("v_src", v_src)):
        if s.dtype != k_pages.dtype or s.stride(1) != 1 or s.shape[1] != kv_heads * head_dim:
            raise KernelArgumentError(f"{what}: {name} has the wrong type, width or inner stride")
    if k_src.stride(0) != v_src.stride(0):
        raise KernelArgumentError(f"{what}: k_src and v_src row strides differ")
    _check(lib().prb_kv_append(_p(k_pages), _p(v_pages), _p(k_src), _p(v_src), k_src.stride(0),
                               _p(slots), n_tokens, kv_heads, head_dim, page_size, num_pages,
                               dtype_code(k_pages.dtype), _p(status), _stream()), what)


def copy_pages(storage, pairs, n_pairs, status) -> None:
    """storage: [pools, pages, ...] contiguous; pairs int32 [n, 2] (source, destination)."""
    what = "copy_pages"
    _need(storage, None, "storage", what)
    _need(pairs, torch.int32, "pairs", what)
    pools, pages = storage.shape[0], storage.shape[1]
    page_bytes = storage[0, 0].numel() * storage.element_size()
    _check(lib().prb_copy_pages(_p(storage), _p(pairs), n_pairs, page_bytes, pools, pages,
                                _p(status), _stream()), what)


def gemm_f32(out, a, w, bias=None, resid=None, act=None) -> None:
    """out[M,N] = act(a[M,K] . w[N,K]^T + bias) (+ resid): true 32-bit FMA."""
    what = "gemm_f32"
    for name, t in (("out", out), ("a", a), ("w", w)):
        if not t.is_cuda or t.dtype != torch.float32 or t.stride(1) != 1:
            raise KernelArgumentError(f"{what}: {name} must be float32 on CUDA with unit inner stride")
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape[0] != m or out.shape[1] != n:
        raise KernelArgumentError(f"{what}: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    if bias is not None:
        _need(bias, torch.float32, "bias", what)
    if resid is not None:
        _need(resid, torch.float32, "resid", what)
        if resid.shape != out.shape or resid.stride(0) != out.stride(0):
            raise KernelArgumentError(f"{what}: resid must have the output's shape and stride")
    _check(lib().prb_gemm_f32(_p(out), _p(a), _p(w), _p(bias), _p(resid), m, n, k, a.stride(0),
                              w.stride(0), out.stride(0), ACT_CODES[act], _stream()), what)


def gemm_bf16(out, a, w, bias=None, resid=None, act=None, tile_n: int = 0, status=None,
              kv_scatter=None, split_k: int = 0, pair: bool = False) -> None:
    """out[M,N] = act(a[M,K] . w[N,K]^T + bias) (+ resid) on the tcgen05 tensor cores:
    bfloat16 operands, float32 accumulation in tensor memory, epilogue in float32; out is
    bfloat16 or float32.  K and the row pitches of a and w must be multiples of 8.
    ``kv_scatter`` = (k_pages, v_pages, slots, q_width[, only_cache]): the key and value
    columns of a fused QKV product also go to the paged cache (of the output's element type);
    with ``only_cache`` they need not reach ``out`` at all.  ``tile_n`` and
    ``split_k`` force a tile width and, for widths 64 and 128, a cluster of 2, 4 or 8 CTAs
    that share a tile's reduction; ``pair`` (widths 64, 128, 192, 256) forces pairs of CTAs on
    256-row tiles (``tcgen05.mma.cta_group::2``); left at 0 the kernel chooses."""
    what = "gemm_bf16"
    for name, t in (("a", a), ("w", w)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.stride(1) != 1:
            raise KernelArgumentError(f"{what}: {name} must be bfloat16 on CUDA with unit inner stride")
    if not out.is_cuda or out.stride(1) != 1:
        raise KernelArgumentError(f"{what}: out must be on CUDA with unit inner stride")
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape[0] != m or out.shape[1] != n:
        raise KernelArgumentError(f"{what}: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    if bias is not None:
        _need(bias, torch.float32, "bias", what)
    if resid is not None:
        _need(resid, torch.float32, "resid", what)
        if resid.shape != out.shape or resid.stride(0) != out.stride(0):
            raise KernelArgumentError(f"{what}: resid must have the output's shape and stride")
    if kv_scatter is not None:
        k_pages, v_pages, slots, q_width = kv_scatter[:4]
        only_cache = bool(kv_scatter[4]) if len(kv_scatter) > 4 else False
        if resid is not None or tile_n or split_k or pair:
            raise KernelArgumentError(f"{what}: a product that scatters takes no residual or tile width")
        if k_pages.dtype != out.dtype or v_pages.dtype != out.dtype or not k_pages.is_contiguous() \
                or not v_pages.is_contiguous():
            raise KernelArgumentError(f"{what}: the cache must be contiguous and of the output's type")
        _need(slots, torch.int32, "slots", what)
        num_pages, kv_heads, page_size, head_dim = k_pages.shape
        _check(lib().prb_gemm_bf16_scatter(
            _p(out), _p(a), _p(w), _p(bias), m, n, k, a.stride(0), w.stride(0), out.stride(0),
            ACT_CODES[act], dtype_code(out.dtype), _p(k_pages), _p(v_pages), _p(slots), int(q_width),
            kv_heads * head_dim, head_dim, page_size, num_pages, int(only_cache), _p(status),
            _stream()), what)
        return
    _check(lib().prb_gemm_bf16(_p(out), _p(a), _p(w), _p(bias), _p(resid), m, n, k, a.stride(0),
                               w.stride(0), out.stride(0), ACT_CODES[act], dtype_code(out.dtype),
                               int(tile_n) | (int(split_k) << 16) | (int(bool(pair)) << 24),
                               _p(status), _stream()), what)


def midm_supports(m: int, n: int, k: int) -> bool:
    return bool(lib().prb_gemm_midm_supports(int(m), int(n), int(k)))


def gemm_midm(out, a, w, bias=None, resid=None, act=None, status=None) -> None:
    """out[M,N] = act(a[M,K] . w[N,K]^T + bias) (+ resid) for up to 64 rows, K a multiple of
    64: the reduction is split over a thread-block cluster (``csrc/gemm_bf16_midm.cu``)."""
    what = "gemm_midm"
    for name, t in (("a", a), ("w", w)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.stride(1) != 1:
            raise KernelArgumentError(f"{what}: {name} must be bfloat16 on CUDA with unit inner stride")
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape[0] != m or out.shape[1] != n or out.stride(1) != 1:
        raise KernelArgumentError(f"{what}: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    if bias is not None:
        _need(bias, torch.float32, "bias", what)
    if resid is not None:
        _need(resid, torch.float32, "resid", what)
        if resid.shape != out.shape or resid.stride(0) != out.stride(0):
            raise KernelArgumentError(f"{what}: resid must have the output's shape and stride")
    _check(lib().prb_gemm_midm(_p(out), _p(a), _p(w), _p(bias), _p(resid), m, n, k, a.stride(0),
                               w.stride(0), out.stride(0), ACT_CODES[act], dtype_code(out.dtype),
                               _p(status), _stream()), what)


_SMALLM = None


def smallm_limits():
    """(most rows, widest fused norm) of the decode-time product kernel."""
    global _SMALLM
    if _SMALLM is None:
        _SMALLM = (lib().prb_gemm_smallm_max_rows(), lib().prb_gemm_smallm_max_norm_width())
    return _SMALLM


def gemm_smallm(out, w, a=None, norm_input=None, gamma=None, beta=None, eps=0.0, bias=None,
                resid=None, act=None, kv_scatter=None, status=None, norm_rows=None) -> None:
    """out[M,N] = act(X . w[N,K]^T + bias) (+ resid) for M <= 64 rows, weights streamed once.
    X is ``a`` (bfloat16 [M,K]) or LayerNorm(``norm_input``) (float32 [M,K]) with ``gamma``,
    ``beta`` and ``eps``, the norm fused into the kernel; with ``norm_rows`` (int32 [M]) row t
    of X is the norm of row norm_rows[t] of ``norm_input`` (an index outside it gives a zero
    row and is recorded in ``status``).  ``kv_scatter`` = (k_pages, v_pages,
    slots, q_width): the product is a fused QKV projection; its key and value columns are also
    written to the paged cache (same element type as ``out``) at each token's slot."""
    what = "gemm_smallm"
    if not w.is_cuda or w.dtype != torch.bfloat16 or w.stride(1) != 1:
        raise KernelArgumentError(f"{what}: w must be bfloat16 on CUDA with unit inner stride")
    n, k = w.shape
    if norm_input is not None:
        x = norm_input
        if x.dtype != torch.float32 or x.stride(1) != 1:
            raise KernelArgumentError(f"{what}: norm_input must be float32 with unit inner stride")
        _need(gamma, torch.float32, "gamma", what)
        if beta is not None:
            _need(beta, torch.float32, "beta", what)
    else:
        x = a
        if x is None or x.dtype != torch.bfloat16 or x.stride(1) != 1:
            raise KernelArgumentError(f"{what}: a must be bfloat16 with unit inner stride")
    m = out.shape[0]
    if norm_rows is not None:
        if norm_input is None:
            raise KernelArgumentError(f"{what}: norm_rows gathers rows of norm_input")
        _need(norm_rows, torch.int32, "norm_rows", what)
        if norm_rows.numel() < m:
            raise KernelArgumentError(f"{what}: {m} output rows, {norm_rows.numel()} row indices")
    if (norm_rows is None and x.shape[0] < m) or x.shape[1] != k or out.shape[1] != n or \
            out.stride(1) != 1:
        raise KernelArgumentError(f"{what}: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    if bias is not None:
        _need(bias, torch.float32, "bias", what)
    if resid is not None:
        if resid.dtype != torch.float32 or resid.shape != out.shape or resid.stride(0) != out.stride(0):
            raise KernelArgumentError(f"{what}: resid must be float32 with the output's shape and stride")
    kv = (None, None, None, 0, 0, 0, 0, 0)
    if kv_scatter is not None:
        k_pages, v_pages, slots, q_width = kv_scatter[:4]
        num_pages, kv_heads, page_size, head_dim = k_pages.shape
        if k_pages.dtype != out.dtype or v_pages.dtype != out.dtype or slots.dtype != torch.int32 \
                or q_width + 2 * kv_heads * head_dim != n:
            raise KernelArgumentError(f"{what}: cache type or widths do not fit the product")
        kv = (_p(k_pages), _p(v_pages), _p(slots), q_width, kv_heads * head_dim, head_dim,
              page_size, num_pages)
    _check(lib().prb_gemm_smallm(
        _p(out), None if norm_input is not None else _p(x),
        _p(x) if norm_input is not None else None, _p(norm_rows),
        x.shape[0] if norm_input is not None else 0, _p(gamma), _p(beta), float(eps), _p(w),
        _p(bias), _p(resid), m, n, k, x.stride(0), w.stride(0), out.stride(0), ACT_CODES[act],
        dtype_code(out.dtype), *kv, _p(status), _stream()), what)


def attention_generic(out, q, k_pages, v_pages, block_table, seq_of_token, positions, n_tokens,
                      n_heads, scale, window, max_context, status) -> None:
    """Attention of every token of the step over its request's cached keys; 32-bit
    arithmetic.  q: [T, n_heads*head_dim] (may be a column slice), out likewise."""
    what = "attention_generic"
    num_pages, kv_heads, page_size, head_dim = k_pages.shape
    for name, t in (("out", out), ("q", q)):
        if t.dtype != k_pages.dtype or t.stride(1) != 1 or t.shape[1] != n_heads * head_dim:
            raise KernelArgumentError(f"{what}: {name} has the wrong type, width or inner stride")
    _need(block_table, torch.int32, "block_table", what)
    _need(seq_of_token, torch.int32, "seq_of_token", what)
    _need(positions, torch.int32, "positions", what)
    _check(lib().prb_attention_generic(
        _p(out), out.stride(0), _p(q), q.stride(0), _p(k_pages), _p(v_pages), _p(block_table),
        _p(seq_of_token), _p(positions), n_tokens, n_heads, kv_heads, head_dim, page_size,
        block_table.shape[1], num_pages, max_context, float(scale), int(window or 0),
        dtype_code(k_pages.dtype), _p(status), _stream()), what)


_SM_COUNT = None


def sm_count() -> int:
    """Streaming multiprocessors of the current device."""
    global _SM_COUNT
    if _SM_COUNT is None:
        _SM_COUNT = max(1, int(lib().prb_device_sm_count()))
    return _SM_COUNT


def decode_max_split_pages() -> int:
    """Most pages one split of the decode attention kernel may span."""
    return lib().prb_attention_decode_max_split_pages()


def decode_split() -> int:
    """Keys per split of the decode attention kernel."""
    return lib().prb_attention_decode_split()


def decode_stream(mode: int) -> None:
    """Which key loop the decode attention kernel runs (for tests and measurements): -1 the
    kernel's own choice, 0 register batches always, 1 the shared-memory ring wherever it
    applies (no window, head size up to 128)."""
    lib().prb_attention_decode_set_stream(int(mode))


def prefill_supports(head_dim: int) -> bool:
    return bool(lib().prb_attention_prefill_supports(int(head_dim)))


def attention_decode(out, q, k_pages, v_pages, block_table, seq_of_token, positions, token_list,
                     token_count, n_list, n_heads, scale, window, workspace, counters, max_splits,
                     status, split_keys: Optional[int] = None) -> None:
    """bfloat16 attention of single tokens (those in ``token_list``, or all of the first
    ``n_list`` when it is None) over their requests' pages, keys split in ranges of
    ``split_keys`` positions (a multiple of ``decode_split()``, the default).  ``workspace`` float32 [n_list, heads, max_splits,
    head_dim + 4] and ``counters`` int32 [n_list * heads] (zero) are scratch."""
    what = "attention_decode"
    num_pages, kv_heads, page_size, head_dim = k_pages.shape
    for name, t in (("out", out), ("q", q)):
        if t.dtype != torch.bfloat16 or t.stride(1) != 1 or t.shape[1] != n_heads * head_dim:
            raise KernelArgumentError(f"{what}: {name} has the wrong type, width or inner stride")
    if k_pages.dtype != torch.bfloat16:
        raise KernelArgumentError(f"{what}: the cache must be bfloat16")
    split_keys = decode_split() if split_keys is None else int(split_keys)
    need = n_list * n_heads * max_splits * (head_dim + 4)
    if workspace.dtype != torch.float32 or workspace.numel() < need or \
            counters.dtype != torch.int32 or counters.numel() < n_list * n_heads:
        raise KernelArgumentError(f"{what}: scratch too small or of the wrong type")
    _check(lib().prb_attention_decode(
        _p(out), out.stride(0), _p(q), q.stride(0), _p(k_pages), _p(v_pages), _p(block_table),
        _p(seq_of_token), _p(positions), _p(token_list), _p(token_count), n_list, n_heads,
        kv_heads, head_dim, page_size, block_table.shape[1], num_pages, float(scale),
        int(window or 0), _p(workspace), _p(counters), max_splits, split_keys, _p(status),
        _stream()), what)


def decode_ring_supports(head_dim: int, page_size: int) -> bool:
    return bool(lib().prb_attention_decode_ring_supports(int(head_dim), int(page_size)))


def decode_ring_prefers(n_list: int, n_heads: int, max_context: int) -> bool:
    """Whether ``attention_decode_ring`` is the faster kernel for this launch (both are right)."""
    return bool(lib().prb_attention_decode_ring_prefers(int(n_list), int(n_heads), int(max_context)))


def decode_ring_max_list() -> int:
    """Most single tokens a launch of ``attention_decode_ring`` takes."""
    return int(lib().prb_attention_decode_ring_max_list())


def decode_ring_workspace(n_list: int, n_heads: int, head_dim: int) -> int:
    """float32 elements of workspace ``attention_decode_ring`` needs for up to ``n_list`` tokens."""
    return int(lib().prb_attention_decode_ring_workspace(int(n_list), int(n_heads), int(head_dim)))


def attention_decode_ring(out, q, k_pages, v_pages, block_table, seq_of_token, positions,
                          token_list, token_count, n_list, n_heads, scale, window, workspace,
                          counters, status, new_keys: int = 1, stages: int = 0,
                          max_context: int = 0, kv_new=None) -> None:
    """bfloat16 attention of single tokens over their requests' pages by persistent CTAs whose
    warps stream keys and values through rings of shared-memory buffers; what was cached before
    the step is requested before the kernel this one depends on has finished (head size 64).
    ``new_keys``: how many of a token's last visible positions the step itself may have
    written (at most 4).  ``kv_new`` = (k, v): the step's own keys and values, row t for token t
    ([T, kv_heads * head_dim], may be column slices of a wider tensor), as the product before
    this kernel left them; with them no part of the kernel waits for the cache rows the step
    appended.  ``workspace``: ``decode_ring_workspace`` floats; ``counters`` int32
    [n_list * heads], zero (left zero)."""
    what = "attention_decode_ring"
    num_pages, kv_heads, page_size, head_dim = k_pages.shape
    for name, t in (("out", out), ("q", q)):
        if t.dtype != torch.bfloat16 or t.stride(1) != 1 or t.shape[1] != n_heads * head_dim:
            raise KernelArgumentError(f"{what}: {name} has the wrong type, width or inner stride")
    if k_pages.dtype != torch.bfloat16 or not k_pages.is_contiguous() or not v_pages.is_contiguous():
        raise KernelArgumentError(f"{what}: the cache must be contiguous bfloat16")
    if workspace.dtype != torch.float32 or \
            workspace.numel() < decode_ring_workspace(n_list, n_heads, head_dim) or \
            counters.dtype != torch.int32 or counters.numel() < n_list * n_heads:
        raise KernelArgumentError(f"{what}: scratch too small or of the wrong type")
    k_new = v_new = None
    kv_stride = 0
    if kv_new is not None:
        k_new, v_new = kv_new
        for name, t in (("k_new", k_new), ("v_new", v_new)):
            if t.dtype != torch.bfloat16 or t.stride(1) != 1 or t.shape[1] != kv_heads * head_dim:
                raise KernelArgumentError(f"{what}: {name} has the wrong type, width or inner stride")
        if k_new.stride(0) != v_new.stride(0):
            raise KernelArgumentError(f"{what}: k_new and v_new row strides differ")
        kv_stride = k_new.stride(0)
    _check(lib().prb_attention_decode_ring(
        _p(out), out.stride(0), _p(q), q.stride(0), _p(k_pages), _p(v_pages), _p(block_table),
        _p(seq_of_token), _p(positions), _p(token_list), _p(token_count), n_list, n_heads,
        kv_heads, head_dim, page_size, block_table.shape[1], num_pages, float(scale),
        int(window or 0), int(new_keys), _p(k_new), _p(v_new), int(kv_stride), _p(workspace),
        _p(counters), int(stages), int(max_context), _p(status), _stream()), what)


def prefill_tile() -> int:
    """Rows per item of the work list the prompt attention kernels take."""
    return lib().prb_attention_prefill_tile()


def prefill_tc_supports(head_dim: int, page_size: int) -> bool:
    return bool(lib().prb_attention_prefill_tc_supports(int(head_dim), int(page_size)))


PREFILL_MAX_PARTS = 16


def attention_prefill_tc(out, q, k_pages, v_pages, block_table, positions, tile_req, tile_row0,
                         tile_rows, tile_count, n_tiles, n_heads, scale, window, status,
                         part_blocks: int = 0, max_parts: int = 1, parts=None, items=None) -> None:
    """bfloat16 causal attention of prompt portions on tcgen05 (head size 64, pages of a
    multiple of 64 positions): one CTA per work item of up to 128 queries and head, or, with
    ``part_blocks`` > 0, one per chunk of ``part_blocks`` * 64 keys of the item (at most
    ``max_parts`` chunks; ``parts`` = (float32 [n_tiles * n_heads * max_parts * 8192],
    float32 [n_tiles * n_heads * max_parts * 256], zeroed int32 [n_tiles * n_heads]) is the
    workspace through which the chunks of an item are merged).

    ``items`` = (item_tile, item_part, item_slot, item_count or None, part_blocks (device
    int32 [1]), n_items, n_slots): the CTAs' work as a list instead (item i is tile
    ``item_tile[i]`` as a whole when ``item_part[i]`` < 0, else that chunk of it, whose
    partial result goes to workspace slot ``item_slot[i]``; a tile's chunks have consecutive
    slots); ``parts`` then holds ``n_slots * n_heads`` slots and counters."""
    what = "attention_prefill_tc"
    num_pages, kv_heads, page_size, head_dim = k_pages.shape
    for name, t in (("out", out), ("q", q)):
        if t.dtype != torch.bfloat16 or t.stride(1) != 1 or t.shape[1] != n_heads * head_dim:
            raise KernelArgumentError(f"{what}: {name} has the wrong type, width or inner stride")
    if k_pages.dtype != torch.bfloat16 or not k_pages.is_contiguous() or not v_pages.is_contiguous():
        raise KernelArgumentError(f"{what}: the cache must be contiguous bfloat16")
    part_o = part_ml = part_count = None
    item_tile = item_part = item_slot = item_count = part_dev = None
    n_items = 0
    if items is not None:
        item_tile, item_part, item_slot, item_count, part_dev, n_items, n_slots = items
        if part_blocks or parts is None:
            raise KernelArgumentError(f"{what}: a work list brings its own chunk size and needs a workspace")
        for name, t in (("item_tile", item_tile), ("item_part", item_part), ("item_slot", item_slot),
                        ("part_blocks", part_dev)):
            _need(t, torch.int32, name, what)
        if min(item_tile.numel(), item_part.numel(), item_slot.numel()) < n_items:
            raise KernelArgumentError(f"{what}: the work list is shorter than {n_items} items")
        part_o, part_ml, part_count = parts
        _need(part_o, torch.float32, "parts[0]", what)
        _need(part_ml, torch.float32, "parts[1]", what)
        _need(part_count, torch.int32, "parts[2]", what)
        units = int(n_slots) * n_heads
        if part_o.numel() < units * 8192 or part_ml.numel() < units * 256 or part_count.numel() < units:
            raise KernelArgumentError(f"{what}: the workspace of the key parts is too small")
    if part_blocks:
        if parts is None or not 1 <= max_parts <= PREFILL_MAX_PARTS:
            raise KernelArgumentError(f"{what}: key parts need a workspace and 1 to "
                                      f"{PREFILL_MAX_PARTS} parts per item")
        part_o, part_ml, part_count = parts
        units = n_tiles * n_heads
        _need(part_o, torch.float32, "parts[0]", what)
        _need(part_ml, torch.float32, "parts[1]", what)
        _need(part_count, torch.int32, "parts[2]", what)
        if part_o.numel() < units * max_parts * 8192 or part_ml.numel() < units * max_parts * 256 \
                or part_count.numel() < units:
            raise KernelArgumentError(f"{what}: the workspace of the key parts is too small")
    _check(lib().prb_attention_prefill_tc(
        _p(out), out.stride(0), _p(q), q.stride(0), q.shape[0], _p(k_pages), _p(v_pages),
        _p(block_table), _p(positions), _p(tile_req), _p(tile_row0), _p(tile_rows), _p(tile_count),
        n_tiles, n_heads, kv_heads, head_dim, page_size, block_table.shape[1], num_pages,
        float(scale), int(window or 0), int(part_blocks), int(max_parts), _p(part_o), _p(part_ml),
        _p(part_count), _p(item_tile), _p(item_part), _p(item_slot), _p(item_count), _p(part_dev),
        int(n_items), _p(status), _stream()), what)


def attention_prefill(out, q, k_pages, v_pages, block_table, positions, tile_req, tile_row0,
                      tile_rows, tile_count, n_tiles, n_heads, scale, window, status) -> None:
    """bfloat16 causal attention of prompt portions (work items of up to 128 queries, two
    CTAs of 64 each) on mma.sync tensor-core instructions; any head size in steps of 16."""
    what = "attention_prefill"
    num_pages, kv_heads, page_size, head_dim = k_pages.shape
    for name, t in (("out", out), ("q", q)):
        if t.dtype != torch.bfloat16 or t.stride(1) != 1 or t.shape[1] != n_heads * head_dim:
            raise KernelArgumentError(f"{what}: {name} has the wrong type, width or inner stride")
    if k_pages.dtype != torch.bfloat16:
        raise KernelArgumentError(f"{what}: the cache must be bfloat16")
    _check(lib().prb_attention_prefill(
        _p(out), out.stride(0), _p(q), q.stride(0), _p(k_pages), _p(v_pages), _p(block_table),
        _p(positions), _p(tile_req), _p(tile_row0), _p(tile_rows), _p(tile_count), n_tiles,
        n_heads, kv_heads, head_dim, page_size, block_table.shape[1], num_pages, float(scale),
        int(window or 0), _p(status), _stream()), what)


def resolve_tokens(tokens, n, prev, status) -> None:
    """tokens[t] = prev[-tokens[t] - 1] wherever tokens[t] < 0 (t < n): ids that name a place
    among the tokens the sampling kernel chose last."""
    what = "resolve_tokens"
    _need(tokens, torch.int32, "tokens", what)
    _need(prev, torch.int32, "prev", what)
    _check(lib().prb_resolve_tokens(_p(tokens), int(n), _p(prev), prev.numel(), _p(status),
                                    _stream()), what)


def host_device_address(host: torch.Tensor) -> int:
    """The address under which kernels reach this pinned host tensor, or 0 if they cannot
    (the caller then copies with the copy engine)."""
    if host.is_cuda or not host.is_pinned():
        return 0
    return int(lib().prb_host_device_address(host.data_ptr()) or 0)


def fetch_step(dev, host_address: int, words: int, tokens_at: int = 0, n_tokens: int = 0,
               prev=None, status=None) -> None:
    """dev[:words] = the int32 words at ``host_address`` (from :func:`host_device_address`),
    read by a kernel; with ``prev``, token ids below zero among words
    [tokens_at, tokens_at + n_tokens) become prev[-id - 1] on the way."""
    what = "fetch_step"
    _need(dev, torch.int32, "dev", what)
    if not host_address or words > dev.numel():
        raise KernelArgumentError(f"{what}: no host address, or {words} words do not fit")
    if prev is not None:
        _need(prev, torch.int32, "prev", what)
    _check(lib().prb_fetch_step(_p(dev), host_address, int(words), int(tokens_at), int(n_tokens),
                                _p(prev), 0 if prev is None else prev.numel(), _p(status),
                                _stream()), what)


def publish_result(host_address: int, dev, words: int) -> None:
    """The int32 words dev[:words] written to pinned host memory at ``host_address`` by a
    kernel; the host sees them once an event recorded after this call has completed."""
    what = "publish_result"
    _need(dev, torch.int32, "dev", what)
    if not host_address or words > dev.numel():
        raise KernelArgumentError(f"{what}: no host address, or {words} words do not fit")
    _check(lib().prb_publish_result(host_address, _p(dev), int(words), _stream()), what)


def max_top_k() -> int:
    return lib().prb_sample_max_top_k()


def sample_workspace_words() -> int:
    return lib().prb_sample_workspace_words()


def sample(out, logits, n_rows, temperature=None, top_k=None, top_p=None, seeds=None, fresh=None,
           slots=None, rng_states=None, publish=None, workspace=None) -> None:
    """out[r] = chosen token of logits[r,:] (float32).  Without ``temperature`` every row
    is greedy; otherwise rows with temperature <= 0 are greedy and the rest sample.
    ``workspace``: :func:`sample_workspace_words` int32 words on the device, zero at first and
    then left to the kernels (one per stream of calls); with it a launch of up to 64 greedy
    rows gives every row to several CTAs.  ``publish`` = (host_address, src, words), with a
    workspace: the launch's last CTA also writes the int32 words src[:words] to pinned host
    memory at ``host_address`` (from :func:`host_device_address`)."""
    what = "sample"
    if workspace is not None:
        _need(workspace, torch.int32, "workspace", what)
        if workspace.numel() < sample_workspace_words() or not workspace.is_contiguous():
            raise KernelArgumentError(f"{what}: the workspace needs {sample_workspace_words()} "
                                      f"contiguous int32 words")
    pub = (None, None, 0)
    if publish is not None:
        address, src, words = publish
        _need(src, torch.int32, "publish source", what)
        if workspace is None or not address or words > src.numel():
            raise KernelArgumentError(f"{what}: publishing needs a workspace and a host address, "
                                      f"and {words} words the source holds")
        pub = (int(address), _p(src), int(words))
    _need(out, torch.int32, "out", what)
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelArgumentError(f"{what}: logits must be float32 with unit inner stride")
    if temperature is not None:
        _need(temperature, torch.float32, "temperature", what)
        _need(top_k, torch.int32, "top_k", what)
        _need(top_p, torch.float32, "top_p", what)
        _need(seeds, torch.int64, "seeds", what)
        _need(fresh, torch.int32, "fresh", what)
        _need(slots, torch.int32, "slots", what)
        _need(rng_states, torch.int64, "rng_states", what)
    _check(lib().prb_sample(_p(out), _p(logits), logits.stride(0), logits.shape[1],
                            _p(temperature), _p(top_k), _p(top_p), _p(seeds), _p(fresh), _p(slots),
                            _p(rng_states), n_rows, *pub, _p(workspace), _stream()), what)

