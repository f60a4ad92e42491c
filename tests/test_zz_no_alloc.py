"""The decode attention entry point for callers that may not allocate device memory.

Some users of the library (a host program whose allocator owns the GPU, a plugin with a
fixed budget) cannot hand it scratch buffers.  ``prb_attention_decode_noalloc`` keeps the
kernel's scratch in fixed arrays inside the library.  It is called here through its
exported C symbol, twice in a row on different inputs (the arrays are shared between calls
and keep the previous call's contents), and compared with the ordinary entry point, which
gets its scratch from the caller.  This file is collected last on purpose."""
import ctypes
from ctypes import c_float, c_int, c_long, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, lengths, n_heads, dh, ps):
    g = torch.Generator(device="cpu").manual_seed(seed)
    pages_needed = sum(-(-n // ps) for n in lengths) + 3
    k = torch.randn(pages_needed, n_heads, ps, dh, generator=g).to(torch.bfloat16).cuda()
    v = torch.randn(pages_needed, n_heads, ps, dh, generator=g).to(torch.bfloat16).cuda()
    perm = torch.randperm(pages_needed, generator=g).tolist()
    max_pages = max(-(-n // ps) for n in lengths) + 1
    table = torch.full((len(lengths), max_pages), -1, dtype=torch.int32)
    for b, n in enumerate(lengths):
        for i in range(-(-n // ps)):
            table[b, i] = perm.pop()
    seq = torch.arange(len(lengths), dtype=torch.int32).cuda()
    pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32).cuda()
    q = torch.randn(len(lengths), n_heads * dh, generator=g).to(torch.bfloat16).cuda()
    return q, k, v, table.cuda(), seq, pos


def test_no_alloc_entry_point_matches_the_ordinary_one():
    from pretrained_rstr_b200.csrc import ops
    lib = ops.lib()
    fn = lib.prb_attention_decode_noalloc
    P, I, L, F = c_void_p, c_int, c_long, c_float
    fn.argtypes = [P, L, P, L, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, I, I, P, P]
    fn.restype = c_int
    lib.prb_attention_decode_noalloc_limits.argtypes = [ctypes.POINTER(c_long), ctypes.POINTER(c_int)]
    lib.prb_attention_decode_noalloc_limits.restype = None
    ws_max, cnt_max = c_long(0), c_int(0)
    lib.prb_attention_decode_noalloc_limits(ctypes.byref(ws_max), ctypes.byref(cnt_max))
    assert ws_max.value == 1 << 20 and cnt_max.value == 1 << 14

    n_heads, dh, ps = 6, 64, 64
    splits = -(-1024 // ops.decode_split())
    stream = torch.cuda.current_stream().cuda_stream
    for seed, lengths in ((1, [1000, 3, 257, 640, 129]), (2, [64, 900, 511])):   # two calls in a row
        q, k, v, table, seq, pos = _case(seed, lengths, n_heads, dh, ps)
        t = q.shape[0]
        status = torch.zeros(4, dtype=torch.int32, device="cuda")
        want = torch.zeros_like(q)
        ws = torch.zeros(t * n_heads * splits * (dh + 4), device="cuda")
        counters = torch.zeros(t * n_heads, dtype=torch.int32, device="cuda")
        ops.attention_decode(want, q, k, v, table, seq, pos, None, None, t, n_heads, 0.125, None,
                             ws, counters, splits, status)
        got = torch.full_like(q, float("nan"))
        rc = fn(got.data_ptr(), got.stride(0), q.data_ptr(), q.stride(0), k.data_ptr(),
                v.data_ptr(), table.data_ptr(), seq.data_ptr(), pos.data_ptr(), None, None, t,
                n_heads, n_heads, dh, ps, table.shape[1], k.shape[0], 0.125, 0, splits,
                ops.decode_split(), status.data_ptr(), stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert status.tolist() == [0, 0, 0, 0]
        assert float((got.float() - want.float()).abs().max()) <= 2e-2
    # a launch that needs more scratch than the fixed arrays hold is refused, nothing runs
    rc = fn(got.data_ptr(), got.stride(0), q.data_ptr(), q.stride(0), k.data_ptr(), v.data_ptr(),
            table.data_ptr(), seq.data_ptr(), pos.data_ptr(), None, None, 4096, n_heads, n_heads,
            dh, ps, table.shape[1], k.shape[0], 0.125, 0, splits, ops.decode_split(),
            status.data_ptr(), stream)
    assert rc == -3
