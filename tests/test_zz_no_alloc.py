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


def _ref(q, k, v, table, pos, n_heads, scale):
    """float32 attention of every query over its request's pages, straight from the formula."""
    t = q.shape[0]
    _pages, _kv_heads, ps, dh = k.shape
    out = torch.zeros(t, n_heads * dh, device="cuda")
    kf, vf, qf = k.float(), v.float(), q.float()
    for i in range(t):
        js = torch.arange(0, int(pos[i]) + 1, device="cuda")
        pages = table[i, (js // ps).long()].long()
        for h in range(n_heads):
            kk, vv = kf[pages, h, (js % ps).long()], vf[pages, h, (js % ps).long()]
            out[i, h * dh:(h + 1) * dh] = torch.softmax((kk @ qf[i, h * dh:(h + 1) * dh]) * scale, 0) @ vv
    return out


def test_no_alloc_entry_point_matches_the_ordinary_one():
    """Contexts of up to 2,048 keys in splits of 128: up to 16 splits per (token, head), more
    than a thread-block cluster takes, so the partial results really go through the scratch
    arrays and the counters decide who merges.  The second call is smaller and differently
    shaped, so contents the first call left in the arrays would show.  Both calls must equal
    the ordinary entry point bit for bit (same kernel, same splits, same order of sums), agree
    with a float32 reference, and take no device memory."""
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

    dh, ps = 64, 64
    split = ops.decode_split()
    stream = torch.cuda.current_stream().cuda_stream
    cases = ((1, 6, [2048, 3, 1500, 640, 129, 1025]), (2, 3, [64, 1100, 511]))
    for seed, n_heads, lengths in cases:                       # two calls in a row
        q, k, v, table, seq, pos = _case(seed, lengths, n_heads, dh, ps)
        t = q.shape[0]
        splits = -(-max(lengths) // split)
        assert splits > 8                                      # beyond a cluster: the workspace path
        assert t * n_heads * splits * (dh + 4) <= ws_max.value
        status = torch.zeros(4, dtype=torch.int32, device="cuda")
        want = torch.zeros_like(q)
        ws = torch.full((t * n_heads * splits * (dh + 4),), float("nan"), device="cuda")
        counters = torch.zeros(t * n_heads, dtype=torch.int32, device="cuda")
        ops.attention_decode(want, q, k, v, table, seq, pos, None, None, t, n_heads, 0.125, None,
                             ws, counters, splits, status)
        assert int(counters.abs().sum()) == 0                  # the kernel leaves its counters at zero
        assert bool(torch.isfinite(ws).any())                  # and did write partial results
        got = torch.full_like(q, float("nan"))
        took = []
        for _attempt in range(3):          # (the figure is the device's: another process may move it)
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
            rc = fn(got.data_ptr(), got.stride(0), q.data_ptr(), q.stride(0), k.data_ptr(),
                    v.data_ptr(), table.data_ptr(), seq.data_ptr(), pos.data_ptr(), None, None, t,
                    n_heads, n_heads, dh, ps, table.shape[1], k.shape[0], 0.125, 0, splits,
                    split, status.data_ptr(), stream)
            assert rc == 0
            torch.cuda.synchronize()
            took.append(free_before - torch.cuda.mem_get_info()[0])
            if took[-1] == 0:
                break
        assert took[-1] == 0, f"the call took device memory: free bytes fell by {took}"
        assert status.tolist() == [0, 0, 0, 0]
        assert torch.equal(got, want)
        assert float((got.float() - _ref(q, k, v, table, pos, n_heads, 0.125)).abs().max()) <= 2e-2
    # a launch that needs more scratch than the fixed arrays hold is refused, nothing runs
    rc = fn(got.data_ptr(), got.stride(0), q.data_ptr(), q.stride(0), k.data_ptr(), v.data_ptr(),
            table.data_ptr(), seq.data_ptr(), pos.data_ptr(), None, None, 4096, n_heads, n_heads,
            dh, ps, table.shape[1], k.shape[0], 0.125, 0, splits, split,
            status.data_ptr(), stream)
    assert rc == -3
