"""Each CUDA kernel alone against a plain float32 PyTorch statement of the same
operation, at sizes other than the engine's."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ops():
    from pretrained_rstr_b200.csrc import ops
    return ops


def _act(name, u):
    if name == "gelu_new":
        return torch.nn.functional.gelu(u, approximate="tanh")
    if name == "gelu":
        return torch.nn.functional.gelu(u)
    if name == "relu":
        return torch.relu(u)
    return u


GEMM_SHAPES = [(5, 192, 64), (130, 320, 96), (300, 96, 320), (1, 2304, 768), (64, 1000, 96),
               (257, 808, 1608), (2048, 768, 3072), (7, 50257, 768), (33, 3072, 768), (64, 768, 3072),
               (17, 6400, 1600)]


@pytest.mark.parametrize("m,n,k", GEMM_SHAPES)
@pytest.mark.parametrize("variant", ["plain_f32", "bias_gelu_bf16", "bias_resid_f32", "erf_bf16"])
def test_gemm_bf16_tcgen05(m, n, k, variant):
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(m * 7 + n * 3 + k)
    a = (torch.randn(m, k, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    bias = torch.randn(n, device="cuda", generator=g) * 0.2
    resid = torch.randn(m, n, device="cuda", generator=g)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ref = a.float() @ w.float().t()
    if variant == "plain_f32":
        out = torch.full((m, n), float("nan"), device="cuda")
        ops.gemm_bf16(out, a, w, status=status)
        tol = 2e-4
    elif variant == "bias_gelu_bf16":
        out = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
        ops.gemm_bf16(out, a, w, bias=bias, act="gelu_new", status=status)
        ref = _act("gelu_new", ref + bias)
        tol = 2e-2
    elif variant == "erf_bf16":
        out = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
        ops.gemm_bf16(out, a, w, bias=bias, act="gelu", status=status)
        ref = _act("gelu", ref + bias)
        tol = 2e-2
    else:
        out = resid.clone()                      # in place on the residual stream
        ops.gemm_bf16(out, a, w, bias=bias, resid=out, status=status)
        ref = ref + bias + resid
        tol = 2e-4
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    scale = float(ref.abs().max())
    err = float((out.float() - ref).abs().max())
    assert err <= tol * max(1.0, scale), f"max |difference| {err:.3e} (scale {scale:.3g})"


@pytest.mark.parametrize("tile_n", [32, 64, 96, 128, 160, 192, 224, 256])
def test_gemm_bf16_every_tile_width(tile_n):
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(tile_n)
    m, n, k = 200, 600, 136
    a = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    w = torch.randn(n, k, device="cuda", generator=g).to(torch.bfloat16)
    out = torch.zeros(m, n, device="cuda")
    ops.gemm_bf16(out, a, w, tile_n=tile_n)
    ref = a.float() @ w.float().t()
    assert float((out - ref).abs().max()) <= 1e-3


@pytest.mark.parametrize("tile_n", [64, 128, 192, 256])
@pytest.mark.parametrize("m,n,k", [(2048, 768, 768), (600, 1000, 1096), (130, 72, 136)])
def test_gemm_bf16_cta_pairs(tile_n, m, n, k):
    """Pairs of CTAs on 256-row tiles (one tcgen05.mma of the pair per 16 of K): both output
    types, with bias, activation and residual, at sizes that leave ragged tiles in every
    direction, an odd CTA with no rows at all, and more tiles than pairs of SMs."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(tile_n + m)
    a = (torch.randn(m, k, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    bias = torch.randn(n, device="cuda", generator=g)
    resid = torch.randn(m, n, device="cuda", generator=g)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ref = a.float() @ w.float().t() + bias
    out = resid.clone()
    ops.gemm_bf16(out, a, w, bias=bias, resid=out, tile_n=tile_n, pair=True, status=status)
    assert float((out - (ref + resid)).abs().max()) <= 2e-3 * max(1.0, float(ref.abs().max()))
    out16 = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
    ops.gemm_bf16(out16, a, w, bias=bias, act="gelu_new", tile_n=tile_n, pair=True, status=status)
    want = _act("gelu_new", ref)
    assert float((out16.float() - want).abs().max()) <= 1e-2 * max(1.0, float(want.abs().max()))
    assert status.tolist() == [0, 0, 0, 0]
    # one CTA per tile gives the same values: the same products summed in the same order
    single = resid.clone()
    ops.gemm_bf16(single, a, w, bias=bias, resid=single, tile_n=tile_n, status=status)
    assert torch.equal(single, out)
    with pytest.raises(ops.KernelArgumentError):
        ops.gemm_bf16(out, a, w, tile_n=96, pair=True)


@pytest.mark.parametrize("tile_n,split_k", [(64, 2), (64, 4), (64, 8), (128, 2), (128, 4), (128, 8),
                                            (192, 2), (256, 2)])
@pytest.mark.parametrize("m,n,k", [(256, 768, 3072), (200, 600, 1000), (130, 72, 520)])
def test_gemm_bf16_split_over_a_cluster(tile_n, split_k, m, n, k):
    """The reduction of a tile split over a thread-block cluster: both output types, with
    bias, activation and residual, at sizes that leave ragged tiles and a ragged last split."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(tile_n + split_k)
    a = (torch.randn(m, k, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    bias = torch.randn(n, device="cuda", generator=g)
    resid = torch.randn(m, n, device="cuda", generator=g)
    blocks = -(-k // 64)
    if -(-blocks // split_k) * (split_k - 1) >= blocks:
        with pytest.raises(ops.KernelArgumentError):
            ops.gemm_bf16(torch.zeros(m, n, device="cuda"), a, w, tile_n=tile_n, split_k=split_k)
        return
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ref = a.float() @ w.float().t() + bias
    out = resid.clone()
    ops.gemm_bf16(out, a, w, bias=bias, resid=out, tile_n=tile_n, split_k=split_k, status=status)
    assert float((out - (ref + resid)).abs().max()) <= 2e-3 * max(1.0, float(ref.abs().max()))
    out16 = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
    ops.gemm_bf16(out16, a, w, bias=bias, act="gelu_new", tile_n=tile_n, split_k=split_k, status=status)
    want = _act("gelu_new", ref)
    assert float((out16.float() - want).abs().max()) <= 1e-2 * max(1.0, float(want.abs().max()))
    assert status.tolist() == [0, 0, 0, 0]
    # the choice left to the kernel gives the same values up to the order of summation
    auto = resid.clone()
    ops.gemm_bf16(auto, a, w, bias=bias, resid=auto, status=status)
    assert float((auto - out).abs().max()) <= 1e-3 * max(1.0, float(ref.abs().max()))


def test_gemm_bf16_refuses_unaligned_k():
    ops = _ops()
    a = torch.zeros(4, 20, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(8, 20, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ops.KernelArgumentError, match="aligned"):
        ops.gemm_bf16(torch.zeros(4, 8, device="cuda"), a, w)


@pytest.mark.parametrize("m,n,k", [(3, 50, 20), (70, 130, 33), (129, 64, 64)])
def test_gemm_f32_is_true_32_bit(m, n, k):
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(1)
    a = torch.randn(m, k, device="cuda", generator=g)
    w = torch.randn(n, k, device="cuda", generator=g)
    bias = torch.randn(n, device="cuda", generator=g)
    out = torch.zeros(m, n, device="cuda")
    ops.gemm_f32(out, a, w, bias=bias, act="gelu")
    ref = _act("gelu", (a.double() @ w.double().t() + bias.double())).float()
    assert float((out - ref).abs().max()) <= 2e-5
    # a row's result does not depend on the rows beside it
    alone = torch.zeros(1, n, device="cuda")
    ops.gemm_f32(alone, a[m - 1:m].contiguous(), w, bias=bias, act="gelu")
    assert torch.equal(alone[0], out[m - 1])


# ------------------------------------------------------------------------ attention
def _paged_case(seed, n_heads, kv_heads, dh, page_size, lengths, portions, dtype, num_pages=64):
    """Random paged cache with shuffled pages.  ``lengths[b]``: tokens request b holds after
    the step; ``portions[b]``: how many of them are the step's queries."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    max_pages = max(-(-n // page_size) for n in lengths) + 1
    num_pages = max(num_pages, sum(-(-n // page_size) for n in lengths) + 5)
    k = (torch.randn(num_pages, kv_heads, page_size, dh, generator=g)).to(dtype).cuda()
    v = (torch.randn(num_pages, kv_heads, page_size, dh, generator=g)).to(dtype).cuda()
    perm = torch.randperm(num_pages, generator=g).tolist()
    table = torch.full((len(lengths), max_pages), -1, dtype=torch.int32)
    for b, n in enumerate(lengths):
        for i in range(-(-n // page_size)):
            table[b, i] = perm.pop()
    seq, pos = [], []
    for b, (n, p) in enumerate(zip(lengths, portions)):
        seq += [b] * p
        pos += list(range(n - p, n))
    t = len(seq)
    q = (torch.randn(t, n_heads * dh, generator=g)).to(dtype).cuda()
    return q, k, v, table.cuda(), torch.tensor(seq, dtype=torch.int32).cuda(), \
        torch.tensor(pos, dtype=torch.int32).cuda()


def _ref_attention(q, k, v, table, seq, pos, n_heads, scale, window):
    t = q.shape[0]
    num_pages, kv_heads, page_size, dh = k.shape
    out = torch.zeros(t, n_heads * dh, dtype=torch.float32, device="cuda")
    kf, vf, qf = k.float(), v.float(), q.float()
    for i in range(t):
        b, p = int(seq[i]), int(pos[i])
        lo = max(0, p - window + 1) if window else 0
        js = torch.arange(lo, p + 1, device="cuda")
        pages = table[b, (js // page_size).long()].long()
        for h in range(n_heads):
            hk = h // (n_heads // kv_heads)
            kk = kf[pages, hk, (js % page_size).long()]          # [n, dh]
            vv = vf[pages, hk, (js % page_size).long()]
            s = (kk @ qf[i, h * dh:(h + 1) * dh]) * scale
            out[i, h * dh:(h + 1) * dh] = torch.softmax(s, 0) @ vv
    return out


ATTN_CASES = [
    # heads, kv heads, head size, page size, window
    (4, 4, 16, 16, None), (3, 3, 32, 64, None), (6, 2, 64, 64, None), (5, 1, 48, 32, 40),
    (2, 2, 128, 128, None), (8, 4, 80, 64, 100), (2, 1, 256, 64, None),
]


@pytest.mark.parametrize("nh,nkv,dh,ps,window", ATTN_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_generic(nh, nkv, dh, ps, window, dtype):
    ops = _ops()
    lengths, portions = [1, 70, 300, 129], [1, 5, 1, 129]
    q, k, v, table, seq, pos = _paged_case(1, nh, nkv, dh, ps, lengths, portions, dtype)
    out = torch.zeros_like(q)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ops.attention_generic(out, q, k, v, table, seq, pos, q.shape[0], nh, 0.3, window, 512, status)
    ref = _ref_attention(q, k, v, table, seq, pos, nh, 0.3, window)
    assert status.tolist() == [0, 0, 0, 0]
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert float((out.float() - ref).abs().max()) <= tol


@pytest.mark.parametrize("nh,nkv,dh,ps,window", ATTN_CASES)
@pytest.mark.parametrize("split_keys", [128, 384, 1024])
def test_attention_decode(nh, nkv, dh, ps, window, split_keys):
    """Short splits, splits of three stages, and one split that walks the whole context
    (its ring of buffers is used again)."""
    ops = _ops()
    lengths, portions = [1, 70, 300, 257, 1000, 256], [1, 2, 1, 3, 1, 1]
    q, k, v, table, seq, pos = _paged_case(2, nh, nkv, dh, ps, lengths, portions, torch.bfloat16)
    t = q.shape[0]
    splits = -(-1024 // split_keys)
    ws = torch.full((t * nh * splits * (dh + 4),), float("nan"), device="cuda")
    counters = torch.zeros(t * nh, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ref = _ref_attention(q, k, v, table, seq, pos, nh, 0.2, window)
    for _ in range(2):                      # twice: the counters must be left at zero
        out = torch.full_like(q, float("nan"))
        ops.attention_decode(out, q, k, v, table, seq, pos, None, None, t, nh, 0.2, window, ws,
                             counters, splits, status, split_keys=split_keys)
        assert status.tolist() == [0, 0, 0, 0]
        assert float((out.float() - ref).abs().max()) <= 2e-2
        assert int(counters.abs().sum()) == 0
    if split_keys == 128:
        # contexts of up to 2,000 keys: 16 splits, more than a cluster takes, so the partial
        # results go through the workspace (filled with NaN here) and the last CTA merges
        lengths2, portions2 = [2000, 5, 1300, 1025], [1, 1, 2, 1]
        q2, k2, v2, table2, seq2, pos2 = _paged_case(8, nh, nkv, dh, ps, lengths2, portions2,
                                                     torch.bfloat16)
        t2, splits2 = q2.shape[0], 16
        ws2 = torch.full((t2 * nh * splits2 * (dh + 4),), float("nan"), device="cuda")
        counters2 = torch.zeros(t2 * nh, dtype=torch.int32, device="cuda")
        ref2 = _ref_attention(q2, k2, v2, table2, seq2, pos2, nh, 0.2, window)
        for _ in range(2):
            out2 = torch.full_like(q2, float("nan"))
            ops.attention_decode(out2, q2, k2, v2, table2, seq2, pos2, None, None, t2, nh, 0.2,
                                 window, ws2, counters2, splits2, status, split_keys=128)
            assert status.tolist() == [0, 0, 0, 0]
            assert float((out2.float() - ref2).abs().max()) <= 2e-2
            assert int(counters2.abs().sum()) == 0
        assert window is not None or bool(torch.isfinite(ws2).any())
    # a token list picks tokens; the others are not touched
    order = torch.tensor([t - 1, 0, 3], dtype=torch.int32, device="cuda")
    count = torch.tensor([2], dtype=torch.int32, device="cuda")
    out = torch.zeros_like(q)
    ops.attention_decode(out, q, k, v, table, seq, pos, order, count, 3, nh, 0.2, window, ws,
                         counters, splits, status, split_keys=split_keys)
    assert float((out[t - 1].float() - ref[t - 1]).abs().max()) <= 2e-2
    assert float((out[0].float() - ref[0]).abs().max()) <= 2e-2
    assert float(out[3].abs().max()) == 0.0


@pytest.mark.parametrize("nh,nkv,dh,ps", [(12, 12, 64, 64), (3, 1, 48, 16), (4, 2, 128, 32),
                                          (2, 2, 16, 128), (5, 5, 80, 8)])
@pytest.mark.parametrize("split_keys", [128, 512, 1024])
def test_attention_decode_streaming_variant_gives_the_same_bits(nh, nkv, dh, ps, split_keys):
    """Keys through the shared-memory ring (bulk copies of page runs) or through register
    batches: the same keys reach the same lanes in the same order, so the outputs are equal
    bit for bit; both agree with the plain reference."""
    ops = _ops()
    lengths, portions = [1, 64, 65, 300, 1000, 1024, 513], [1, 1, 2, 1, 3, 1, 1]
    q, k, v, table, seq, pos = _paged_case(6, nh, nkv, dh, ps, lengths, portions, torch.bfloat16)
    t = q.shape[0]
    splits = -(-1024 // split_keys)
    ws = torch.full((t * nh * splits * (dh + 4),), float("nan"), device="cuda")
    counters = torch.zeros(t * nh, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ref = _ref_attention(q, k, v, table, seq, pos, nh, 0.2, None)
    outs = []
    try:
        for mode in (0, 1, 1):
            ops.decode_stream(mode)
            out = torch.full_like(q, float("nan"))
            ops.attention_decode(out, q, k, v, table, seq, pos, None, None, t, nh, 0.2, None, ws,
                                 counters, splits, status, split_keys=split_keys)
            torch.cuda.synchronize()
            assert status.tolist() == [0, 0, 0, 0]
            assert int(counters.abs().sum()) == 0
            outs.append(out)
    finally:
        ops.decode_stream(-1)
    assert float((outs[0].float() - ref).abs().max()) <= 2e-2
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])


RING_CASES = [
    # heads, kv heads, page size, window
    (12, 12, 64, None), (6, 2, 64, None), (4, 2, 16, None), (3, 1, 8, 70), (5, 5, 128, 100),
    (2, 2, 32, None),
]


@pytest.mark.parametrize("nh,nkv,ps,window", RING_CASES)
@pytest.mark.parametrize("stages", [0, 2, 3, 4])
def test_attention_decode_ring(nh, nkv, ps, window, stages):
    """The ring kernel (persistent CTAs, keys and values by bulk copies into per-warp rings)
    against the plain reference: contexts from 1 to 2,000 keys (a (token, head) shared by many
    warps, and many of them to a warp), several tokens of one request, a token list, and the
    unused tail of every page poisoned with NaN (what an earlier owner left must not leak)."""
    ops = _ops()
    dh = 64
    assert ops.decode_ring_supports(dh, ps) and not ops.decode_ring_supports(48, ps)
    lengths, portions = [1, 70, 300, 257, 2000, 256, 33, 1025], [1, 2, 1, 4, 1, 1, 3, 1]
    q, k, v, table, seq, pos = _paged_case(11, nh, nkv, dh, ps, lengths, portions, torch.bfloat16)
    for b, n in enumerate(lengths):                      # rows past a request's last token
        last = int(table[b, (n - 1) // ps])
        k[last, :, (n - 1) % ps + 1:, :] = float("nan")
        v[last, :, (n - 1) % ps + 1:, :] = float("nan")
    t = q.shape[0]
    ws = torch.full((ops.decode_ring_workspace(t, nh, dh),), float("nan"), device="cuda")
    counters = torch.zeros(t * nh, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ref = _ref_attention(q, k, v, table, seq, pos, nh, 0.2, window)
    for _ in range(2):                                   # twice: the counters must be left at zero
        out = torch.full_like(q, float("nan"))
        ops.attention_decode_ring(out, q, k, v, table, seq, pos, None, None, t, nh, 0.2, window,
                                  ws, counters, status, new_keys=4, stages=stages, max_context=2048)
        torch.cuda.synchronize()
        assert status.tolist() == [0, 0, 0, 0]
        err = (out.float() - ref).abs()
        assert float(err.max()) <= 2e-2, f"worst token {int(err.max(dim=1).values.argmax())}"
        assert int(counters.abs().sum()) == 0
    # the step's own keys and values handed over beside the queries: the kernel must take
    # those rows from there (their cache rows are poisoned here) and everything else from the cache
    k_new = torch.zeros(t, nkv * dh, dtype=torch.bfloat16, device="cuda")
    v_new = torch.zeros_like(k_new)
    k2, v2 = k.clone(), v.clone()
    for i in range(t):
        b, p = int(seq[i]), int(pos[i])
        page, off = int(table[b, p // ps]), p % ps
        k_new[i], v_new[i] = k[page, :, off, :].reshape(-1), v[page, :, off, :].reshape(-1)
        k2[page, :, off, :] = float("nan")
        v2[page, :, off, :] = float("nan")
    both = torch.cat([k_new, v_new], dim=1)              # column slices of one wider tensor
    out = torch.full_like(q, float("nan"))
    ops.attention_decode_ring(out, q, k2, v2, table, seq, pos, None, None, t, nh, 0.2, window, ws,
                              counters, status, new_keys=4, stages=stages, max_context=2048,
                              kv_new=(both[:, :nkv * dh], both[:, nkv * dh:]))
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    assert float((out.float() - ref).abs().max()) <= 2e-2
    # a token list picks tokens (its length on the device); the others are not touched
    order = torch.tensor([t - 1, 0, 5, 3], dtype=torch.int32, device="cuda")
    count = torch.tensor([3], dtype=torch.int32, device="cuda")
    out = torch.zeros_like(q)
    ops.attention_decode_ring(out, q, k, v, table, seq, pos, order, count, 4, nh, 0.2, window, ws,
                              counters, status, new_keys=4, stages=stages, max_context=2048)
    for i in (t - 1, 0, 5):
        assert float((out[i].float() - ref[i]).abs().max()) <= 2e-2
    assert float(out[3].abs().max()) == 0.0
    # a position beyond the block table is recorded, not read
    bad = pos.clone()
    bad[0] = table.shape[1] * ps + 5
    ops.attention_decode_ring(out, q, k, v, table, seq, bad, None, None, t, nh, 0.2, window, ws,
                              counters, status, new_keys=4, stages=stages, max_context=2048)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 2


def test_attention_decode_ring_sees_what_the_step_appended():
    """The kernel asks for old keys before the kernel it depends on has finished, and for the
    rows the step itself wrote only afterwards: a far key written by the kernel right before it
    in the stream, at the token's own position and three before it, must be seen."""
    ops = _ops()
    nh, dh, ps, n = 2, 64, 64, 1000
    q, k, v, table, seq, pos = _paged_case(4, nh, nh, dh, ps, [n], [1], torch.bfloat16)
    ws = torch.zeros(ops.decode_ring_workspace(1, nh, dh), device="cuda")
    counters = torch.zeros(nh, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    big = (q[0].view(nh, dh) * 4.0).clone()
    for back in (0, 3):
        kk, vv = k.clone(), v.clone()
        p = n - 1 - back
        page, off = int(table[0, p // ps]), p % ps
        out = torch.zeros_like(q)
        # a long kernel first, then the write, then attention: all on one stream
        filler = torch.randn(4096, 4096, device="cuda")
        for _ in range(3):
            filler = filler @ filler
        kk[page, :, off, :] = big                      # aligned with the query: huge score
        ops.attention_decode_ring(out, q, kk, vv, table, seq, pos, None, None, 1, nh, 0.125, None,
                                  ws, counters, status, new_keys=4, max_context=1024)
        torch.cuda.synchronize()
        assert status.tolist() == [0, 0, 0, 0]
        assert float((out[0].view(nh, dh).float() - vv[page, :, off].float()).abs().max()) < 0.05, back


def _prefill_parts(units, most):
    """Workspace of the tensor-memory prompt kernel's key parts."""
    return (torch.empty(units * most * 8192, device="cuda"),
            torch.empty(units * most * 256, device="cuda"),
            torch.zeros(units, dtype=torch.int32, device="cuda"))


PREFILL_CASES = ATTN_CASES + [(12, 12, 64, 64, None), (4, 2, 64, 128, 100), (3, 1, 64, 64, 70)]


@pytest.mark.parametrize("nh,nkv,dh,ps,window", PREFILL_CASES)
@pytest.mark.parametrize("tile", [64, 128])
def test_attention_prefill(nh, nkv, dh, ps, window, tile):
    """Both prompt kernels (mma.sync for every head size, tcgen05 where it applies) on work
    items of up to 64 and up to 128 rows."""
    ops = _ops()
    assert ops.prefill_supports(dh) and ops.prefill_tile() == 128
    lengths, portions = [5, 70, 300, 200, 64, 500], [5, 70, 130, 9, 64, 300]
    q, k, v, table, seq, pos = _paged_case(3, nh, nkv, dh, ps, lengths, portions, torch.bfloat16)
    tiles, row = [], 0
    for b, p in enumerate(portions):
        for r0 in range(0, p, tile):
            tiles.append((b, row + r0, min(tile, p - r0)))
        row += p
    tr = torch.tensor([x[0] for x in tiles], dtype=torch.int32, device="cuda")
    t0 = torch.tensor([x[1] for x in tiles], dtype=torch.int32, device="cuda")
    tn = torch.tensor([x[2] for x in tiles], dtype=torch.int32, device="cuda")
    ref = _ref_attention(q, k, v, table, seq, pos, nh, 0.2, window)
    kernels = [("mma.sync", ops.attention_prefill, {})]
    if ops.prefill_tc_supports(dh, ps):
        # one CTA per tile, and the keys of a tile in chunks of 1, 2 and 4 blocks, a CTA each
        kernels.append(("tcgen05", ops.attention_prefill_tc, {}))
        for part in (1, 2, 4):
            most = -(-(-(-max(lengths) // 64)) // part) + 1
            kernels.append((f"tcgen05 / parts of {part}", ops.attention_prefill_tc,
                            {"part_blocks": part, "max_parts": most,
                             "parts": _prefill_parts(len(tiles) * nh, most)}))
        if tile == 128:
            # the planner's own list (exactly the CTAs with work, longest first, long tiles in
            # parts): with the balance it chooses, and with small parts forced by telling it
            # of a device with few SMs
            import numpy as np
            from pretrained_rstr_b200.parts.attention import AttentionWork
            for small in (False, True):
                planner = AttentionWork()
                if small:
                    planner.MIN_PART = 1
                planner.note_mixer(nh, window, 10_000 if small else None)
                host = {name: np.full(cap, fill, dtype=np.int32)
                        for name, (cap, fill) in planner.arrays(sum(portions), len(portions)).items()}
                got = planner.fill(host, portions, [n - p for n, p in zip(lengths, portions)])
                assert got["tiles"] == len(tiles)
                assert host["tile_row0"][:len(tiles)].tolist() == [x[1] for x in tiles]
                dev = {name: torch.from_numpy(a).cuda() for name, a in host.items()}
                slots = planner.slot_cap()
                ws = (torch.full((slots * nh * 8192,), float("nan"), device="cuda"),
                      torch.full((slots * nh * 256,), float("nan"), device="cuda"),
                      torch.zeros(slots * nh, dtype=torch.int32, device="cuda"))
                split = int((host["item_part"][:got["items"]] >= 0).sum())
                assert not small or split > 0
                kernels.append((f"tcgen05 / listed, {got['items']} items, {split} of them parts",
                                ops.attention_prefill_tc,
                                {"parts": ws, "items": (dev["item_tile"], dev["item_part"], dev["item_slot"],
                                                        None, dev["part_blocks"], got["items"], slots)}))
    else:
        assert not (dh == 64 and ps % 64 == 0)
    # what a page's earlier owner may have left after a request's last position must not
    # reach the output: not-a-number there, in keys and in values
    k, v = k.clone(), v.clone()
    for b, n in enumerate(lengths):
        if n % ps:
            page = int(table[b, (n - 1) // ps])
            k[page, :, n % ps:, :] = float("nan")
            v[page, :, n % ps:, :] = float("nan")
    for name, kernel, kw in kernels:
        status = torch.zeros(4, dtype=torch.int32, device="cuda")
        out = torch.full_like(q, float("nan"))
        kernel(out, q, k, v, table, pos, tr, t0, tn, None, len(tiles), nh, 0.2, window, status, **kw)
        assert status.tolist() == [0, 0, 0, 0], name
        err = (out.float() - ref).abs()
        assert float(err.max()) <= 2e-2, \
            f"{name}: worst row {int(err.max(dim=1).values.argmax())}"


def test_attention_far_key_stands_out():
    """One early key among a thousand is made to dominate: every kernel must find it."""
    ops = _ops()
    nh, dh, ps, n = 2, 64, 64, 1000
    q, k, v, table, seq, pos = _paged_case(4, nh, nh, dh, ps, [n], [66], torch.bfloat16)
    far = 3
    page, off = int(table[0, far // ps]), far % ps
    k[page, :, off, :] = q[-1].view(nh, dh) * 4.0      # aligned with the last query: huge score
    ref = _ref_attention(q, k, v, table, seq, pos, nh, 0.125, None)
    assert float((ref[-1].view(nh, dh) - v[page, :, off].float()).abs().max()) < 0.05
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    out = torch.zeros_like(q)
    tr = torch.zeros(2, dtype=torch.int32, device="cuda")
    t0 = torch.tensor([0, 64], dtype=torch.int32, device="cuda")
    tn = torch.tensor([64, 2], dtype=torch.int32, device="cuda")
    ops.attention_prefill(out, q, k, v, table, pos, tr, t0, tn, None, 2, nh, 0.125, None, status)
    assert float((out.float() - ref).abs().max()) <= 2e-2
    for part in (0, 1, 3, 8):
        out_tc = torch.zeros_like(q)
        most = -(-16 // part) if part else 1
        ops.attention_prefill_tc(out_tc, q, k, v, table, pos, tr, t0, tn, None, 2, nh, 0.125, None,
                                 status, part_blocks=part, max_parts=most,
                                 parts=_prefill_parts(2 * nh, most) if part else None)
        assert float((out_tc.float() - ref).abs().max()) <= 2e-2, part
        assert status.tolist() == [0, 0, 0, 0]
    t = q.shape[0]
    splits = -(-1024 // ops.decode_split())
    ws = torch.zeros(t * nh * splits * (dh + 4), device="cuda")
    counters = torch.zeros(t * nh, dtype=torch.int32, device="cuda")
    out2 = torch.zeros_like(q)
    ops.attention_decode(out2, q, k, v, table, seq, pos, None, None, t, nh, 0.125, None, ws,
                         counters, splits, status)
    assert float((out2.float() - ref).abs().max()) <= 2e-2
    # a launch with too few splits for the context is recorded, not computed wrongly
    ops.attention_decode(out2, q, k, v, table, seq, pos, None, None, t, nh, 0.125, None, ws,
                         counters, 2, status)
    assert status.tolist()[0] == 2


# ------------------------------------------------------------------ decode-time product
@pytest.mark.parametrize("m,n,k", [(1, 192, 64), (8, 2304, 768), (5, 1000, 96), (16, 320, 96),
                                   (33, 768, 3072), (64, 50257, 768), (3, 24, 1608),
                                   (8, 100, 6400), (12, 200, 1000), (2, 50, 1600), (16, 72, 3072),
                                   (13, 808, 768), (24, 2304, 768), (32, 328, 3072), (17, 100, 64),
                                   (29, 1000, 1600)])
@pytest.mark.parametrize("variant", ["plain_f32", "bias_gelu_bf16", "bias_resid_f32", "norm_bf16"])
def test_gemm_smallm(m, n, k, variant):
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    a = (torch.randn(m, k, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    bias = torch.randn(n, device="cuda", generator=g) * 0.2
    resid = torch.randn(m, n, device="cuda", generator=g)
    ref = a.float() @ w.float().t()
    if variant == "plain_f32":
        out = torch.full((m, n), float("nan"), device="cuda")
        ops.gemm_smallm(out, w, a=a)
        tol = 2e-4
    elif variant == "bias_gelu_bf16":
        out = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
        ops.gemm_smallm(out, w, a=a, bias=bias, act="gelu_new")
        ref = _act("gelu_new", ref + bias)
        tol = 2e-2
    elif variant == "bias_resid_f32":
        out = resid.clone()
        ops.gemm_smallm(out, w, a=a, bias=bias, resid=out)
        ref = ref + bias + resid
        tol = 2e-4
    else:
        xf = torch.randn(m, k, device="cuda", generator=g) * 3.0 + 0.5
        gamma = torch.randn(k, device="cuda", generator=g)
        beta = torch.randn(k, device="cuda", generator=g)
        out = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
        if k > ops.smallm_limits()[1]:          # too wide for the fused norm: refused, not wrong
            with pytest.raises(ops.KernelArgumentError, match="size"):
                ops.gemm_smallm(out, w, norm_input=xf, gamma=gamma, beta=beta, eps=1e-6)
            return
        ops.gemm_smallm(out, w, norm_input=xf, gamma=gamma, beta=beta, eps=1e-6, bias=bias)
        normed = torch.nn.functional.layer_norm(xf, (k,), gamma, beta, 1e-6).to(torch.bfloat16)
        ref = normed.float() @ w.float().t() + bias
        tol = 3e-2
    scale = float(ref.abs().max())
    err = float((out.float() - ref).abs().max())
    assert err <= tol * max(1.0, scale), f"max |difference| {err:.3e} (scale {scale:.3g})"


@pytest.mark.parametrize("k", [768, 3072, 1000])
def test_gemm_smallm_rows_do_not_depend_on_the_batch(k):
    """One row alone and among 12: the same bits, the weights chunked or not; among 40
    (another kernel): the same up to rounding."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(9)
    a = torch.randn(40, k, device="cuda", generator=g).to(torch.bfloat16)
    w = torch.randn(256, k, device="cuda", generator=g).to(torch.bfloat16)
    big = torch.zeros(40, 256, device="cuda")
    ops.gemm_smallm(big, w, a=a)
    mid = torch.zeros(12, 256, device="cuda")
    ops.gemm_smallm(mid, w, a=a[10:22].contiguous())
    one = torch.zeros(1, 256, device="cuda")
    ops.gemm_smallm(one, w, a=a[17:18].contiguous())
    assert torch.equal(one[0], mid[7])             # the same kernel: the same bits
    wide = torch.zeros(30, 256, device="cuda")     # 30 rows: the other kernel again
    ops.gemm_smallm(wide, w, a=a[5:35].contiguous())
    assert float((wide[12] - one[0]).abs().max()) <= 2e-4 * float(big[17].abs().max())
    # 40 rows go to another kernel, which adds the same products in another order
    assert float((big[17] - one[0]).abs().max()) <= 2e-4 * float(big[17].abs().max())


@pytest.mark.parametrize("m", [5, 13, 16, 30])
@pytest.mark.parametrize("k", [64, 768, 1024, 1600])
def test_gemm_smallm_fused_norm_with_an_outlier_channel(k, m):
    """A row whose first channel is thousands among values of order one (as massive
    activations are): the fused norm's statistics are mean first, then centred squares, and
    agree with the two-pass norm kernel followed by the plain product; a one-pass variance on
    data shifted by the first element would cancel here."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(k)
    n = 96
    x = torch.randn(m, k, device="cuda", generator=g)
    x[:, 0] = torch.tensor([3e3, -2e3, 5e3, 1.0, 8e3], device="cuda").repeat(7)[:m]
    x[2, k // 2] = -4e3
    x[m - 1, k // 3] = 6e3
    gamma = torch.rand(k, device="cuda", generator=g) + 0.5
    beta = torch.randn(k, device="cuda", generator=g) * 0.1
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    fused = torch.zeros(m, n, device="cuda")
    ops.gemm_smallm(fused, w, norm_input=x, gamma=gamma, beta=beta, eps=1e-5)
    normed = torch.zeros(m, k, device="cuda", dtype=torch.bfloat16)
    ops.layernorm(normed, x, gamma, beta, 1e-5)
    apart = torch.zeros(m, n, device="cuda")
    ops.gemm_smallm(apart, w, a=normed)
    ref = torch.nn.functional.layer_norm(x.double(), (k,), gamma.double(), beta.double(), 1e-5)
    ref = (ref.float().to(torch.bfloat16).float() @ w.float().t())
    scale = max(1.0, float(ref.abs().max()))
    assert float((fused - apart).abs().max()) <= 2e-3 * scale
    assert float((fused - ref).abs().max()) <= 1e-2 * scale


# ------------------------------------------------------------------------ small kernels
@pytest.mark.parametrize("rows,width", [(1, 64), (7, 96), (33, 1608), (5, 50000), (40, 768), (17, 64), (300, 1000)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_layernorm(rows, width, out_dtype):
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(rows)
    x = torch.randn(rows + 3, width, device="cuda", generator=g) * 2 + 1
    gamma = torch.randn(width, device="cuda", generator=g)
    beta = torch.randn(width, device="cuda", generator=g)
    idx = torch.randperm(rows + 3, device="cuda", generator=g)[:rows].to(torch.int32)
    out = torch.zeros(rows, width, device="cuda", dtype=out_dtype)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ops.layernorm(out, x, gamma, beta, 1e-6, rows=idx, status=status)
    ref = torch.nn.functional.layer_norm(x[idx.long()].double(), (width,), gamma.double(),
                                         beta.double(), 1e-6).float()
    tol = 2e-5 if out_dtype == torch.float32 else 4e-2
    assert float((out.float() - ref).abs().max()) <= tol * max(1.0, float(ref.abs().max()))
    bad = torch.tensor([rows + 10], dtype=torch.int32, device="cuda")
    ops.layernorm(out[:1], x, gamma, beta, 1e-6, rows=bad, status=status)
    assert status.tolist()[0] == 6                      # refused, recorded, nothing read


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_and_range_check(dtype):
    ops = _ops()
    wte = torch.randn(1000, 96, device="cuda").to(dtype)
    wpe = torch.randn(256, 96, device="cuda").to(dtype)
    tok = torch.tensor([5, 999, 0, 17], dtype=torch.int32, device="cuda")
    pos = torch.tensor([0, 255, 3, 9], dtype=torch.int32, device="cuda")
    out = torch.zeros(4, 96, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ops.embed(out, tok, pos, wte, wpe, status)
    assert torch.equal(out, wte[tok.long()].float() + wpe[pos.long()].float())
    assert status.tolist() == [0, 0, 0, 0]
    ops.embed(out, torch.tensor([1, 1000, 2, 3], dtype=torch.int32, device="cuda"), pos, wte, wpe,
              status)
    assert status.tolist() == [1, 1, 1000, 1000] and float(out[1].abs().max()) == 0.0


def test_kv_append_and_copy_pages():
    ops = _ops()
    pages, heads, ps, dh = 6, 3, 16, 32
    store = torch.zeros(4, pages, heads, ps, dh, device="cuda", dtype=torch.bfloat16)
    k, v = store[2], store[3]
    qkv = torch.randn(5, 3 * heads * dh, device="cuda").to(torch.bfloat16)
    slots = torch.tensor([3 * ps + 15, -1, 0, 5 * ps + 1, 2 * ps + 7], dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ops.kv_append(k, v, qkv[:, heads * dh:2 * heads * dh], qkv[:, 2 * heads * dh:], slots, 5, status)
    for t, s in enumerate(slots.tolist()):
        if s < 0:
            continue
        assert torch.equal(k[s // ps, :, s % ps, :].reshape(-1), qkv[t, heads * dh:2 * heads * dh])
        assert torch.equal(v[s // ps, :, s % ps, :].reshape(-1), qkv[t, 2 * heads * dh:])
    assert int((k != 0).any(dim=-1).sum()) <= 4 * heads      # the skipped token wrote nothing
    pairs = torch.tensor([[3, 1], [5, 4]], dtype=torch.int32, device="cuda")
    ops.copy_pages(store, pairs, 2, status)
    assert torch.equal(store[:, 1], store[:, 3]) and torch.equal(store[:, 4], store[:, 5])
    assert status.tolist() == [0, 0, 0, 0]
    ops.kv_append(k, v, qkv[:, :heads * dh], qkv[:, :heads * dh],
                  torch.tensor([pages * ps], dtype=torch.int32, device="cuda"), 1, status)
    assert status.tolist()[0] == 3


@pytest.mark.parametrize("words", [1, 37, 256, 1500, 4096])
def test_step_words_cross_the_bus_inside_kernels(words):
    """A step's description read from pinned memory by a kernel (with the ids that name
    places among the last tokens put in on the way), and a result written back by one."""
    ops = _ops()
    g = torch.Generator().manual_seed(words)
    host = torch.randint(0, 1000, (words + 8,), dtype=torch.int32, generator=g).pin_memory()
    address = ops.host_device_address(host)
    assert address != 0
    assert ops.host_device_address(torch.zeros(4, dtype=torch.int32)) == 0      # pageable
    prev = torch.arange(100, 108, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    tokens_at, n_tokens = min(5, words - 1), min(20, words - min(5, words - 1))
    expect = host.clone()
    for i in range(tokens_at, tokens_at + n_tokens, 3):
        host[i] = -(i % 8) - 1
        expect[i] = 100 + i % 8
    if words > 30:                       # a negative word outside the token range stays
        host[words - 1] = -3
        expect[words - 1] = -3
    dev = torch.full((words + 8,), -7, dtype=torch.int32, device="cuda")
    ops.fetch_step(dev, address, words, tokens_at, n_tokens, prev, status)
    assert torch.equal(dev[:words].cpu(), expect[:words])
    assert bool((dev[words:] == -7).all())
    assert int(status[0]) == 0
    # without the last tokens nothing is replaced
    ops.fetch_step(dev, address, words, tokens_at, n_tokens, None, status)
    assert torch.equal(dev[:words].cpu(), host[:words])
    # a place beyond the last tokens is recorded, not read
    host[tokens_at] = -9
    ops.fetch_step(dev, address, words, tokens_at, n_tokens, prev, status)
    torch.cuda.synchronize()
    assert int(status[0]) != 0 and int(dev[tokens_at]) == 0
    # and back
    out = torch.full((words + 8,), -1, dtype=torch.int32).pin_memory()
    n_back = min(words, 128 + 68)
    ops.publish_result(ops.host_device_address(out), dev, n_back)
    torch.cuda.synchronize()
    assert torch.equal(out[:n_back], dev[:n_back].cpu())
    assert bool((out[n_back:] == -1).all())


@pytest.mark.parametrize("rows", [1, 5, 64])
def test_sample_kernel_publishes_its_result(rows):
    """The launch's last CTA writes the chosen ids and the words behind them to pinned host
    memory; the counter it uses is zero again afterwards, launch after launch."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(rows)
    result = torch.zeros(rows + 4, dtype=torch.int32, device="cuda")
    result[rows:] = torch.tensor([0, 11, 22, 33], dtype=torch.int32)
    workspace = torch.zeros(ops.sample_workspace_words(), dtype=torch.int32, device="cuda")
    counter = workspace[:1]
    host = torch.full((rows + 8,), -5, dtype=torch.int32).pin_memory()
    address = ops.host_device_address(host)
    for turn in range(3):
        logits = torch.randn(rows, 1000, device="cuda", generator=g)
        ops.sample(result[:rows], logits, rows, publish=(address, result, rows + 4), workspace=workspace)
        torch.cuda.synchronize()
        assert host[:rows].tolist() == logits.argmax(dim=1).tolist()
        assert host[rows:rows + 4].tolist() == [0, 11, 22, 33] and host[rows + 4:].tolist() == [-5] * 4
        assert int(counter[0]) == 0
    # greedy rows with a publishing target are searched in slices by several CTAs: ties go to
    # the lowest id and a NaN wins, wherever in the row they lie; odd widths and row starts
    for vocab in (1000, 50257, 515):
        wide = torch.randn(rows, vocab + 3, device="cuda", generator=g)[:, 1:vocab + 1]
        want = wide.argmax(dim=1).tolist()
        if rows >= 5:
            wide[0, vocab - 1] = 50.0
            wide[0, vocab // 2] = 50.0
            wide[0, 7] = 50.0
            wide[1, vocab - 2] = float("nan")
            wide[2, vocab - 2] = float("nan")
            wide[2, vocab // 3] = float("nan")
            wide[3, :] = float("-inf")
            wide[4, vocab - 1] = 60.0
            want[:5] = [7, vocab - 2, vocab // 3, 0, vocab - 1]
        ops.sample(result[:rows], wide, rows, publish=(address, result, rows + 4), workspace=workspace)
        torch.cuda.synchronize()
        assert host[:rows].tolist() == want and result[:rows].tolist() == want
        alone = torch.zeros(rows, dtype=torch.int32, device="cuda")
        ops.sample(alone, wide, rows)                   # one CTA a row: the same ids
        assert alone.tolist() == want
    temp = torch.full((rows,), 0.7, device="cuda")
    args = dict(temperature=temp, top_k=torch.full((rows,), 20, dtype=torch.int32, device="cuda"),
                top_p=torch.ones(rows, device="cuda"),
                seeds=torch.arange(rows, dtype=torch.int64, device="cuda"),
                fresh=torch.ones(rows, dtype=torch.int32, device="cuda"),
                slots=torch.arange(rows, dtype=torch.int32, device="cuda"),
                rng_states=torch.zeros(rows, dtype=torch.int64, device="cuda"))
    ops.sample(result[:rows], logits, rows, publish=(address, result, rows + 4), workspace=workspace, **args)
    torch.cuda.synchronize()
    assert host[:rows].tolist() == result[:rows].tolist() and int(counter[0]) == 0
    assert int(workspace[:4].abs().sum()) == 0             # the launch's counter is back at zero
    # the same rows by one CTA each choose the same tokens
    args["rng_states"] = torch.zeros(rows, dtype=torch.int64, device="cuda")
    alone = torch.zeros(rows, dtype=torch.int32, device="cuda")
    ops.sample(alone, logits, rows, **args)
    assert alone.tolist() == result[:rows].tolist()


def test_sample_kernel_greedy_ties_and_nan():
    ops = _ops()
    logits = torch.randn(6, 50257, device="cuda")
    logits[1, 77] = logits[1, 40000] = 99.0            # tie: lowest id
    logits[2, 123] = float("nan")                       # NaN wins
    logits[3, 50256] = 50.0                             # last column
    out = torch.zeros(6, dtype=torch.int32, device="cuda")
    ops.sample(out, logits, 6)
    want = logits.argmax(dim=1).tolist()
    want[1], want[2], want[3] = 77, 123, 50256
    assert out.tolist() == want


@pytest.mark.parametrize("several", [False, True])
@pytest.mark.parametrize("vocab", [50257, 1000, 37])
def test_sample_kernel_matches_the_plain_sampler(vocab, several):
    """Top-k selection (any k up to the limit, ties, NaN, rows of equal logits), temperature
    softmax, nucleus cut and the draw: the same token as the plain sampler on the same row,
    and the generator state left for the next draw."""
    import plain_gpt2
    ops = _ops()
    g = torch.Generator(device="cpu").manual_seed(vocab)
    rows = torch.randn(12, vocab, generator=g) * 0.7
    rows[1, 5] = rows[1, vocab - 1] = rows[1, 17] = 2.5        # ties among the candidates
    rows[2, 3] = float("nan")                                   # never a candidate
    rows[3, :] = 0.25                                           # all equal: the lowest ids
    rows[4, ::2] = -0.0                                         # -0 and +0 tie
    rows[4, 1::2] = 0.0
    rows[5] = torch.round(rows[5] * 4) / 4                      # many ties at the k-th value
    rows[6, 9] = float("-inf")
    ks = [40, 40, 40, 7, 5, 40, 40, 1, min(1024, vocab), 3, min(300, vocab), 40]
    ps = [1.0, 1.0, 0.9, 1.0, 1.0, 0.5, 1.0, 1.0, 0.95, 0.3, 1.0, 0.999]
    ts = [0.8, 1.0, 0.7, 1.3, 0.9, 0.8, 2.0, 0.5, 1.0, 0.8, 0.6, 1.5]
    # (the reference's candidate search skips -inf and NaN logits and leaves the unfilled
    # candidate slots at id 0, sampling.clj:14-29; the kernel takes such a logit as a candidate
    # of weight zero instead.  The two differ only when k exceeds the number of finite logits,
    # which these rows avoid.)
    ks[2], ks[6] = min(ks[2], vocab - 2), min(ks[6], vocab - 2)
    n = rows.shape[0]
    logits = rows.cuda()
    out = torch.zeros(n, dtype=torch.int32, device="cuda")
    states = torch.zeros(n, dtype=torch.int64, device="cuda")
    args = dict(temperature=torch.tensor(ts, device="cuda"),
                top_k=torch.tensor(ks, dtype=torch.int32, device="cuda"),
                top_p=torch.tensor(ps, device="cuda"),
                seeds=torch.arange(100, 100 + n, dtype=torch.int64, device="cuda"),
                slots=torch.arange(n, dtype=torch.int32, device="cuda"), rng_states=states)
    if several:       # (a workspace changes nothing for rows that sample)
        args["workspace"] = torch.zeros(ops.sample_workspace_words(), dtype=torch.int32, device="cuda")
    rngs = [plain_gpt2.JavaRandom(100 + i) for i in range(n)]
    for draw in range(3):                       # the second and third draw go on from the state
        fresh = torch.full((n,), 1 if draw == 0 else 0, dtype=torch.int32, device="cuda")
        ops.sample(out, logits, n, fresh=fresh, **args)
        got = out.tolist()
        for i in range(n):
            # (the kernel's temperature is a float32, the plain sampler gets the same value)
            t32 = float(torch.tensor(ts[i], dtype=torch.float32))
            p32 = float(torch.tensor(ps[i], dtype=torch.float32))
            want = plain_gpt2.sample(rows[i], t32, ks[i], p32, rngs[i])
            assert got[i] == want, f"row {i}, draw {draw}: {got[i]} != {want}"


@pytest.mark.parametrize("m", [1, 8, 13])
def test_gemm_smallm_fused_norm_of_gathered_rows(m):
    """The fused norm may take its rows from anywhere in the input (the wanted rows of a
    step before the head): the same bits as the norm of those rows placed in order; an index
    outside the input gives a zero row and is recorded."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(m)
    k, n, t = 768, 1000, 40
    x = torch.randn(t, k, device="cuda", generator=g)
    gamma = torch.rand(k, device="cuda", generator=g) + 0.5
    beta = torch.randn(k, device="cuda", generator=g) * 0.1
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    rows = torch.randperm(t, generator=torch.Generator().manual_seed(m))[:m].to(torch.int32).cuda()
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    gathered = torch.zeros(m, n, device="cuda")
    ops.gemm_smallm(gathered, w, norm_input=x, gamma=gamma, beta=beta, eps=1e-5, norm_rows=rows,
                    status=status)
    in_order = torch.zeros(m, n, device="cuda")
    ops.gemm_smallm(in_order, w, norm_input=x[rows.long()].contiguous(), gamma=gamma, beta=beta, eps=1e-5)
    assert torch.equal(gathered, in_order) and status.tolist() == [0, 0, 0, 0]
    ref = torch.nn.functional.layer_norm(x[rows.long()].double(), (k,), gamma.double(), beta.double(), 1e-5)
    ref = ref.float().to(torch.bfloat16).float() @ w.float().t()
    assert float((gathered - ref).abs().max()) <= 1e-2 * float(ref.abs().max())
    rows[m - 1] = t                                      # one index outside the input
    ops.gemm_smallm(gathered, w, norm_input=x, gamma=gamma, beta=beta, eps=1e-5, norm_rows=rows,
                    status=status)
    torch.cuda.synchronize()
    assert status.tolist()[0] != 0 and float(gathered[m - 1].abs().max()) == 0.0
    assert torch.equal(gathered[:m - 1], in_order[:m - 1])


def test_gemm_smallm_scatters_keys_and_values_to_the_cache():
    """The decode-time QKV product writes its key and value columns to the cache slots
    itself; the result equals the product followed by the append kernel."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(3)
    m, heads, kv_heads, dh, ps, pages, k = 7, 6, 3, 32, 16, 9, 96
    q_width, kv_width = heads * dh, kv_heads * dh
    n = q_width + 2 * kv_width
    a = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.2).to(torch.bfloat16)
    bias = torch.randn(n, device="cuda", generator=g)
    slots = torch.tensor([5, ps * 3 + 15, -1, ps * 8, 0, ps * 2 + 1, ps * 8 + 7], dtype=torch.int32,
                         device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    k1 = torch.zeros(pages, kv_heads, ps, dh, device="cuda", dtype=torch.bfloat16)
    v1, k2, v2 = torch.zeros_like(k1), torch.zeros_like(k1), torch.zeros_like(k1)
    out1 = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
    out2 = torch.zeros_like(out1)
    ops.gemm_smallm(out1, w, a=a, bias=bias, kv_scatter=(k1, v1, slots, q_width), status=status)
    ops.gemm_smallm(out2, w, a=a, bias=bias)
    ops.kv_append(k2, v2, out2[:, q_width:q_width + kv_width], out2[:, q_width + kv_width:], slots, m,
                  status)
    torch.cuda.synchronize()
    assert torch.equal(out1, out2) and torch.equal(k1, k2) and torch.equal(v1, v2)
    assert int((k1 != 0).any(dim=-1).sum()) == 6 * kv_heads and status.tolist() == [0, 0, 0, 0]


def test_gemm_smallm_scatters_at_27_rows():
    """The same with 27 tokens, against the tensor-memory product and the append kernel."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(4)
    m, heads, kv_heads, dh, ps, pages, k = 27, 6, 3, 32, 16, 9, 128
    q_width, kv_width = heads * dh, kv_heads * dh
    n = q_width + 2 * kv_width
    a = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.2).to(torch.bfloat16)
    bias = torch.randn(n, device="cuda", generator=g)
    order = torch.randperm(pages * ps, generator=torch.Generator().manual_seed(1))[:m].to(torch.int32)
    order[3] = -1
    slots = order.cuda()
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    k1 = torch.zeros(pages, kv_heads, ps, dh, device="cuda", dtype=torch.bfloat16)
    v1, k2, v2 = torch.zeros_like(k1), torch.zeros_like(k1), torch.zeros_like(k1)
    out1 = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
    out2 = torch.zeros_like(out1)
    ops.gemm_smallm(out1, w, a=a, bias=bias, kv_scatter=(k1, v1, slots, q_width), status=status)
    ops.gemm_bf16(out2, a, w, bias)
    ops.kv_append(k2, v2, out2[:, q_width:q_width + kv_width], out2[:, q_width + kv_width:], slots, m,
                  status)
    torch.cuda.synchronize()
    ref = a.float() @ w.float().t() + bias
    assert float((out1.float() - ref).abs().max()) <= 2e-2 * float(ref.abs().max())
    assert float((k1.float() - k2.float()).abs().max()) <= 2e-2 * float(ref.abs().max())
    assert int((k1 != 0).any(dim=-1).sum()) == 26 * kv_heads and status.tolist() == [0, 0, 0, 0]
    # each cached row is the output row's own bits
    for t in (0, 11, 26):
        slot = int(slots[t])
        assert torch.equal(k1[slot // ps, :, slot % ps].reshape(-1), out1[t, q_width:q_width + kv_width])
        assert torch.equal(v1[slot // ps, :, slot % ps].reshape(-1), out1[t, q_width + kv_width:])


@pytest.mark.parametrize("m,heads,kv_heads,dh,ps", [(200, 6, 3, 32, 16), (130, 12, 12, 64, 64), (70, 5, 1, 24, 32),
                                                    (40, 6, 3, 32, 16), (64, 12, 12, 64, 64)])
def test_gemm_bf16_scatters_keys_and_values_to_the_cache(m, heads, kv_heads, dh, ps):
    """The prompt-time QKV product writes its key and value columns to the cache slots itself
    (whole 16-byte pieces, or element by element when the width is not a multiple of 32); the
    result equals the product followed by the append kernel."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(m)
    pages, k = (m + ps - 1) // ps + 3, 96
    q_width, kv_width = heads * dh, kv_heads * dh
    n = q_width + 2 * kv_width
    a = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.2).to(torch.bfloat16)
    bias = torch.randn(n, device="cuda", generator=g)
    slots = torch.randperm(pages * ps, device="cuda", generator=g)[:m].to(torch.int32)
    slots[3] = -1
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    k1 = torch.zeros(pages, kv_heads, ps, dh, device="cuda", dtype=torch.bfloat16)
    v1, k2, v2 = torch.zeros_like(k1), torch.zeros_like(k1), torch.zeros_like(k1)
    out1 = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
    out2 = torch.zeros_like(out1)
    ops.gemm_bf16(out1, a, w, bias=bias, kv_scatter=(k1, v1, slots, q_width), status=status)
    ops.gemm_bf16(out2, a, w, bias=bias, status=status)
    ops.kv_append(k2, v2, out2[:, q_width:q_width + kv_width], out2[:, q_width + kv_width:], slots, m,
                  status)
    torch.cuda.synchronize()
    assert torch.equal(out1, out2) and torch.equal(k1, k2) and torch.equal(v1, v2)
    assert status.tolist() == [0, 0, 0, 0]
    assert int((k1 != 0).any(dim=-1).sum()) == (m - 1) * kv_heads
    # keys and values to the cache alone: the same cache, the query columns as before; what
    # lies in the output's key and value columns afterwards does not matter
    k3, v3 = torch.zeros_like(k1), torch.zeros_like(k1)
    out3 = torch.full_like(out1, 7.0)
    ops.gemm_bf16(out3, a, w, bias=bias, kv_scatter=(k3, v3, slots, q_width, True), status=status)
    torch.cuda.synchronize()
    assert torch.equal(k3, k1) and torch.equal(v3, v1)
    assert torch.equal(out3[:, :q_width], out1[:, :q_width])


@pytest.mark.parametrize("m,n,k", [(64, 768, 768), (17, 768, 3072), (40, 1600, 6400), (33, 4800, 1600),
                                   (64, 100, 64), (20, 50257, 128), (1, 40, 192), (64, 2304, 768)])
@pytest.mark.parametrize("variant", ["plain_f32", "bias_gelu_bf16", "bias_resid_f32"])
def test_gemm_midm(m, n, k, variant):
    """The cluster split-K product for up to 64 rows against float32 arithmetic, and a row's
    bits do not depend on the other rows."""
    ops = _ops()
    assert ops.midm_supports(m, n, k)
    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    a = (torch.randn(m, k, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    bias = torch.randn(n, device="cuda", generator=g) * 0.2
    resid = torch.randn(m, n, device="cuda", generator=g)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ref = a.float() @ w.float().t()
    if variant == "plain_f32":
        out = torch.full((m, n), float("nan"), device="cuda")
        ops.gemm_midm(out, a, w, status=status)
        tol = 3e-4
        one = torch.zeros(1, n, device="cuda")
        ops.gemm_midm(one, a[m // 2:m // 2 + 1].contiguous(), w, status=status)
        assert torch.equal(one[0], out[m // 2])
    elif variant == "bias_gelu_bf16":
        out = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
        ops.gemm_midm(out, a, w, bias=bias, act="gelu_new", status=status)
        ref = _act("gelu_new", ref + bias)
        tol = 2e-2
    else:
        out = resid.clone()
        ops.gemm_midm(out, a, w, bias=bias, resid=out, status=status)
        ref = ref + bias + resid
        tol = 3e-4
    assert status.tolist() == [0, 0, 0, 0]
    scale = float(ref.abs().max())
    err = float((out.float() - ref).abs().max())
    assert err <= tol * max(1.0, scale), f"max |difference| {err:.3e} (scale {scale:.3g})"
