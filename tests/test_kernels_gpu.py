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
               (257, 808, 1608), (2048, 768, 3072), (7, 50257, 768)]


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


@pytest.mark.parametrize("tile_n", [32, 64, 128, 256])
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
