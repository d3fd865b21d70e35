"""Shared (bf16) expert: the kind::f16 form of the GEMM kernel, SwiGLU forward / backward and the
transposes, against fp32 torch references on the CPU (tolerance: relative Frobenius error 1e-2 for the
GEMMs, whose fp32 accumulation order differs from the CPU's; 2 bf16 ulps for the element-wise kernels,
which use the fast exponential and reciprocal)."""
import pytest
import torch

import mx8
from oracle import moe_oracle as MO
from oracle import mx8_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rand_bf16(rows, cols, seed, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(rows, cols, generator=g) * std).to(torch.bfloat16)


def ulp_diff(a, b):
    """distance in bf16 representable steps between two bf16 tensors (same sign assumed near zero)"""
    ia = a.view(torch.int16).to(torch.int32)
    ib = b.view(torch.int16).to(torch.int32)
    key = lambda i: torch.where(i < 0, -(i & 0x7FFF), i)
    return (key(ia) - key(ib)).abs()


@pytest.mark.parametrize("shape", [(128, 128, 64), (256, 256, 128), (384, 640, 1024), (128, 384, 192), (1024, 512, 448)])
@pytest.mark.parametrize("c_dtype", [torch.bfloat16, torch.float32])
def test_gemm_bf16(shape, c_dtype):
    M, N, K = shape
    a, b = rand_bf16(M, K, 1, K ** -0.5), rand_bf16(N, K, 2)
    c = torch.full((M, N), float("nan"), dtype=c_dtype, device=DEV)
    mx8.gemm_bf16(a.to(DEV), b.to(DEV), c)
    assert mx8.device_status() == 0
    ref = a.float() @ b.float().t()
    assert O.rel_frobenius(c.cpu().float(), ref) < (1e-5 if c_dtype == torch.float32 else 4e-3)


def test_gemm_bf16_dual_accumulates_both_products():
    M, N, K1, K2 = 256, 384, 256, 128
    a1, b1, a2, b2 = rand_bf16(M, K1, 1, 0.1), rand_bf16(N, K1, 2), rand_bf16(M, K2, 3, 0.1), rand_bf16(N, K2, 4)
    c = torch.empty(M, N, dtype=torch.float32, device=DEV)
    mx8.gemm_bf16(a1.to(DEV), b1.to(DEV), c, a2.to(DEV), b2.to(DEV))
    assert mx8.device_status() == 0
    ref = a1.float() @ b1.float().t() + a2.float() @ b2.float().t()
    assert O.rel_frobenius(c.cpu(), ref) < 1e-5


def test_gemm_bf16_matches_library_at_size():
    M, N, K = 4096, 2048, 7168
    a, b = rand_bf16(M, K, 5, K ** -0.5).to(DEV), rand_bf16(N, K, 6).to(DEV)
    c = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    mx8.gemm_bf16(a, b, c)
    assert mx8.device_status() == 0
    lib = a @ b.t()
    assert O.rel_frobenius(c.float().cpu(), lib.float().cpu()) < 4e-3


def test_swiglu_forward_backward():
    g, u, dh = rand_bf16(256, 512, 1, 2.0), rand_bf16(256, 512, 2), rand_bf16(256, 512, 3)
    h = mx8.swiglu_bf16(g.to(DEV), u.to(DEV)).cpu()
    gf = g.float()
    den = torch.exp(-gf) + 1.0
    silu = gf / den
    want = (silu * u.float()).to(torch.bfloat16)
    assert int(ulp_diff(h, want).max()) <= 2
    dg, du = mx8.swiglu_bwd_bf16(dh.to(DEV), g.to(DEV), u.to(DEV))
    d_silu = (1.0 - silu) / den + silu
    want_g = ((dh.float() * d_silu) * u.float()).to(torch.bfloat16)
    want_u = (silu * dh.float()).to(torch.bfloat16)
    # values that cancel to nearly zero can be many ulps apart while tiny in absolute terms
    for got, want_t in ((dg.cpu(), want_g), (du.cpu(), want_u)):
        close = (ulp_diff(got, want_t) <= 2) | ((got.float() - want_t.float()).abs() <= 1e-3 * want_t.float().abs().max())
        assert bool(close.all())


@pytest.mark.parametrize("shape", [(64, 64), (128, 320), (1024, 192)])
def test_transpose(shape):
    x = rand_bf16(*shape, seed=9)
    got = mx8.transpose_bf16(x.to(DEV)).cpu()
    assert torch.equal(got.view(torch.int16), x.t().contiguous().view(torch.int16))


def test_shared_expert_forward_backward_against_oracle():
    T, H, I = 256, 512, 384
    x = rand_bf16(T, H, 1)
    wg, wu, wd = rand_bf16(I, H, 2, 0.05), rand_bf16(I, H, 3, 0.05), rand_bf16(H, I, 4, 0.05)
    d_y = rand_bf16(T, H, 5)
    gate, up, hidden, y = MO.shared_mlp_ref(x, wg, wu, wd)
    bf = lambda r, c: torch.empty(r, c, dtype=torch.bfloat16, device=DEV)
    xd = x.to(DEV)
    g_d = mx8.gemm_bf16(xd, wg.to(DEV), bf(T, I))
    u_d = mx8.gemm_bf16(xd, wu.to(DEV), bf(T, I))
    h_d = mx8.swiglu_bf16(g_d, u_d)
    y_d = mx8.gemm_bf16(h_d, wd.to(DEV), bf(T, H))
    for got, want in ((g_d, gate), (u_d, up), (h_d, hidden), (y_d, y)):
        assert O.rel_frobenius(got.cpu().float(), want.float()) < 1e-2
    # backward on the oracle's forward tensors, so that every stage is compared on identical inputs
    ref = MO.shared_mlp_bwd_ref(d_y, x, gate, up, hidden, wg, wu, wd)
    dyd = d_y.to(DEV)
    d_h = mx8.gemm_bf16(dyd, wd.t().contiguous().to(DEV), bf(T, I))
    d_g, d_u = mx8.swiglu_bwd_bf16(ref[3].to(DEV), gate.to(DEV), up.to(DEV))
    d_x = mx8.gemm_bf16(ref[1].to(DEV), wg.t().contiguous().to(DEV), bf(T, H), ref[2].to(DEV), wu.t().contiguous().to(DEV))
    x_t = mx8.transpose_bf16(xd)
    dwg = mx8.gemm_bf16(mx8.transpose_bf16(ref[1].to(DEV)), x_t, bf(I, H))
    dwu = mx8.gemm_bf16(mx8.transpose_bf16(ref[2].to(DEV)), x_t, bf(I, H))
    dwd = mx8.gemm_bf16(mx8.transpose_bf16(dyd), mx8.transpose_bf16(hidden.to(DEV)), bf(H, I))
    assert mx8.device_status() == 0
    for name, got, want in (("d_hidden", d_h, ref[3]), ("d_gate", d_g, ref[1]), ("d_up", d_u, ref[2]), ("d_x", d_x, ref[0]),
                            ("d_w_gate", dwg, ref[4]), ("d_w_up", dwu, ref[5]), ("d_w_down", dwd, ref[6])):
        assert O.rel_frobenius(got.cpu().float(), want.float()) < 1e-2, name
