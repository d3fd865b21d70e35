"""Host-buffer entry points (banded copy-in / kernel / copy-out pipeline): same bytes as the oracle
and as the device-resident entry points, including a ragged last band and reuse of the workspace."""
import pytest
import torch

import mx8
from oracle import mx8_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def host_outputs(M, N):
    mk = lambda *s: torch.full(s, 0xFF, dtype=torch.uint8).pin_memory()
    return mk(M, N), mk(M // 128, N // 128, 32, 16), mk(N, M), mk(N // 128, M // 128, 32, 16)


@pytest.mark.parametrize("mode", ["rceil", "floor"])
@pytest.mark.parametrize("shape,band", [((640, 384), 256), ((256, 256), 2048), ((1152, 512), 128), ((2304, 256), 512)])
def test_quantize_host_matches_oracle(shape, band, mode):
    M, N = shape
    x = O.make_input(M, N, seed=M + N, outliers=True, zero_blocks=True).pin_memory()
    outs = host_outputs(M, N)
    ws = mx8.mxfp8_quantize_host(x, *outs, True, True, band_rows=band, device=DEV, scale_mode=mode)
    assert mx8.device_status() == 0
    want = O.quantize_both(x, mode)
    for name, g, w in zip(("fp8", "sc", "fp8_t", "sc_t"), outs, want):
        assert int((g != w).sum()) == 0, name
    # second call reusing the workspace, one orientation only: the other pair stays untouched
    outs2 = host_outputs(M, N)
    mx8.mxfp8_quantize_host(x, outs2[0], outs2[1], None, None, True, False, band_rows=band, workspace=ws, device=DEV,
                            scale_mode=mode)
    assert mx8.device_status() == 0
    assert torch.equal(outs2[0], want[0]) and torch.equal(outs2[1], want[1])
    assert bool((outs2[2] == 0xFF).all()) and bool((outs2[3] == 0xFF).all())


def test_quantize_host_argument_errors():
    x = torch.zeros(256, 256, dtype=torch.bfloat16).pin_memory()
    outs = host_outputs(256, 256)
    with pytest.raises(mx8.Mx8Error):
        mx8.mxfp8_quantize_host(x, *outs, True, True, band_rows=100, device=DEV)       # not a multiple of 128
    small = torch.empty(1024, dtype=torch.uint8, device=DEV)
    with pytest.raises(ValueError):
        mx8.mxfp8_quantize_host(x, *outs, True, True, band_rows=128, workspace=small, device=DEV)
    lib = mx8.load()
    rc = lib.mx8_quantize_host(x.data_ptr(), 256, 256, outs[0].data_ptr(), outs[1].data_ptr(), None, None, 0, 128,
                               small.data_ptr(), 1024, None)
    assert rc == 7                                                                      # MX8_ERR_LIMIT


@pytest.mark.parametrize("c_dtype", [torch.bfloat16, torch.float32])
def test_gemm_host_matches_device_path(c_dtype):
    M, N, K, band = 640, 384, 512, 256
    g = torch.Generator().manual_seed(5)
    a = (torch.randn(M, K, generator=g) * K ** -0.5).to(torch.bfloat16)
    b = (torch.randn(N, K, generator=g) * K ** -0.5).to(torch.bfloat16)
    aq, asc, _, _ = mx8.mxfp8_quantize(a.to(DEV), True, False)
    bq, bsc, _, _ = mx8.mxfp8_quantize(b.to(DEV), True, False)
    c_dev = torch.empty(M, N, dtype=c_dtype, device=DEV)
    mx8.kernel(aq, asc, bq, bsc, c_dev)
    host = [t.cpu().pin_memory() for t in (aq.view(torch.uint8), asc, bq.view(torch.uint8), bsc)]
    c_h = torch.full((M, N), float("nan"), dtype=c_dtype).pin_memory()
    mx8.kernel_host(host[0], host[1], host[2], host[3], c_h, band_rows=band, device=DEV)
    assert mx8.device_status() == 0
    assert torch.equal(c_h, c_dev.cpu())
    ref = O.gemm_ref(host[0], host[1], host[2], host[3], out_dtype=c_dtype)
    assert O.rel_frobenius(c_h.float(), ref.float()) < 1e-2
