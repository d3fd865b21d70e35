"""Bit-exact parity of the CUDA quantizer (through the C ABI) with the CPU oracle."""
import os

import numpy as np
import pytest
import torch

import mx8
from oracle import mx8_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def run_quant(x_cpu, rn=True, rt=True, mode="rceil"):
    """Poison-filled outputs so unwritten bytes are caught; returns CPU uint8 tensors."""
    x = x_cpu.to(DEV)
    E = x.shape[0] if x.dim() == 3 else 1
    M, N = x.shape[-2:]
    lead = (E,) if x.dim() == 3 else ()
    fp8 = torch.full(lead + (M, N), 0xFF, dtype=torch.uint8, device=DEV)
    sc = torch.full((E * M // 128, N // 128, 32, 16), 0xFF, dtype=torch.uint8, device=DEV)
    fp8_t = torch.full(lead + (N, M), 0xFF, dtype=torch.uint8, device=DEV)
    sc_t = torch.full((E * N // 128, M // 128, 32, 16), 0xFF, dtype=torch.uint8, device=DEV)
    mx8.mxfp8_quantize(x, fp8, sc, fp8_t, sc_t, rn, rt, scale_mode=mode)
    assert mx8.device_status() == 0
    return fp8.cpu(), sc.cpu(), fp8_t.cpu(), sc_t.cpu()


def check(x_cpu, rn=True, rt=True, mode="rceil"):
    got = run_quant(x_cpu, rn, rt, mode)
    want = O.quantize_both(x_cpu, mode)
    names = ["fp8", "sc", "fp8_t", "sc_t"]
    for i, (g, w) in enumerate(zip(got, want)):
        requested = rn if i < 2 else rt
        if requested:
            bad = int((g != w).sum())
            assert bad == 0, f"{names[i]}: {bad} mismatching bytes of {w.numel()} (mode {mode})"
        else:
            assert bool((g == 0xFF).all()), f"{names[i]} was written although not requested"


def test_golden_vectors(golden_dir):
    g = np.load(os.path.join(golden_dir, "quantize_256x384.npz"))
    x = O.bits_to_bf16(g["x_bits"])
    fp8, sc, fp8_t, sc_t = run_quant(x)
    assert np.array_equal(fp8.numpy(), g["fp8"])
    assert np.array_equal(O.scale_unswizzle(sc).numpy(), g["sc"])
    assert np.array_equal(fp8_t.numpy(), g["fp8_t"])
    assert np.array_equal(O.scale_unswizzle(sc_t).numpy(), g["sc_t"])


@pytest.mark.parametrize("mode", ["rceil", "floor"])
@pytest.mark.parametrize("shape", [(128, 128), (128, 384), (640, 256), (1024, 1024)])
def test_parity_shapes(shape, mode):
    check(O.make_input(*shape, seed=shape[0] + shape[1], outliers=True, zero_blocks=True), mode=mode)


@pytest.mark.parametrize("rn,rt", [(True, False), (False, True)])
def test_single_orientation(rn, rt):
    check(O.make_input(384, 512, seed=5, outliers=True), rn, rt)


def test_expert_batched_3d():
    x = torch.stack([O.make_input(256, 384, seed=s, outliers=True) for s in range(3)])
    check(x)


def test_all_bf16_bit_patterns():
    # every finite bf16 bit pattern appears; each 32-block mixes magnitudes from one binade window
    bits = np.arange(1 << 16, dtype=np.uint16)
    finite = bits[(bits & 0x7F80) != 0x7F80]
    rng = np.random.default_rng(0)
    pad = (-finite.size) % (128 * 128)
    allb = np.concatenate([finite, rng.choice(finite, pad)])
    x = O.bits_to_bf16(np.sort(allb).reshape(-1, 128))      # sorted: neighbours share a binade
    assert x.shape[0] % 128 == 0
    check(x)
    check(x, mode="floor")
    xs = O.bits_to_bf16(rng.permutation(allb).reshape(-1, 128))   # shuffled: huge dynamic range per block
    check(xs)


def test_scale_rule_every_amax(golden_dir):
    g = np.load(os.path.join(golden_dir, "scale_all_amax.npz"))
    n = g["amax_bits"].size                                    # 32640 blocks, one per amax value
    rows = (n * 32 + 127) // 128
    rows += (-rows) % 128
    flat = np.zeros(rows * 128, dtype=np.uint16)
    flat[3:n * 32:32] = g["amax_bits"]
    x = O.bits_to_bf16(flat.reshape(rows, 128))
    fp8, sc, _, _ = run_quant(x, True, False)
    un = O.scale_unswizzle(sc).reshape(-1).numpy()[:n]
    assert np.array_equal(un, g["sc"])
    assert np.array_equal(fp8.reshape(-1).numpy()[3:n * 32:32], g["fp8_at_amax"])


def test_deterministic_and_idempotent_layout():
    x = O.make_input(512, 768, seed=9, outliers=True)
    a = run_quant(x)
    b = run_quant(x)
    for u, v in zip(a, b):
        assert torch.equal(u, v)
    # the transposed outputs equal the normal outputs of the transposed input
    c = run_quant(x.t().contiguous())
    assert torch.equal(a[2], c[0]) and torch.equal(a[3], c[1])


def test_full_size_properties():
    # benchmark-sized input (16384 x 16384 with outliers and zero blocks), checked against the
    # oracle on row bands and through transpose consistency
    M = N = 16384
    x = O.make_input(M, N, seed=1234, outliers=True, zero_blocks=True)
    xd = x.to(DEV)
    fp8, sc, fp8_t, sc_t = mx8.mxfp8_quantize(xd, True, True)
    assert mx8.device_status() == 0
    for r0 in (0, 8192 - 128, M - 256):
        band = x[r0:r0 + 256]
        q, s, qt, st = O.quantize_both(band)
        assert torch.equal(fp8[r0:r0 + 256].view(torch.uint8).cpu(), q)
        assert torch.equal(sc[r0 // 128:r0 // 128 + 2].cpu(), s)
        assert torch.equal(fp8_t[:, r0:r0 + 256].view(torch.uint8).cpu(), qt)
        assert torch.equal(sc_t[:, r0 // 128:r0 // 128 + 2].cpu(), st)
    # zero blocks: scale byte 88, payload zero
    un = O.scale_unswizzle(sc[:8].cpu())
    assert un[0, 0] == 88 and not fp8[0, :32].view(torch.uint8).any()
    # checksum of the transposed bytes against the normal bytes of the transposed input
    fp8_b, sc_b, _, _ = mx8.mxfp8_quantize(xd.t().contiguous(), True, False)
    assert torch.equal(fp8_b.view(torch.uint8), fp8_t.view(torch.uint8)) and torch.equal(sc_b, sc_t)


def test_shape_errors_raise():
    x = torch.zeros(100, 128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(mx8.Mx8Error):
        mx8.mxfp8_quantize(x, True, False)
