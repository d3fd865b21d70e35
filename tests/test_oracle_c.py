"""The C restatement of the oracle against the golden vectors and the Python oracle."""
import ctypes
import os
import subprocess

import numpy as np
import pytest
import torch

from oracle import mx8_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
u8p = ctypes.POINTER(ctypes.c_uint8)
u16p = ctypes.POINTER(ctypes.c_uint16)


@pytest.fixture(scope="module")
def clib():
    so = os.path.join(ROOT, "oracle", "libmx8_oracle.so")
    if not os.path.exists(so):
        subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "oracle")])
    lib = ctypes.CDLL(so)
    lib.mx8o_scale_byte.restype = ctypes.c_uint8
    lib.mx8o_scale_byte.argtypes = [ctypes.c_uint16, ctypes.c_int]
    lib.mx8o_e4m3_encode.restype = ctypes.c_uint8
    lib.mx8o_e4m3_encode.argtypes = [ctypes.c_float]
    lib.mx8o_e4m3_decode.restype = ctypes.c_float
    lib.mx8o_e4m3_decode.argtypes = [ctypes.c_uint8]
    lib.mx8o_quantize_both.restype = ctypes.c_int
    lib.mx8o_gemm.restype = ctypes.c_int
    return lib


def p8(a):
    return a.ctypes.data_as(u8p)


def c_quantize_both(lib, x_bits, mode):
    M, N = x_bits.shape
    q = np.empty((M, N), np.uint8)
    sc = np.empty((M // 128, N // 128, 512), np.uint8)
    qt = np.empty((N, M), np.uint8)
    sct = np.empty((N // 128, M // 128, 512), np.uint8)
    x = np.ascontiguousarray(x_bits)
    rc = lib.mx8o_quantize_both(x.ctypes.data_as(u16p), M, N, mode, p8(q), p8(sc), p8(qt), p8(sct))
    assert rc == 0
    return q, sc, qt, sct


def test_c_quantize_matches_reference_vectors(clib, golden_dir):
    g = np.load(os.path.join(golden_dir, "quantize_256x384.npz"))
    q, sc, qt, sct = c_quantize_both(clib, g["x_bits"], 0)
    assert np.array_equal(q, g["fp8"]) and np.array_equal(qt, g["fp8_t"])
    assert np.array_equal(O.scale_unswizzle(torch.from_numpy(sc)).numpy(), g["sc"])
    assert np.array_equal(O.scale_unswizzle(torch.from_numpy(sct)).numpy(), g["sc_t"])


def test_c_scale_rule_and_codec_exhaustive(clib, golden_dir):
    g = np.load(os.path.join(golden_dir, "scale_all_amax.npz"))
    got = np.array([clib.mx8o_scale_byte(int(a), 0) for a in g["amax_bits"]], np.uint8)
    assert np.array_equal(got, g["sc"])
    tab = O.e4m3_decode_table()
    for b in range(256):
        v = clib.mx8o_e4m3_decode(b)
        if (b & 0x7F) == 0x7F:
            assert np.isnan(v)
        else:
            assert v == tab[b] and clib.mx8o_e4m3_encode(v) == b
    vals = np.concatenate([np.linspace(-500, 500, 4001), np.array([0.0, -0.0, 2.0 ** -10, 3 * 2.0 ** -10, 2.0 ** -9, 1e-8])]).astype(np.float32)
    want = O.e4m3_encode(vals)
    assert np.array_equal(np.array([clib.mx8o_e4m3_encode(float(v)) for v in vals], np.uint8), want)


@pytest.mark.parametrize("mode", [0, 1])
def test_c_and_python_oracles_agree(clib, mode):
    x = O.make_input(256, 256, seed=17, outliers=True, zero_blocks=True)
    got = c_quantize_both(clib, O.bf16_bits(x), mode)
    want = O.quantize_both(x, mode)
    for g, w in zip(got, want):
        assert np.array_equal(g.reshape(-1), w.numpy().reshape(-1))


def test_c_gemm_matches_reference_vectors(clib, golden_dir):
    g = np.load(os.path.join(golden_dir, "gemm_256x384x512.npz"))
    M, N, K = 256, 384, 512
    c = np.empty((M, N), np.uint16)
    rc = clib.mx8o_gemm(p8(np.ascontiguousarray(g["a_fp8"])), p8(np.ascontiguousarray(g["a_sc"])),
                        p8(np.ascontiguousarray(g["b_fp8"])), p8(np.ascontiguousarray(g["b_sc"])), M, N, K,
                        c.ctypes.data_as(u16p), None)
    assert rc == 0
    ref = O.bits_to_bf16(g["c_bits"])
    assert O.rel_frobenius(O.bits_to_bf16(c), ref) < 1e-3
