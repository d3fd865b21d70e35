"""CPU oracle for the MXFP8 hot path.  TEST INFRASTRUCTURE ONLY.

This module is the checker, never the product: only the test-suite, the smoke
check and the benchmark's CPU-baseline leg may import it.  The shipped CUDA
path never calls into it and has no CPU fallback.

Parity status: PINNED.  ``tests/golden/make_golden.py`` executes the reference's
own pure-torch functions (extracted by AST from the reference's harness files)
on CPU and stores their outputs; ``tests/test_oracle.py`` checks every function
below against those stored vectors.

Two independent restatements live here:

* a float restatement that follows the reference's torch code operation by
  operation (``quantize_ref_float``), and
* an integer restatement on raw bf16 bit patterns (``quantize_ref``) that the
  CUDA kernels mirror.  The two are cross-checked exhaustively in the tests.

Reference lines followed (paths inside the reference project):

* quantize, rceil scale rule ........ blackwell-ultra/019-mxfp8-quantize.py:31-46
                                      (same code: blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.py:43-58)
* scale layout (unswizzle) .......... blackwell-ultra/019-mxfp8-quantize.py:49-53
* scale layout (older form) ......... blackwell/047-mxfp8-mma-2cta-MNK128-polished.py:54-90
* dequantize ........................ blackwell/047-mxfp8-mma-2cta-MNK128-polished.py:36-51
* GEMM check ........................ blackwell/047-mxfp8-mma-2cta-MNK128-polished.py:138-143

Scale modes
-----------
``rceil``  the reference's rule: E = ceil(log2(amax / 448)), amax/448 clamped to
           1e-12 (an all-zero block therefore gets scale byte 88), E >= -127.
``floor``  the OCP rule named by the benchmark's first configuration:
           E = floor(log2(amax)) - 8, with E4M3 saturation live because
           amax / 2^E lies in [256, 512).  An all-zero block gets scale byte 0.
"""
from __future__ import annotations

import numpy as np
import torch

MODE_RCEIL = 0
MODE_FLOOR = 1
_MODES = {"rceil": MODE_RCEIL, "floor": MODE_FLOOR, MODE_RCEIL: MODE_RCEIL, MODE_FLOOR: MODE_FLOOR}

BLOCK = 32          # elements per scale block
TILE = 128          # rows / columns per scale-layout tile
SCALE_TILE_BYTES = 512


def _mode(mode) -> int:
    return _MODES[mode]


# --------------------------------------------------------------------------------------
# bit-level helpers
# --------------------------------------------------------------------------------------
def bf16_bits(x: torch.Tensor) -> np.ndarray:
    """bf16 tensor -> uint16 numpy array of its bit patterns."""
    assert x.dtype == torch.bfloat16
    return x.contiguous().view(torch.int16).numpy().view(np.uint16)


def bits_to_bf16(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def scale_byte_from_amax_bits(amax_bits: np.ndarray, mode) -> np.ndarray:
    """E8M0 scale byte from the bit pattern of |amax| (a non-negative bf16).

    rceil: byte = max(88, e_biased - 8 + (mant7 > 0x60)); this integer rule equals
    ceil(log2(max(amax/448, 1e-12))) + 127 for every finite bf16 amax (checked
    exhaustively in the tests against the float restatement).
    floor: byte = max(0, e_biased - 8).
    """
    a = amax_bits.astype(np.int32) & 0x7FFF
    if _mode(mode) == MODE_RCEIL:
        return np.maximum(88, ((a + 0x1F) >> 7) - 8).astype(np.uint8)
    return np.maximum(0, (a >> 7) - 8).astype(np.uint8)


def e4m3_encode(v: np.ndarray) -> np.ndarray:
    """float -> E4M3 (fn) byte, round-to-nearest-even, saturating to +-448.

    Matches ``cvt.rn.satfinite.e4m3x2.f32``; for |v| <= 448 it also matches
    torch's CPU ``.to(torch.float8_e4m3fn)`` (which the reference relies on).
    NaN input is unsupported (the hot path never produces one).
    """
    v = np.asarray(v, dtype=np.float64)
    sign = (np.signbit(v).astype(np.uint8)) << 7
    a = np.minimum(np.abs(v), 448.0)
    out = np.zeros(v.shape, dtype=np.int32)
    sub = a < 2.0 ** -6
    # subnormals: multiples of 2^-9; rint is round-half-even; 8 rolls into the first normal
    out_sub = np.rint(a * 512.0).astype(np.int32)
    m, e = np.frexp(a)                      # a = m * 2^e, m in [0.5, 1)
    e = e - 1                               # a = (2m) * 2^e, 2m in [1, 2)
    q = np.rint(m * 16.0).astype(np.int32)  # 2m * 8 in [8, 16]
    carry = q == 16
    e = np.where(carry, e + 1, e)
    q = np.where(carry, 8, q)
    out_norm = ((e + 7) << 3) | (q - 8)
    out = np.where(sub, out_sub, out_norm)
    out = np.minimum(out, 0x7E)
    return (out.astype(np.uint8) | sign).astype(np.uint8)


_E4M3_TABLE = None


def e4m3_decode_table() -> np.ndarray:
    """float32 value of each of the 256 E4M3 (fn) bytes; 0x7F/0xFF are NaN."""
    global _E4M3_TABLE
    if _E4M3_TABLE is None:
        t = np.zeros(256, dtype=np.float32)
        for b in range(256):
            s = -1.0 if b & 0x80 else 1.0
            e = (b >> 3) & 0xF
            m = b & 7
            if e == 0xF and m == 7:
                val = np.nan
            elif e == 0:
                val = s * m * 2.0 ** -9
            else:
                val = s * (1 + m / 8.0) * 2.0 ** (e - 7)
            t[b] = val
        _E4M3_TABLE = t
    return _E4M3_TABLE


# --------------------------------------------------------------------------------------
# quantize
# --------------------------------------------------------------------------------------
def quantize_ref(x: torch.Tensor, mode="rceil"):
    """bf16 [M, N] -> (fp8 bytes uint8 [M, N], scale bytes uint8 [M, N/32]).

    Integer restatement of blackwell-ultra/019-mxfp8-quantize.py:31-46 (mode
    "rceil"); "floor" is the OCP variant described in the module docstring.
    Blocks run along the last dimension.
    """
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[1] % BLOCK == 0
    M, N = x.shape
    bits = bf16_bits(x).reshape(M, N // BLOCK, BLOCK)
    amax_bits = (bits & 0x7FFF).max(axis=-1)
    sc = scale_byte_from_amax_bits(amax_bits, mode)                     # [M, N/32]
    # 2^-(sc-127) is exact in float32 for sc in [0, 254]
    inv = np.ldexp(np.float32(1.0), 127 - sc.astype(np.int32)).astype(np.float32)
    v = bf16_bits_to_f32(bits) * inv[..., None]                        # exact power-of-two scaling
    q = e4m3_encode(v).reshape(M, N)
    return torch.from_numpy(q), torch.from_numpy(sc)


def quantize_ref_float(x: torch.Tensor, mode="rceil"):
    """Same contract as quantize_ref, computed with torch float ops in the order
    the reference uses (blackwell-ultra/019-mxfp8-quantize.py:31-46).  The floor
    mode adds the clamp to +-448 that torch's CPU fp8 cast lacks."""
    M, N = x.shape
    xf = x.to(torch.float32)
    dest_max = torch.tensor(448.0, dtype=torch.float32)
    min_exp = torch.tensor(-127.0, dtype=torch.float32)
    bias = torch.tensor(127.0, dtype=torch.float32)
    block_amax = torch.amax(torch.abs(xf).view(M, N // BLOCK, BLOCK), dim=-1)
    if _mode(mode) == MODE_RCEIL:
        decode_scale = torch.clamp(block_amax / dest_max, min=1e-12)
        e = torch.clamp(torch.ceil(torch.log2(decode_scale)), min=min_exp)
    else:
        tiny = torch.tensor(2.0 ** -119, dtype=torch.float32)          # floor(log2)-8 = -127
        e = torch.clamp(torch.floor(torch.log2(torch.clamp(block_amax, min=tiny))) - 8.0, min=min_exp)
    scaled = xf / (2 ** e.repeat_interleave(BLOCK, dim=-1))
    if _mode(mode) == MODE_FLOOR:
        scaled = torch.clamp(scaled, -448.0, 448.0)
    q = scaled.to(torch.float8_e4m3fn).view(torch.uint8)
    sc = (e + bias).to(torch.uint8)
    return q, sc


# --------------------------------------------------------------------------------------
# scale-factor layout (tcgen05 "scale_vec::1X" tile layout)
# --------------------------------------------------------------------------------------
def scale_swizzle(sc: torch.Tensor) -> torch.Tensor:
    """uint8 [R, C/32] -> uint8 [R/128, C/128, 32, 16].

    Inside one 128-row x 4-block tile the byte for (row r, block kb) sits at
    offset (r % 32) * 16 + (r // 32) * 4 + kb.  Inverse of scale_unswizzle.
    Follows blackwell-ultra/019-mxfp8-quantize.py:49-53 and the kernel's store
    address at blackwell-ultra/019-mxfp8-quantize.cu:131.
    """
    R, KB = sc.shape
    assert R % TILE == 0 and KB % 4 == 0
    t = sc.view(R // TILE, 4, 32, KB // 4, 4)          # [rb, rq, r32, cb, kb]
    t = t.permute(0, 3, 2, 1, 4)                       # [rb, cb, r32, rq, kb]
    return t.reshape(R // TILE, KB // 4, 32, 16).contiguous()


def scale_unswizzle(sc: torch.Tensor) -> torch.Tensor:
    """uint8 [R/128, C/128, 32, 16] (or [.., 512]) -> uint8 [R, C/32]."""
    rb, cb = sc.shape[0], sc.shape[1]
    t = sc.reshape(rb, cb, 32, 4, 4)
    t = t.permute(0, 3, 2, 1, 4)
    return t.reshape(rb * TILE, cb * 4).contiguous()


def quantize_tiled(x: torch.Tensor, mode="rceil"):
    """bf16 [M, N] -> (fp8 uint8 [M, N], swizzled scales uint8 [M/128, N/128, 32, 16])."""
    q, sc = quantize_ref(x, mode)
    return q, scale_swizzle(sc)


def quantize_both(x: torch.Tensor, mode="rceil"):
    """The four outputs of the reference's mxfp8_quantize for a 2-D or 3-D input:
    row-wise (fp8, scales) and transposed (fp8_t [.., N, M], scales_t) with the
    transposed blocks running along the original row index
    (blackwell-ultra/019-mxfp8-quantize.py:71-74)."""
    if x.dim() == 3:
        # [E, M, N]: fp8 tensors keep the expert dimension, scale tensors stack the
        # experts' row tiles (blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.cu:404-448)
        outs = [quantize_both(x[e], mode) for e in range(x.shape[0])]
        return (torch.stack([o[0] for o in outs]), torch.cat([o[1] for o in outs]),
                torch.stack([o[2] for o in outs]), torch.cat([o[3] for o in outs]))
    q, sc = quantize_tiled(x, mode)
    qt, sct = quantize_tiled(x.t().contiguous(), mode)
    return q, sc, qt, sct


# --------------------------------------------------------------------------------------
# dequantize and GEMM
# --------------------------------------------------------------------------------------
def dequantize(q: torch.Tensor, sc_unswizzled: torch.Tensor) -> torch.Tensor:
    """fp8 bytes [R, C] + scale bytes [R, C/32] -> float32 [R, C]
    (blackwell/047-mxfp8-mma-2cta-MNK128-polished.py:36-51; exact in fp32)."""
    vals = torch.from_numpy(e4m3_decode_table())[q.to(torch.int64)]
    scale = torch.from_numpy(np.ldexp(np.float32(1.0), sc_unswizzled.numpy().astype(np.int32) - 127).astype(np.float32))
    return vals * scale.repeat_interleave(BLOCK, dim=-1)


def gemm_ref(a_q, a_sc_swz, b_q, b_sc_swz, out_dtype=torch.bfloat16) -> torch.Tensor:
    """C = dequant(A) . dequant(B)^T, fp32 accumulate, rounded to out_dtype
    (blackwell/047-mxfp8-mma-2cta-MNK128-polished.py:138-143).
    A: fp8 bytes [M, K]; B: fp8 bytes [N, K]; scales in the swizzled tile layout."""
    a = dequantize(a_q, scale_unswizzle(a_sc_swz))
    b = dequantize(b_q, scale_unswizzle(b_sc_swz))
    return torch.matmul(a, b.t()).to(out_dtype)


def rel_frobenius(c: torch.Tensor, ref: torch.Tensor) -> float:
    c = c.to(torch.float64)
    ref = ref.to(torch.float64)
    return float(torch.linalg.norm(c - ref) / torch.linalg.norm(ref).clamp_min(1e-300))


# --------------------------------------------------------------------------------------
# seeded synthetic inputs shared by tests, smoke and bench (identical bits on every box)
# --------------------------------------------------------------------------------------
def make_input(M: int, N: int, seed: int, std: float = 1.0, outliers: bool = False,
               zero_blocks: bool = False) -> torch.Tensor:
    """bf16 [M, N] ~ N(0, std).  outliers: 0.1 % of entries multiplied by 1000.
    zero_blocks: the first 1x32 block of every 1024-row band set to zero."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, N, generator=g, dtype=torch.float32) * std
    if outliers:
        mask = torch.rand(M, N, generator=g) < 1e-3
        x = torch.where(mask, x * 1000.0, x)
    x = x.to(torch.bfloat16)
    if zero_blocks:
        x[0::1024, 0:BLOCK] = 0
    return x
