"""Generate the golden vectors in this directory from the reference's own code.

Run once, in a checkout that has the reference project next to it:

    python tests/golden/make_golden.py /path/to/reference

The reference's harness files cannot be imported (they import a compiled CUDA
module and run GPU code at import time), so this script parses them, pulls out
the pure-torch functions by name, executes exactly that source on CPU and
stores inputs and outputs.  The functions taken are

    blackwell-ultra/019-mxfp8-quantize.py     mxfp8_quantize_ref, scale_unswizzle
    blackwell/047-mxfp8-mma-2cta-MNK128-polished.py
                                              quantize_2d, dequantize_2d, reshape_sc

The test-suite only reads the stored .npz files; it never needs the reference.
"""
import ast
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def extract(path, names):
    src = open(path).read()
    tree = ast.parse(src)
    ns = {"torch": torch, "np": np}
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in names:
            code = compile(ast.Module(body=[node], type_ignores=[]), path, "exec")
            exec(code, ns)
    missing = [n for n in names if n not in ns]
    assert not missing, missing
    return ns


def u8(t):
    return t.view(torch.uint8).numpy() if t.dtype != torch.uint8 else t.numpy()


def bf16_bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def main(ref_root):
    q19 = extract(os.path.join(ref_root, "blackwell-ultra/019-mxfp8-quantize.py"),
                  ["mxfp8_quantize_ref", "scale_unswizzle"])
    g47 = extract(os.path.join(ref_root, "blackwell/047-mxfp8-mma-2cta-MNK128-polished.py"),
                  ["quantize_2d", "dequantize_2d", "reshape_sc"])

    # ---- 1. quantize on a 256 x 384 matrix with outliers, an all-zero block, signed zeros,
    #         boundary mantissas and the largest finite bf16 --------------------------------
    g = torch.Generator().manual_seed(1234)
    x = torch.randn(256, 384, generator=g)
    mask = torch.rand(256, 384, generator=g) < 1e-3
    x = torch.where(mask, x * 1000.0, x).to(torch.bfloat16)
    x[0, 0:32] = 0                                   # all-zero block
    x[1, 0:32] = 0
    x[1, 5] = -0.0                                   # zero block holding a negative zero
    xb = bf16_bits(x).copy()
    xb[2, 0:32] = 0x0001                             # smallest subnormal everywhere
    xb[3, 0:32] = 0x3F80                             # 1.0
    xb[3, 7] = 0x7F7F                                # largest finite bf16
    for i, m in enumerate([0x5F, 0x60, 0x61, 0x7F, 0x00]):   # mantissa boundary of the ceil rule
        xb[4 + i, 32:64] = 0x3C00
        xb[4 + i, 40] = 0x4000 | m
    x = torch.from_numpy(xb.view(np.int16)).view(torch.bfloat16)

    fp8, sc = q19["mxfp8_quantize_ref"](x)
    fp8_t, sc_t = q19["mxfp8_quantize_ref"](x.t().contiguous())
    np.savez_compressed(os.path.join(HERE, "quantize_256x384.npz"),
                        x_bits=bf16_bits(x), fp8=u8(fp8), sc=u8(sc), fp8_t=u8(fp8_t), sc_t=u8(sc_t))

    # ---- 2. scale byte for every finite positive bf16 amax (one block each) ----------------
    amax_bits = np.arange(0, 0x7F80, dtype=np.uint16)
    blk = np.zeros((amax_bits.size, 32), dtype=np.uint16)
    blk[:, 3] = amax_bits
    xa = torch.from_numpy(blk.view(np.int16)).view(torch.bfloat16)
    fp8a, sca = q19["mxfp8_quantize_ref"](xa)
    np.savez_compressed(os.path.join(HERE, "scale_all_amax.npz"),
                        amax_bits=amax_bits, sc=u8(sca)[:, 0], fp8_at_amax=u8(fp8a)[:, 3])

    # ---- 3. scale layout: the reference's unswizzle of a counting pattern, and the older
    #         reshape_sc of the same scales ----------------------------------------------------
    swz = torch.arange(2 * 3 * 512, dtype=torch.int64).remainder(251).to(torch.uint8).view(2, 3, 32, 16)
    unswz = q19["scale_unswizzle"](swz)                         # [256, 12]
    older = g47["reshape_sc"](unswz.t().contiguous())           # takes (k_blocks, m)
    np.savez_compressed(os.path.join(HERE, "scale_layout.npz"),
                        swizzled=swz.numpy(), unswizzled=unswz.numpy(), reshape_sc=older.numpy())

    # ---- 4. GEMM: operands quantized by the reference's quantize_2d, expected product from
    #         its dequantize_2d + fp32 matmul -> bf16 ------------------------------------------
    torch.manual_seed(42)
    M, N, K = 256, 384, 512
    A = torch.randn(M, K, dtype=torch.float32) / K ** 0.25
    B = torch.randn(N, K, dtype=torch.float32) / K ** 0.25
    # quantize_2d takes fp32; round through bf16 first so the same bits can be fed to the new quantizer
    A = A.to(torch.bfloat16).to(torch.float32)
    B = B.to(torch.bfloat16).to(torch.float32)
    A_fp8, A_sc_kmajor = g47["quantize_2d"](A)
    B_fp8, B_sc_kmajor = g47["quantize_2d"](B)
    A_deq = g47["dequantize_2d"](A_fp8, A_sc_kmajor)
    B_deq = g47["dequantize_2d"](B_fp8, B_sc_kmajor)
    C = torch.matmul(A_deq, B_deq.T).to(torch.bfloat16)
    np.savez_compressed(os.path.join(HERE, "gemm_256x384x512.npz"),
                        a_bits=bf16_bits(A.to(torch.bfloat16)), b_bits=bf16_bits(B.to(torch.bfloat16)),
                        a_fp8=u8(A_fp8), b_fp8=u8(B_fp8),
                        a_sc=g47["reshape_sc"](A_sc_kmajor).numpy(), b_sc=g47["reshape_sc"](B_sc_kmajor).numpy(),
                        c_bits=bf16_bits(C))
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
