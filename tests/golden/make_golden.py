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
    blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.py
                                              mxfp8_quantize_ref, scale_unswizzle, dequant, quant_and_dequant,
                                              mlp_swiglu_fwd_ref, mlp_swiglu_bwd_ref

The MoE functions call the harness's mxfp8_gemm_ref, which wraps torch._scaled_mm with block scales and
needs a GPU.  Here that one name is bound to a CPU stand-in of the same contract (operands given as
(fp8, scales) or quantized on the fly by the reference's mxfp8_quantize_ref, scales unswizzled or in
128 x 4 tiles; result = fp32 product of the dequantized operands, rounded to the output type), so the
fixture pins everything the reference's functions do around the GEMMs — the order of the steps, what
is rounded to bf16 and where, which operand is quantized along which axis — and the GEMM itself is
pinned separately by gemm_256x384x512.npz.

The test-suite only reads the stored .npz files; it never needs the reference.
"""
import ast
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def extract(path, names, extra=None):
    src = open(path).read()
    tree = ast.parse(src)
    ns = {"torch": torch, "np": np}
    ns.update(extra or {})
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
    moe_fixture(ref_root)
    print("golden vectors written to", HERE)


def moe_fixture(ref_root):
    """Routed + shared expert MLP, forward and backward, through the reference's own torch functions."""
    path = os.path.join(ref_root, "blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.py")
    ns = extract(path, ["mxfp8_quantize_ref", "scale_unswizzle", "dequant", "quant_and_dequant"])

    def mxfp8_gemm_ref(x, w, out_dtype=torch.bfloat16):
        def operand(o):
            fp8, sc = o if isinstance(o, tuple) else ns["mxfp8_quantize_ref"](o)
            if sc.dim() != 2:
                sc = ns["scale_unswizzle"](sc)
            rows, K = fp8.shape
            return (fp8.float().reshape(rows, K // 32, 32) * (2.0 ** (sc.float() - 127.0)).unsqueeze(-1)).reshape(rows, K)
        return (operand(x) @ operand(w).t()).to(out_dtype)

    ns = extract(path, ["mxfp8_quantize_ref", "scale_unswizzle", "dequant", "quant_and_dequant", "mlp_swiglu_fwd_ref",
                        "mlp_swiglu_bwd_ref"], extra={"mxfp8_gemm_ref": mxfp8_gemm_ref})
    quant = ns["mxfp8_quantize_ref"]

    def quant_tiles(w):
        """[E, R, C] bf16 -> (fp8 [E, R, C], scale tiles [E*R/128, C/128, 32, 16]) as the reference's quantize kernel
        lays them out; the tile permutation is the one its mxfp8_gemm_ref applies to unswizzled scales."""
        E, R, C = w.shape
        fp8, sc = zip(*(quant(w[e]) for e in range(E)))
        sc = torch.stack(sc).reshape(E * R, C // 32)
        sc = sc.view(E * R // 128, 4, 32, C // 128, 4).permute(0, 3, 2, 1, 4).contiguous().view(E * R // 128, C // 128, 32, 16)
        return torch.stack(fp8), sc

    E, H, I, Ts, Is = 2, 256, 256, 32, 64             # the grouped GEMM wants whole 256-column tiles
    tokens_per_expert = torch.tensor([256, 256], dtype=torch.int32)
    valid_rows = [96, 40]                                       # the rest of every segment is padding: zero rows
    R = int(tokens_per_expert.sum())
    g = torch.Generator().manual_seed(2022)
    rn = lambda *shape: torch.randn(*shape, generator=g)
    x_routed = rn(R, H).to(torch.bfloat16)
    d_y_routed = (rn(R, H) * H ** -0.5).to(torch.bfloat16)
    off = 0
    for n, v in zip(tokens_per_expert.tolist(), valid_rows):
        x_routed[off + v:off + n] = 0
        d_y_routed[off + v:off + n] = 0
        off += n
    w_gate = (rn(E, I, H) * H ** -0.5).to(torch.bfloat16)
    w_up = (rn(E, I, H) * H ** -0.5).to(torch.bfloat16)
    w_down = (rn(E, H, I) * I ** -0.5).to(torch.bfloat16)
    x_shared = rn(Ts, H).to(torch.bfloat16)
    d_y_shared = (rn(Ts, H) * H ** -0.5).to(torch.bfloat16)
    ws_gate = (rn(Is, H) * H ** -0.5).to(torch.bfloat16)
    ws_up = (rn(Is, H) * H ** -0.5).to(torch.bfloat16)
    ws_down = (rn(H, Is) * Is ** -0.5).to(torch.bfloat16)
    wq = {n: quant_tiles(w) for n, w in (("gate", w_gate), ("up", w_up), ("down", w_down))}
    wq_T = {n: quant_tiles(w.transpose(-2, -1).contiguous()) for n, w in (("gate", w_gate), ("up", w_up), ("down", w_down))}

    fwd_names = ["gate_shared", "gate_routed", "up_shared", "up_routed", "hidden_shared", "hidden_routed", "y_shared", "y_routed"]
    fwd = dict(zip(fwd_names, ns["mlp_swiglu_fwd_ref"](x_shared, x_routed, ws_gate, wq["gate"], ws_up, wq["up"], ws_down, wq["down"],
                                                        tokens_per_expert)))
    bwd_names = ["d_x_shared", "d_x_routed", "d_gate_shared", "d_gate_routed", "d_up_shared", "d_up_routed", "d_hidden_shared",
                 "d_hidden_routed", "d_w_shared_gate", "d_w_routed_gate", "d_w_shared_up", "d_w_routed_up", "d_w_shared_down",
                 "d_w_routed_down"]
    bwd = dict(zip(bwd_names, ns["mlp_swiglu_bwd_ref"](
        d_y_shared, d_y_routed, x_shared, x_routed, fwd["gate_shared"], fwd["gate_routed"], fwd["up_shared"], fwd["up_routed"],
        fwd["hidden_shared"], fwd["hidden_routed"], ws_gate, wq_T["gate"], ws_up, wq_T["up"], ws_down, wq_T["down"], tokens_per_expert)))
    out = dict(tokens_per_expert=tokens_per_expert.numpy(), valid_rows=np.array(valid_rows, np.int32),
               x_routed=bf16_bits(x_routed), d_y_routed=bf16_bits(d_y_routed), x_shared=bf16_bits(x_shared),
               d_y_shared=bf16_bits(d_y_shared), w_shared_gate=bf16_bits(ws_gate), w_shared_up=bf16_bits(ws_up),
               w_shared_down=bf16_bits(ws_down))
    for n in ("gate", "up", "down"):
        out["w_%s_fp8" % n], out["w_%s_sc" % n] = u8(wq[n][0]), wq[n][1].numpy()
        out["w_%s_T_fp8" % n], out["w_%s_T_sc" % n] = u8(wq_T[n][0]), wq_T[n][1].numpy()
    for d in (fwd, bwd):
        for n, t in d.items():
            out[n] = bf16_bits(t)
    np.savez_compressed(os.path.join(HERE, "moe_fwd_bwd.npz"), **out)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
