"""Parity at the shapes the benchmark configurations name (the other GPU tests use small shapes):
the full 16384 x 16384 quantize against the C oracle, the FFN chain with K and N = 28672, and the MoE layer at
hidden 7168 / intermediate 2048 with 256 expert groups in one call.  Operands that would take minutes to
produce on the host are drawn and quantized on the GPU (the quantizer is checked bit for bit elsewhere and,
in full, by the first test here); the oracle then works on the bytes the GPU path actually consumed."""
import concurrent.futures
import ctypes
import os
import subprocess

import numpy as np
import pytest
import torch

import mx8
from oracle import moe_oracle as MO
from oracle import mx8_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# relative Frobenius error of a bf16 result against the fp32-accumulated dequantized product: the benchmark's bound
REL_FRO_TOL = 1e-2


def _c_oracle():
    so = os.path.join(ROOT, "oracle", "libmx8_oracle.so")
    if not os.path.exists(so):
        subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "oracle")])
    lib = ctypes.CDLL(so)
    lib.mx8o_quantize_both.restype = ctypes.c_int
    return lib


def test_quantize_configuration_full_matrix_against_the_c_oracle():
    # configuration 2 in full: every byte of both orientations and every scale byte of all 16384 rows, the
    # oracle's C restatement working on 1024-row slabs in parallel threads
    M = N = 16384
    x = O.make_input(M, N, seed=1234, outliers=True, zero_blocks=True)
    fp8, sc, fp8_t, sc_t = (t.view(torch.uint8).cpu().numpy() for t in mx8.mxfp8_quantize(x.to(DEV), True, True))
    assert mx8.device_status() == 0
    lib = _c_oracle()
    xb = x.view(torch.int16).numpy().view(np.uint16)
    u8p, u16p = ctypes.POINTER(ctypes.c_uint8), ctypes.POINTER(ctypes.c_uint16)
    R = 1024

    def slab(r0):
        q, s = np.empty((R, N), np.uint8), np.empty((R // 128, N // 128, 512), np.uint8)
        qt, st = np.empty((N, R), np.uint8), np.empty((N // 128, R // 128, 512), np.uint8)
        rc = lib.mx8o_quantize_both(np.ascontiguousarray(xb[r0:r0 + R]).ctypes.data_as(u16p), R, N, 0, q.ctypes.data_as(u8p),
                                    s.ctypes.data_as(u8p), qt.ctypes.data_as(u8p), st.ctypes.data_as(u8p))
        assert rc == 0
        t0 = r0 // 128
        return (r0, np.array_equal(fp8[r0:r0 + R], q), np.array_equal(sc[t0:t0 + R // 128].reshape(R // 128, N // 128, 512), s),
                np.array_equal(fp8_t[:, r0:r0 + R], qt), np.array_equal(sc_t[:, t0:t0 + R // 128].reshape(N // 128, R // 128, 512), st))

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(16, os.cpu_count() or 1)) as pool:
        results = list(pool.map(slab, range(0, M, R)))
    assert len(results) == M // R
    for r0, *same in results:
        assert all(same), f"rows {r0}..{r0 + R}: fp8 / scales / fp8_t / scales_t equal = {same}"


def _gpu_weight(rows, cols, seed, std=0.02):
    """bf16 weights ~ N(0, std) drawn on the GPU and quantized row-wise there; returns device (fp8, scale tiles)"""
    g = torch.Generator(device=DEV).manual_seed(seed)
    w = (torch.randn(rows, cols, device=DEV, generator=g) * std).to(torch.bfloat16)
    q, sc, _, _ = mx8.mxfp8_quantize(w, True, False)
    return q, sc


def _band_product(a_q, a_sc, b_q_dev, b_sc_dev):
    """oracle product of a band of A (CPU bytes) with a whole device-resident B, 4096 rows of B at a time"""
    out = []
    for n0 in range(0, b_q_dev.shape[0], 4096):
        bq = b_q_dev[n0:n0 + 4096].view(torch.uint8).cpu()
        bs = b_sc_dev[n0 // 128:(n0 + 4096) // 128].cpu()
        out.append(O.gemm_ref(a_q, a_sc, bq, bs))
    return torch.cat(out, dim=1)


def test_ffn_chain_at_llama_70b_shape():
    # configuration 4: X [16384 x 8192] -> quantize -> H = X W1^T leaves the epilogue as MXFP8 -> Y = H W2^T.
    # The whole problem runs on the GPU; three 256-row bands are checked against the oracle (K = 8192 then 28672).
    T, D, F = 16384, 8192, 28672
    x = O.make_input(T, D, seed=4)
    w1q, w1s = _gpu_weight(F, D, 41)
    w2q, w2s = _gpu_weight(D, F, 42)
    xq, xs, _, _ = mx8.mxfp8_quantize(x.to(DEV), True, False)
    hq = torch.empty(T, F, dtype=torch.float8_e4m3fn, device=DEV)
    hs = torch.empty(T // 128, F // 128, 32, 16, dtype=torch.uint8, device=DEV)
    mx8.gemm_grouped(xq, xs, w1q, w1s, hq, hs)
    y = torch.empty(T, D, dtype=torch.bfloat16, device=DEV)
    mx8.kernel(hq, hs, w2q, w2s, y)
    assert mx8.device_status() == 0
    for r0 in (0, 8192 + 256, T - 256):
        rows, tiles = slice(r0, r0 + 256), slice(r0 // 128, r0 // 128 + 2)
        q_ref, s_ref = O.quantize_tiled(x[rows])
        assert torch.equal(xq[rows].view(torch.uint8).cpu(), q_ref) and torch.equal(xs[tiles].cpu(), s_ref)
        # first GEMM: bf16-rounded accumulator, quantized in the epilogue; against the oracle's product, quantized the same way
        h_ref_q, h_ref_s = O.quantize_tiled(_band_product(q_ref, s_ref, w1q, w1s))
        h_got_q, h_got_s = hq[rows].view(torch.uint8).cpu(), hs[tiles].cpu()
        deq = lambda q, s: O.dequantize(q, O.scale_unswizzle(s))
        assert O.rel_frobenius(deq(h_got_q, h_got_s), deq(h_ref_q, h_ref_s)) < REL_FRO_TOL
        assert float((h_got_q != h_ref_q).float().mean()) < 2e-2      # a bf16 flip of the accumulator moves an E4M3 byte
        # second GEMM on the bytes the first one wrote (K = 28672), and the chain from the oracle's own H
        y_got = y[rows].cpu()
        assert O.rel_frobenius(y_got, _band_product(h_got_q, h_got_s, w2q, w2s)) < 2e-3
        assert O.rel_frobenius(y_got, _band_product(h_ref_q, h_ref_s, w2q, w2s)) < REL_FRO_TOL


@pytest.mark.parametrize("pipelined", [False, True])
def test_moe_layer_at_deepseek_v3_shape_with_256_expert_groups(pipelined):
    # configuration 5 at one GPU: 256 local experts, hidden 7168, intermediate 2048.  Three experts receive
    # tokens (one of them two row tiles, all with padding rows), the other 253 groups are empty; the layer runs
    # once as one sequence and once in minibatches of experts on three streams.
    E, H, I, T = 256, 7168, 2048, 1024
    live = {3: 200, 130: 300, 255: 90}
    ids = torch.empty(T, dtype=torch.int32)
    t = 0
    for e, n in live.items():
        ids[t:t + n] = e
        t += n
    ids[t:] = torch.tensor(list(live), dtype=torch.int32)[torch.arange(T - t) % 3]
    counts = {e: int((ids == e).sum()) for e in live}
    cap = 2048
    x = O.make_input(T, H, seed=5)
    xd = x.to(DEV)
    cb = torch.zeros(T, H, dtype=torch.bfloat16, device=DEV)

    def weights(rows, cols, seed):
        q = torch.empty(E, rows, cols, dtype=torch.float8_e4m3fn, device=DEV)
        sc = torch.empty(E * rows // 128, cols // 128, 32, 16, dtype=torch.uint8, device=DEV)
        g = torch.Generator(device=DEV).manual_seed(seed)
        for e0 in range(0, E, 32):
            w = (torch.randn(32, rows, cols, device=DEV, generator=g) * 0.02).to(torch.bfloat16)
            mx8.mxfp8_quantize(w, q[e0:e0 + 32], sc[e0 * rows // 128:(e0 + 32) * rows // 128], None, None, True, False)
        return q, sc

    wg, wu, wd = weights(I, H, 51), weights(I, H, 52), weights(H, I, 53)
    topk_all = ids.view(1, T, 1).to(DEV)
    pr, pt, nt, tpe = mx8.schedule(topk_all, E, cap, 0)
    rpr, rpt, rnt, rtpe, written = MO.schedule_ref(ids.view(1, T, 1), E, cap, 0)
    assert torch.equal(pr.cpu(), rpr) and torch.equal(tpe.cpu(), rtpe) and int(nt) == int(rnt)
    assert [int(rtpe[e]) for e in live] == [-(-counts[e] // 256) * 256 for e in live] and int(rtpe.sum()) == int(rnt)
    kw = dict(num_comm_sms=28, minibatch_size=512) if pipelined else {}
    f = mx8.dispatch_mlp_swiglu_combine_fwd(xd, [xd.data_ptr()], cb, [cb.data_ptr()], None, *wg, None, *wu, None, *wd, pr, pt, nt, tpe, 1, **kw)
    assert mx8.device_status() == 0
    n = int(nt)
    x_routed = MO.dispatch_ref(x.view(1, T, H), rpr, rpt, n, 1)
    # the oracle gets only the three live experts' weights (as a 3-expert problem with the same row segments)
    sel = sorted(live)
    pick = lambda w, rows: (torch.cat([w[0][e:e + 1] for e in sel]).view(torch.uint8).cpu(),
                            torch.cat([w[1][e * rows // 128:(e + 1) * rows // 128] for e in sel]).cpu())
    ref = MO.expert_mlp_ref(x_routed, rtpe[sel], pick(wg, I), pick(wu, I), pick(wd, H))
    deq = lambda q, s: O.dequantize(q.view(torch.uint8).cpu(), O.scale_unswizzle(s.cpu()))
    assert torch.equal(f[0][:, :n].view(torch.uint8).cpu(), ref["x_fp8_t"])                       # dispatch + transposed quantize
    assert torch.equal(f[1][:, :n // 128].cpu(), ref["x_sc_t"])
    for name, q, s in (("gate", f[3], f[4]), ("up", f[6], f[7])):
        assert O.rel_frobenius(deq(q[:n], s[:n // 128]), deq(ref[name + "_fp8"], ref[name + "_sc"])) < REL_FRO_TOL, name
        assert float((q[:n].view(torch.uint8).cpu() != ref[name + "_fp8"]).float().mean()) < 2e-2, name
    assert O.rel_frobenius(deq(f[9][:, :n], f[10][:, :n // 128]), deq(ref["hidden_fp8_t"], ref["hidden_sc_t"])) < REL_FRO_TOL
    y = f[12][:n].cpu()
    assert O.rel_frobenius(y, ref["y"]) < REL_FRO_TOL
    assert not y[rpr[:n] < 0].any()                                                               # padding rows stay zero
    valid = rpr[:n] >= 0
    assert torch.equal(cb.cpu()[rpt[:n][valid].long()].view(torch.int16), y[valid].view(torch.int16))   # combine is a copy
