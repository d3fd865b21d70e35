"""The pybind11/torch module mx8._C, called the way the reference's harnesses call their `_C`."""
import pytest
import torch

from oracle import mx8_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def C():
    from mx8 import _C
    return _C


def test_quantize_harness_flow(C):
    # follows the reference harness: preallocated outputs, three modes, exact byte equality
    M, N = 512, 384
    x_cpu = O.make_input(M, N, seed=1234, outliers=True, zero_blocks=True)
    x = x_cpu.to(DEV)
    x_fp8 = torch.zeros(M, N, dtype=torch.float8_e4m3fn, device=DEV)
    x_sc = torch.zeros(M // 128, N // 128, 32, 16, dtype=torch.uint8, device=DEV)
    x_fp8_t = torch.zeros(N, M, dtype=torch.float8_e4m3fn, device=DEV)
    x_sc_t = torch.zeros(N // 128, M // 128, 32, 16, dtype=torch.uint8, device=DEV)
    want = O.quantize_both(x_cpu)
    for rn, rt in ((True, False), (False, True), (True, True)):
        for t in (x_fp8, x_sc, x_fp8_t, x_sc_t):
            t.view(torch.uint8).zero_()
        C.mxfp8_quantize(x, x_fp8, x_sc, x_fp8_t, x_sc_t, rn, rt)
        assert C.device_status() == 0
        errors = 0
        if rn:
            errors += int((x_fp8.view(torch.uint8).cpu() != want[0]).sum()) + int((x_sc.cpu() != want[1]).sum())
        if rt:
            errors += int((x_fp8_t.view(torch.uint8).cpu() != want[2]).sum()) + int((x_sc_t.cpu() != want[3]).sum())
        assert errors == 0


def test_allocating_form_and_3d(C):
    x_cpu = torch.stack([O.make_input(256, 384, seed=s) for s in range(2)])
    q, sc, qt, sct = C.mxfp8_quantize(x_cpu.to(DEV), True, True)
    want = O.quantize_both(x_cpu)
    for got, w in zip((q, sc, qt, sct), want):
        assert torch.equal(got.view(torch.uint8).cpu(), w)
    q, sc, qt, sct = C.mxfp8_quantize(x_cpu[0].to(DEV), True, False)
    assert qt is None and sct is None and q.shape == (256, 384)


def test_gemm_and_legacy_names(C):
    M, N, K = 256, 384, 512
    a = O.make_input(M, K, seed=1, std=K ** -0.25)
    b = O.make_input(N, K, seed=2, std=K ** -0.25)
    # legacy quantize bindings: kernel(A, A_fp8, A_sc) with A_sc [M/128, K/128, 512], kernel_transpose
    a_fp8 = torch.empty(M, K, dtype=torch.float8_e4m3fn, device=DEV)
    a_sc = torch.empty(M // 128, K // 128, 512, dtype=torch.uint8, device=DEV)
    C.kernel(a.to(DEV), a_fp8, a_sc)
    b_fp8, b_sc, _, _ = C.mxfp8_quantize(b.to(DEV), True, False)
    at_fp8 = torch.empty(K, M, dtype=torch.float8_e4m3fn, device=DEV)
    at_sc = torch.empty(K // 128, M // 128, 512, dtype=torch.uint8, device=DEV)
    C.kernel_transpose(a.to(DEV), at_fp8, at_sc)
    want = O.quantize_both(a)
    assert torch.equal(a_fp8.view(torch.uint8).cpu(), want[0]) and torch.equal(a_sc.cpu().view(-1), want[1].view(-1))
    assert torch.equal(at_fp8.view(torch.uint8).cpu(), want[2]) and torch.equal(at_sc.cpu().view(-1), want[3].view(-1))
    ref = O.gemm_ref(want[0], want[1], *O.quantize_tiled(b))
    for dtype in (torch.bfloat16, torch.float32):
        c = torch.zeros(M, N, dtype=dtype, device=DEV)
        C.kernel(a_fp8, a_sc, b_fp8, b_sc, c)
        assert C.device_status() == 0
        assert O.rel_frobenius(c.cpu(), ref) < 1e-2      # benchmark tolerance; observed ~1e-5
        assert O.rel_frobenius(c.cpu(), ref) < 2e-3


def test_errors_raise_runtime_error(C):
    x = torch.zeros(100, 128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError):
        C.mxfp8_quantize(x, True, False)


def test_moe_forward_through_the_cpp_module(C):
    # the reference harness's run_fwd_once with one rank: schedule -> fused forward -> epilogue
    from oracle import moe_oracle as MO
    T, H, I, k, E = 256, 512, 256, 4, 4
    g = torch.Generator().manual_seed(3)
    ids, w = MO.route(torch.randn(T, E, generator=g), k)
    x_cpu = O.make_input(T, H, seed=5)
    x = x_cpu.to(DEV)
    cb = torch.zeros(T * k, H, dtype=torch.bfloat16, device=DEV)
    ws = []
    for seed, (r, c) in ((10, (I, H)), (20, (I, H)), (30, (H, I))):
        wt = torch.stack([O.make_input(r, c, seed=seed + e, std=c ** -0.5) for e in range(E)])
        ws.append(C.mxfp8_quantize(wt.to(DEV), True, False)[:2])
    cap = ((T * k) // 256 + E) * 256
    pr, pt, nt, tpe = C.schedule(ids.view(1, T, k).to(DEV), E, cap, 0)
    outs = C.dispatch_mlp_swiglu_combine_fwd(x, [x.data_ptr()], cb, [cb.data_ptr()], None, ws[0][0], ws[0][1], None, ws[1][0], ws[1][1],
                                             None, ws[2][0], ws[2][1], pr, pt, nt, tpe, k, 40, 8 * 16384, 16384)
    out = C.fwd_epilogue(None, cb, w.to(DEV))
    assert C.device_status() == 0 and len(outs) == 13 and outs[2] is None
    n = int(nt)
    rpr, rpt, rnt, rtpe, _ = MO.schedule_ref(ids.view(1, T, k), E, cap, 0)
    assert torch.equal(pr.cpu(), rpr) and n == int(rnt)
    ref = MO.expert_mlp_ref(MO.dispatch_ref(x_cpu.view(1, T, H), rpr, rpt, n, k), rtpe,
                            *[(q.view(torch.uint8).cpu(), s.cpu()) for q, s in ws])
    assert torch.equal(outs[0][:, :n].view(torch.uint8).cpu(), ref["x_fp8_t"])
    assert O.rel_frobenius(outs[12][:n].cpu(), ref["y"]) < 1e-2
    cb_ref = MO.combine_ref([ref["y"]], [rpr], [rpt], 0, T, k)
    ref_out = MO.fwd_epilogue_ref(torch.zeros(T, H, dtype=torch.bfloat16), cb_ref, w)
    assert O.rel_frobenius(out.cpu(), ref_out) < 1e-2


def test_moe_backward_through_the_cpp_module(C):
    # forward then backward through mx8._C; the result must equal the ctypes host path bit for bit
    import mx8
    from oracle import moe_oracle as MO
    T, H, I, k, E = 256, 512, 256, 4, 6
    g = torch.Generator().manual_seed(4)
    ids, w = MO.route(torch.randn(T, E, generator=g), k)
    x = O.make_input(T, H, seed=6).to(DEV)
    mk = lambda r, c, sd: torch.stack([O.make_input(r, c, seed=sd + e, std=c ** -0.5) for e in range(E)]).to(DEV)
    wg, wu, wd = mk(I, H, 10), mk(I, H, 20), mk(H, I, 30)
    fw = [C.mxfp8_quantize(t, True, False)[:2] for t in (wg, wu, wd)]
    bw = [C.mxfp8_quantize(t.transpose(1, 2).contiguous(), True, False)[:2] for t in (wg, wu, wd)]
    cap = ((T * k) // 256 + E) * 256
    pr, pt, nt, tpe = C.schedule(ids.view(1, T, k).to(DEV), E, cap, 0)
    cb = torch.zeros(T * k, H, dtype=torch.bfloat16, device=DEV)
    f = C.dispatch_mlp_swiglu_combine_fwd(x, [x.data_ptr()], cb, [cb.data_ptr()], None, *fw[0], None, *fw[1], None, *fw[2], pr, pt, nt, tpe, k)
    d_out = O.make_input(T, H, seed=7, std=H ** -0.5).to(DEV)
    results = []
    for host in (C, mx8):
        d_cb = torch.zeros(T * k, H, dtype=torch.bfloat16, device=DEV)
        d_xb = torch.zeros(T * k, H, dtype=torch.bfloat16, device=DEV)
        d_y_shared = host.bwd_prologue(d_out, w.to(DEV), d_cb)
        b = host.dispatch_mlp_swiglu_combine_bwd(None, d_cb, [d_cb.data_ptr()], d_xb, [d_xb.data_ptr()], None, *bw[0], None, *bw[1],
                                                 None, *bw[2], f[0], f[1], None, f[3], f[4], None, f[6], f[7], None, f[9], f[10],
                                                 x, [x.data_ptr()], *fw[0], *fw[1], pr, pt, nt, tpe, k, 28, 8 * 16384, 16384)
        d_x = host.bwd_epilogue(torch.zeros(T, H, dtype=torch.bfloat16, device=DEV), d_xb)
        assert len(b) == 18 and b[0] is None and d_y_shared.data_ptr() == d_out.data_ptr()
        results.append((b, d_x))
    assert C.device_status() == 0
    n = int(nt)
    (bc, dxc), (bp, dxp) = results
    assert torch.equal(dxc.view(torch.int16), dxp.view(torch.int16))
    for i in (1, 9):
        assert torch.equal(bc[i][:n].view(torch.int16), bp[i][:n].view(torch.int16))
    for i in (13, 15, 17):
        assert torch.equal(bc[i].view(torch.int16), bp[i].view(torch.int16))


def test_shared_expert_through_both_hosts(C):
    # layer forward + backward with shared-expert weights: the C++ module and the ctypes host give the
    # same bits (same kernels, same launch order) and both agree with the oracle's bf16 expert
    import mx8
    from oracle import moe_oracle as MO
    T, H, I, Is, k, E = 256, 512, 256, 384, 4, 6
    g = torch.Generator().manual_seed(14)
    ids, w = MO.route(torch.randn(T, E, generator=g), k)
    x_cpu = O.make_input(T, H, seed=16)
    x = x_cpu.to(DEV)
    mk = lambda r, c, sd: torch.stack([O.make_input(r, c, seed=sd + e, std=c ** -0.5) for e in range(E)]).to(DEV)
    wg, wu, wd = mk(I, H, 10), mk(I, H, 20), mk(H, I, 30)
    sg, su, sd = (O.make_input(Is, H, seed=40, std=H ** -0.5), O.make_input(Is, H, seed=41, std=H ** -0.5),
                  O.make_input(H, Is, seed=42, std=Is ** -0.5))
    fw = [C.mxfp8_quantize(t, True, False)[:2] for t in (wg, wu, wd)]
    bw = [C.mxfp8_quantize(t.transpose(1, 2).contiguous(), True, False)[:2] for t in (wg, wu, wd)]
    cap = ((T * k) // 256 + E) * 256
    pr, pt, nt, tpe = C.schedule(ids.view(1, T, k).to(DEV), E, cap, 0)
    d_out = O.make_input(T, H, seed=17, std=H ** -0.5)
    res = []
    for host in (C, mx8):
        cb = torch.zeros(T * k, H, dtype=torch.bfloat16, device=DEV)
        f = host.dispatch_mlp_swiglu_combine_fwd(x, [x.data_ptr()], cb, [cb.data_ptr()], sg.to(DEV), *fw[0], su.to(DEV), *fw[1],
                                                 sd.to(DEV), *fw[2], pr, pt, nt, tpe, k)
        d_cb = torch.zeros(T * k, H, dtype=torch.bfloat16, device=DEV)
        d_xb = torch.zeros(T * k, H, dtype=torch.bfloat16, device=DEV)
        d_y_shared = host.bwd_prologue(d_out.to(DEV), w.to(DEV), d_cb)
        b = host.dispatch_mlp_swiglu_combine_bwd(d_y_shared, d_cb, [d_cb.data_ptr()], d_xb, [d_xb.data_ptr()],
                                                 sg.t().contiguous().to(DEV), *bw[0], su.t().contiguous().to(DEV), *bw[1],
                                                 sd.t().contiguous().to(DEV), *bw[2], f[0], f[1], f[2], f[3], f[4], f[5], f[6], f[7],
                                                 f[8], f[9], f[10], x, [x.data_ptr()], *fw[0], *fw[1], pr, pt, nt, tpe, k, 28, 8 * 16384, 16384)
        res.append((f, b))
    assert C.device_status() == 0
    (fc, bc), (fp, bp) = res
    for i in (2, 5, 8, 11):
        assert torch.equal(fc[i].view(torch.int16), fp[i].view(torch.int16)), i
    for i in (0, 2, 5, 8, 12, 14, 16):
        assert torch.equal(bc[i].view(torch.int16), bp[i].view(torch.int16)), i
    gate, up, hidden, y = MO.shared_mlp_ref(x_cpu, sg, su, sd)
    for got, want in ((fc[2], gate), (fc[5], up), (fc[8], hidden), (fc[11], y)):
        assert O.rel_frobenius(got.cpu().float(), want.float()) < 1e-2
    ref = MO.shared_mlp_bwd_ref(d_out, x_cpu, fc[2].cpu(), fc[5].cpu(), fc[8].cpu(), sg, su, sd)
    for i, want in ((0, ref[0]), (2, ref[1]), (5, ref[2]), (8, ref[3]), (12, ref[4]), (14, ref[5]), (16, ref[6])):
        assert O.rel_frobenius(bc[i].cpu().float(), want.float()) < 1e-2, i


def test_pipelined_forward_through_the_cpp_module(C):
    # minibatches on three streams (num_comm_sms, minibatch_size as in the reference's call): same bytes as the
    # one-stream sequence, from the C++ module and from the ctypes host
    import mx8
    from oracle import moe_oracle as MO
    T, H, I, k, E = 384, 512, 256, 4, 5
    g = torch.Generator().manual_seed(24)
    ids, _ = MO.route(torch.randn(T, E, generator=g), k)
    x = O.make_input(T, H, seed=26).to(DEV)
    mk = lambda r, c, sd: torch.stack([O.make_input(r, c, seed=sd + e, std=c ** -0.5) for e in range(E)]).to(DEV)
    fw = [C.mxfp8_quantize(t, True, False)[:2] for t in (mk(I, H, 10), mk(I, H, 20), mk(H, I, 30))]
    cap = ((T * k) // 256 + E) * 256
    pr, pt, nt, tpe = C.schedule(ids.view(1, T, k).to(DEV), E, cap, 0)
    n = int(nt)
    res = []
    for host, knobs in ((C, (0, 0, 0)), (C, (28, 0, 512)), (mx8, (28, 0, 512))):
        cb = torch.full((T * k, H), -2.0, dtype=torch.bfloat16, device=DEV)
        f = host.dispatch_mlp_swiglu_combine_fwd(x, [x.data_ptr()], cb, [cb.data_ptr()], None, *fw[0], None, *fw[1], None, *fw[2],
                                                 pr, pt, nt, tpe, k, *knobs)
        torch.cuda.synchronize()
        res.append((f, cb))
    assert C.device_status() == 0
    for f, cb in res[1:]:
        assert torch.equal(cb.view(torch.int16), res[0][1].view(torch.int16))
        assert torch.equal(f[12][:n].view(torch.int16), res[0][0][12][:n].view(torch.int16))
        for i in (3, 6):
            assert torch.equal(f[i][:n].view(torch.uint8), res[0][0][i][:n].view(torch.uint8))
        for i in (0, 9):
            assert torch.equal(f[i][:, :n].view(torch.uint8), res[0][0][i][:, :n].view(torch.uint8))


def test_pipelined_backward_through_the_cpp_module(C):
    import mx8
    from oracle import moe_oracle as MO
    T, H, I, k, E = 384, 512, 256, 4, 5
    g = torch.Generator().manual_seed(34)
    ids, w = MO.route(torch.randn(T, E, generator=g), k)
    x = O.make_input(T, H, seed=36).to(DEV)
    mk = lambda r, c, sd: torch.stack([O.make_input(r, c, seed=sd + e, std=c ** -0.5) for e in range(E)]).to(DEV)
    wg, wu, wd = mk(I, H, 10), mk(I, H, 20), mk(H, I, 30)
    fw = [C.mxfp8_quantize(t, True, False)[:2] for t in (wg, wu, wd)]
    bw = [C.mxfp8_quantize(t.transpose(1, 2).contiguous(), True, False)[:2] for t in (wg, wu, wd)]
    cap = ((T * k) // 256 + E) * 256
    pr, pt, nt, tpe = C.schedule(ids.view(1, T, k).to(DEV), E, cap, 0)
    cb = torch.zeros(T * k, H, dtype=torch.bfloat16, device=DEV)
    f = C.dispatch_mlp_swiglu_combine_fwd(x, [x.data_ptr()], cb, [cb.data_ptr()], None, *fw[0], None, *fw[1], None, *fw[2], pr, pt, nt, tpe, k)
    d_out = O.make_input(T, H, seed=37, std=H ** -0.5).to(DEV)
    d_cb = torch.zeros(T * k, H, dtype=torch.bfloat16, device=DEV)
    C.bwd_prologue(d_out, w.to(DEV), d_cb)
    res = []
    for host, knobs in ((C, (0, 0, 0)), (C, (28, 0, 512)), (mx8, (28, 0, 512))):
        d_xb = torch.full((T * k, H), -4.0, dtype=torch.bfloat16, device=DEV)
        b = host.dispatch_mlp_swiglu_combine_bwd(None, d_cb, [d_cb.data_ptr()], d_xb, [d_xb.data_ptr()], None, *bw[0], None, *bw[1],
                                                 None, *bw[2], f[0], f[1], None, f[3], f[4], None, f[6], f[7], None, f[9], f[10],
                                                 x, [x.data_ptr()], *fw[0], *fw[1], pr, pt, nt, tpe, k, *knobs)
        torch.cuda.synchronize()
        res.append((b, d_xb))
    assert C.device_status() == 0
    n = int(nt)
    for b, d_xb in res[1:]:
        assert torch.equal(d_xb.view(torch.int16), res[0][1].view(torch.int16))
        for i in (1, 9):
            assert torch.equal(b[i][:n].view(torch.int16), res[0][0][i][:n].view(torch.int16))
        for i in (13, 15, 17):
            assert torch.equal(b[i].view(torch.int16), res[0][0][i].view(torch.int16))
