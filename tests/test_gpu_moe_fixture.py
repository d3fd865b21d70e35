"""The routed-expert MLP on the GPU, forward and backward, against outputs of the reference harness's own
mlp_swiglu_fwd_ref / mlp_swiglu_bwd_ref stored in tests/golden/moe_fwd_bwd.npz
(blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.py:91-215, run on CPU by tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest
import torch

import mx8
from oracle import mx8_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_layer_forward_and_backward_match_the_reference_fixture(golden_dir):
    z = np.load(os.path.join(golden_dir, "moe_fwd_bwd.npz"))
    bf = lambda n: torch.from_numpy(z[n].view(np.int16)).view(torch.bfloat16)
    w = lambda n: (torch.from_numpy(z["w_%s_fp8" % n]).view(torch.float8_e4m3fn).to(DEV), torch.from_numpy(z["w_%s_sc" % n]).to(DEV))
    tpe_cpu = torch.from_numpy(z["tokens_per_expert"])
    R, H = z["x_routed"].shape
    # one rank, one routed pair per token: the fixture's rows are the token matrix and the schedule is the identity on
    # the live rows, so dispatch hands the expert GEMMs exactly the fixture's x_routed (padding rows zero-filled)
    pr = torch.full((R,), -1, dtype=torch.int32)
    off = 0
    for n, v in zip(tpe_cpu.tolist(), z["valid_rows"].tolist()):
        pr[off:off + v] = 0
        off += n
    pt = torch.arange(R, dtype=torch.int32)
    pr, pt, nt, tpe = pr.to(DEV), pt.to(DEV), torch.tensor([R], dtype=torch.int32, device=DEV), tpe_cpu.to(DEV)
    x = bf("x_routed").to(DEV)
    cb = torch.zeros(R, H, dtype=torch.bfloat16, device=DEV)
    f = mx8.dispatch_mlp_swiglu_combine_fwd(x, [x.data_ptr()], cb, [cb.data_ptr()], None, *w("gate"), None, *w("up"), None, *w("down"),
                                            pr, pt, nt, tpe, 1)
    assert mx8.device_status() == 0
    live = (pr >= 0).cpu()

    def deq(q, sc):
        return O.dequantize(q.view(torch.uint8).cpu(), O.scale_unswizzle(sc.cpu()))

    # gate / up leave the GEMM epilogue as MXFP8: compare with the quantization of the reference's bf16 gate / up
    for name, q, sc in (("gate", f[3], f[4]), ("up", f[6], f[7])):
        wq, wsc = O.quantize_tiled(bf(name + "_routed"))
        assert O.rel_frobenius(deq(q, sc), O.dequantize(wq, O.scale_unswizzle(wsc))) < 1e-2, name
        assert float((q.view(torch.uint8).cpu() != wq).float().mean()) < 2e-2, name
    # hidden^T as MXFP8 against the transposed quantization of the reference's hidden
    _, _, hq_t, hsc_t = O.quantize_both(bf("hidden_routed"))
    assert O.rel_frobenius(deq(f[9], f[10]), O.dequantize(hq_t, O.scale_unswizzle(hsc_t))) < 1e-2
    y = f[12].cpu()
    assert O.rel_frobenius(y, bf("y_routed")) < 1e-2                       # tolerance of the path's GEMMs, relative Frobenius
    assert not y[~live].any()                                            # padding rows stay zero
    assert torch.equal(cb.cpu()[live].view(torch.int16), y[live].view(torch.int16))   # combine is a copy

    # backward: the gradient rows sit in the (single) rank's own d_combine buffer, one row per routed pair
    d_cb = bf("d_y_routed").to(DEV)
    d_xb = torch.zeros(R, H, dtype=torch.bfloat16, device=DEV)
    b = mx8.dispatch_mlp_swiglu_combine_bwd(None, d_cb, [d_cb.data_ptr()], d_xb, [d_xb.data_ptr()],
                                            None, *w("gate_T"), None, *w("up_T"), None, *w("down_T"),
                                            f[0], f[1], None, f[3], f[4], None, f[6], f[7], None, f[9], f[10],
                                            x, [x.data_ptr()], *w("gate"), *w("up"), pr, pt, nt, tpe, 1)
    assert mx8.device_status() == 0
    tol = 2e-2      # chained MXFP8 GEMMs on re-quantized activations: a bf16 flip upstream moves a few E4M3 bytes downstream
    assert O.rel_frobenius(b[9].cpu(), bf("d_hidden_routed")) < 1e-2
    assert O.rel_frobenius(b[1].cpu(), bf("d_x_routed")) < tol
    for got, name in ((b[13], "d_w_routed_gate"), (b[15], "d_w_routed_up"), (b[17], "d_w_routed_down")):
        assert O.rel_frobenius(got.cpu(), bf(name)) < tol, name
    for (q, sc), name in (((b[3], b[4]), "d_gate_routed"), ((b[6], b[7]), "d_up_routed")):
        wq, wsc = O.quantize_tiled(bf(name))
        assert O.rel_frobenius(deq(q, sc), O.dequantize(wq, O.scale_unswizzle(wsc))) < tol, name
    assert torch.equal(d_xb.cpu()[live].view(torch.int16), b[1].cpu()[live].view(torch.int16))
