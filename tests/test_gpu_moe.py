"""MoE pieces on the GPU (through the C ABI) against the CPU oracle."""
import pytest
import torch

import mx8
from oracle import moe_oracle as MO
from oracle import mx8_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def make_topk(W, T, E_total, k, seed):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(W * T, E_total, generator=g)
    ids, w = MO.route(logits, k)
    return ids.view(W, T, k), w.view(W, T, k)


@pytest.mark.parametrize("W,T,E_local,k,rank", [(1, 512, 8, 4, 0), (4, 256, 4, 8, 2), (8, 512, 32, 8, 5), (2, 1024, 3, 2, 1)])
def test_schedule_matches_oracle(W, T, E_local, k, rank):
    topk_all, _ = make_topk(W, T, W * E_local, k, seed=W * 100 + T)
    cap = ((W * T * k) // 256 + E_local) * 256            # every pair could land here, plus padding
    pr, pt, nt, tpe = mx8.schedule(topk_all.to(DEV), E_local, cap, rank)
    assert mx8.device_status() == 0
    rpr, rpt, rnt, rtpe, written = MO.schedule_ref(topk_all, E_local, cap, rank)
    assert torch.equal(nt.cpu(), rnt) and torch.equal(tpe.cpu(), rtpe)
    assert torch.equal(pr.cpu(), rpr)
    assert torch.equal(pt.cpu()[written], rpt[written])      # rows never written hold no defined index
    assert int(tpe.sum()) == int(nt) and bool((tpe % 256 == 0).all())


def test_schedule_is_a_permutation_of_the_routed_pairs():
    W, T, E_local, k, rank = 4, 512, 8, 8, 1
    topk_all, _ = make_topk(W, T, W * E_local, k, seed=5)
    cap = W * T * k
    pr, pt, nt, tpe = (t.cpu() for t in mx8.schedule(topk_all.to(DEV), E_local, cap, rank))
    valid = pr >= 0
    chosen = topk_all.view(W, T * k)[pr[valid].long(), pt[valid].long()]
    bounds = torch.cumsum(tpe, 0)
    rows = torch.nonzero(valid).squeeze(1)
    expert_of_row = torch.bucketize(rows, bounds, right=True)
    assert torch.equal(chosen.long(), rank * E_local + expert_of_row)
    n_local = int(((topk_all >= rank * E_local) & (topk_all < (rank + 1) * E_local)).sum())
    assert int(valid.sum()) == n_local
    keys = pr[valid].long() * (T * k) + pt[valid].long()
    assert keys.unique().numel() == n_local


def test_schedule_overflow_is_reported_not_trapped():
    topk_all, _ = make_topk(2, 512, 4, 2, seed=9)
    pr, pt, nt, tpe = mx8.schedule(topk_all.to(DEV), 2, 256, 0)
    with pytest.raises(mx8.Mx8Error):
        mx8.device_status()
    assert int(nt) > 256
    assert mx8.device_status() == 0          # the word is cleared by the read


def _quant(x):
    return O.quantize_tiled(x)


def test_gemm_quantizing_epilogue_dense():
    # C emitted as MXFP8 must equal the oracle's quantization of the kernel's own bf16 C, bit for bit
    M, N, K = 512, 768, 512
    aq, asc = _quant(O.make_input(M, K, seed=1, std=K ** -0.25))
    bq, bsc = _quant(O.make_input(N, K, seed=2, std=K ** -0.25))
    d = [t.to(DEV) for t in (aq, asc, bq, bsc)]
    c_bf16 = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    mx8.gemm_grouped(*d, c_bf16)
    c_q = torch.full((M, N), 0xFF, dtype=torch.uint8, device=DEV)
    c_sc = torch.full((M // 128, N // 128, 32, 16), 0xFF, dtype=torch.uint8, device=DEV)
    mx8.gemm_grouped(*d, c_q, c_sc)
    assert mx8.device_status() == 0
    ref = O.gemm_ref(aq, asc, bq, bsc)
    assert O.rel_frobenius(c_bf16.cpu(), ref) < 2e-3
    want_q, want_sc = O.quantize_tiled(c_bf16.cpu())
    assert torch.equal(c_q.cpu(), want_q)
    assert torch.equal(c_sc.cpu(), want_sc)


@pytest.mark.parametrize("mode", ["bf16", "mxfp8"])
def test_gemm_grouped_by_expert(mode):
    E, N, K = 5, 512, 384
    group_rows = torch.tensor([512, 0, 256, 768, 256], dtype=torch.int32)
    used = int(group_rows.sum())
    cap = used + 512                                     # capacity beyond the rows present
    a = O.make_input(cap, K, seed=3, std=K ** -0.25)
    w = torch.stack([O.make_input(N, K, seed=10 + e, std=K ** -0.25) for e in range(E)])
    aq, asc = _quant(a)
    wq, wsc, _, _ = O.quantize_both(w)
    num_rows = torch.tensor([used], dtype=torch.int32)
    d = [t.to(DEV) for t in (aq, asc, wq, wsc)]
    if mode == "bf16":
        c = torch.full((cap, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        mx8.gemm_grouped(*d, c, None, num_rows.to(DEV), group_rows.to(DEV))
    else:
        c = torch.full((cap, N), 0xFF, dtype=torch.uint8, device=DEV)
        csc = torch.full((cap // 128, N // 128, 32, 16), 0xFF, dtype=torch.uint8, device=DEV)
        mx8.gemm_grouped(*d, c, csc, num_rows.to(DEV), group_rows.to(DEV))
    assert mx8.device_status() == 0
    off = 0
    for e, n in enumerate(group_rows.tolist()):
        if n == 0:
            continue
        ref = O.gemm_ref(aq[off:off + n], asc[off // 128:(off + n) // 128], wq[e], wsc[e * N // 128:(e + 1) * N // 128])
        if mode == "bf16":
            got = c[off:off + n].cpu()
            assert not torch.isnan(got.float()).any()
            assert O.rel_frobenius(got, ref) < 2e-3, f"expert {e}"
        else:
            deq = O.dequantize(c[off:off + n].cpu(), O.scale_unswizzle(csc[off // 128:(off + n) // 128].cpu()))
            # E4M3 payload: half an ulp of 3 mantissa bits relative to the block amax
            assert O.rel_frobenius(deq, ref) < 5e-2, f"expert {e}"
        off += n
    # rows beyond num_rows are untouched
    tail = c[used:].cpu()
    assert bool(torch.isnan(tail.float()).all()) if mode == "bf16" else bool((tail == 0xFF).all())
