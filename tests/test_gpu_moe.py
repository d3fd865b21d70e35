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
