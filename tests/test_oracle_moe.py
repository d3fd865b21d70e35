"""CPU checks of the MoE oracle: the schedule's placement rule, padding, and the layer composition."""
import torch

from oracle import moe_oracle as MO
from oracle import mx8_oracle as O


def _topk(W, T, E, k, seed):
    g = torch.Generator().manual_seed(seed)
    return MO.route(torch.randn(W * T, E, generator=g), k)[0].view(W, T, k)


def test_schedule_interleaves_source_ranks_round_by_round():
    # 2 ranks, one local expert (id 0): rank 0 routes pairs 1 and 5 to it, rank 1 routes pairs 0, 2, 7
    topk_all = torch.full((2, 4, 2), 9, dtype=torch.int32)
    topk_all.view(2, 8)[0, [1, 5]] = 0
    topk_all.view(2, 8)[1, [0, 2, 7]] = 0
    pr, pt, nt, tpe, written = MO.schedule_ref(topk_all, 1, 512, 0)
    assert pr[:5].tolist() == [0, 1, 0, 1, 1] and pt[:5].tolist() == [1, 0, 5, 2, 7]
    assert int(nt) == 256 and tpe.tolist() == [256] and bool((pr[5:] == -1).all())


def test_schedule_transcription_equals_thread_by_thread_execution():
    # the array form of the reference's placement kernel against the same kernel run thread by thread,
    # below, at and above 1024 entries per rank (where the order stops being table order)
    for (W, T, k, E_local, rank, seed) in ((2, 64, 4, 2, 1, 1), (1, 128, 8, 16, 0, 2), (2, 512, 4, 2, 0, 3), (3, 700, 3, 2, 2, 4)):
        topk_all = _topk(W, T, W * E_local, k, seed)
        cap = (W * T * k + 256 * E_local + 255) // 256 * 256
        a = MO.schedule_ref(topk_all, E_local, cap, rank)
        b = MO.schedule_ref_threads(topk_all, E_local, cap, rank)
        n = int(a[2])
        assert int(b[2]) == n and torch.equal(a[3], b[3])
        assert torch.equal(a[0], b[0])
        assert torch.equal(a[1][a[4]], b[1][a[4]])


def test_schedule_order_is_thread_strided_above_1024_entries():
    # one rank, one expert, every pair routed to it: 2048 entries -> thread t holds entries t and t + 1024,
    # so the rows read 0, 1024, 1, 1025, ...
    topk_all = torch.zeros(1, 512, 4, dtype=torch.int32)
    pr, pt, nt, tpe, written = MO.schedule_ref(topk_all, 1, 2048, 0)
    assert int(nt) == 2048 and bool(written.all())
    assert pt[:6].tolist() == [0, 1024, 1, 1025, 2, 1026]
    # at 1024 entries the order is table order
    pr, pt, nt, tpe, written = MO.schedule_ref(torch.zeros(1, 256, 4, dtype=torch.int32), 1, 1024, 0)
    assert pt.tolist() == list(range(1024))


def test_schedule_segments_are_padded_and_complete():
    W, T, E_local, k = 4, 128, 4, 4
    topk_all = _topk(W, T, W * E_local, k, 3)
    for rank in range(W):
        pr, pt, nt, tpe, written = MO.schedule_ref(topk_all, E_local, W * T * k, rank)
        assert bool((tpe % 256 == 0).all()) and int(tpe.sum()) == int(nt)
        n_local = int(((topk_all >= rank * E_local) & (topk_all < (rank + 1) * E_local)).sum())
        assert int((pr >= 0).sum()) == n_local == int(written.sum())


def test_layer_composition_shapes_and_padding_rows():
    W, T, H, I, k, E_local, rank = 2, 128, 256, 128, 2, 2, 0
    topk_all = _topk(W, T, W * E_local, k, 5)
    x_all = torch.stack([O.make_input(T, H, seed=r) for r in range(W)])
    pr, pt, nt, tpe, _ = MO.schedule_ref(topk_all, E_local, 1024, rank)
    n = int(nt)
    xr = MO.dispatch_ref(x_all, pr, pt, n, k)
    assert not xr[pr[:n] < 0].any()
    q = lambda w: O.quantize_both(w)[:2]
    wg = q(torch.stack([O.make_input(I, H, seed=10 + e, std=H ** -0.5) for e in range(E_local)]))
    wu = q(torch.stack([O.make_input(I, H, seed=20 + e, std=H ** -0.5) for e in range(E_local)]))
    wd = q(torch.stack([O.make_input(H, I, seed=30 + e, std=I ** -0.5) for e in range(E_local)]))
    ref = MO.expert_mlp_ref(xr, tpe, wg, wu, wd)
    assert ref["y"].shape == (n, H) and ref["hidden_fp8_t"].shape == (I, n)
    assert not ref["y"][pr[:n] < 0].any()            # zero rows stay zero through the whole MLP
    w = torch.softmax(torch.randn(T, k), -1)
    out = MO.fwd_epilogue_ref(torch.zeros(T, H, dtype=torch.bfloat16), torch.ones(T * k, H, dtype=torch.bfloat16), w)
    assert torch.allclose(out.float(), torch.ones(T, H), atol=1e-2)


def test_shared_expert_backward_matches_autograd():
    # the oracle's hand-written bf16 expert backward against autograd of the same forward in float64
    # (bf16 rounding of the intermediates bounds the agreement)
    T, H, I = 64, 96, 80
    g = torch.Generator().manual_seed(3)
    r = lambda *s: torch.randn(*s, generator=g)
    x, wg, wu, wd, d_y = r(T, H).bfloat16(), (r(I, H) * 0.1).bfloat16(), (r(I, H) * 0.1).bfloat16(), (r(H, I) * 0.1).bfloat16(), r(T, H).bfloat16()
    gate, up, hidden, y = MO.shared_mlp_ref(x, wg, wu, wd)
    got = MO.shared_mlp_bwd_ref(d_y, x, gate, up, hidden, wg, wu, wd)
    xs, wgs, wus, wds = [t.double().requires_grad_() for t in (x, wg, wu, wd)]
    gt, ut = xs @ wgs.t(), xs @ wus.t()
    out = (torch.nn.functional.silu(gt) * ut) @ wds.t()
    out.backward(d_y.double())
    for have, want in ((got[0], xs.grad), (got[4], wgs.grad), (got[5], wus.grad), (got[6], wds.grad)):
        assert O.rel_frobenius(have.float(), want.float()) < 2e-2
    assert O.rel_frobenius(y.float(), out.detach().float()) < 2e-2


def _fixture(golden_dir):
    import os

    import numpy as np
    z = np.load(os.path.join(golden_dir, "moe_fwd_bwd.npz"))
    bf = lambda n: torch.from_numpy(z[n].view(np.int16)).view(torch.bfloat16)
    w = lambda n: (torch.from_numpy(z["w_%s_fp8" % n]), torch.from_numpy(z["w_%s_sc" % n]))
    return z, bf, w


def test_expert_mlp_oracle_reproduces_the_reference_functions(golden_dir):
    # moe_fwd_bwd.npz holds inputs and outputs of the reference harness's mlp_swiglu_fwd_ref / mlp_swiglu_bwd_ref
    # (two experts, segments of 256 rows with 96 and 40 live rows).  Both sides run the same fp32 products on CPU,
    # so bf16 results may differ only where an fp32 sum lands on a rounding boundary: equality is asked of the
    # quantized bytes and of nearly all bf16 elements, closeness of the rest.
    z, bf, w = _fixture(golden_dir)
    tpe = torch.from_numpy(z["tokens_per_expert"])
    fwd = MO.expert_mlp_ref(bf("x_routed"), tpe, w("gate"), w("up"), w("down"))

    def close(have, want, name):
        assert have.shape == want.shape, name
        diff = (have.view(torch.int16) != want.view(torch.int16)).float().mean().item()
        assert diff < 1e-3 and O.rel_frobenius(have, want) < 1e-4, (name, diff)

    for name in ("gate", "up"):
        q, sc = O.quantize_tiled(bf(name + "_routed"))
        same = (q == fwd[name + "_fp8"]).float().mean().item()
        assert same > 0.999 and torch.equal(sc, fwd[name + "_sc"]), name
    close(fwd["hidden"], bf("hidden_routed"), "hidden")
    close(fwd["y"], bf("y_routed"), "y")
    bwd = MO.expert_mlp_bwd_ref(bf("d_y_routed"), fwd, tpe, w("gate_T"), w("up_T"), w("down_T"))
    for mine, theirs in (("d_hidden", "d_hidden_routed"), ("d_gate", "d_gate_routed"), ("d_up", "d_up_routed"), ("d_x", "d_x_routed"),
                         ("d_w_gate", "d_w_routed_gate"), ("d_w_up", "d_w_routed_up"), ("d_w_down", "d_w_routed_down")):
        close(bwd[mine], bf(theirs), mine)
    # padding rows stay zero through the layer, as in the reference
    off = 0
    for n, v in zip(tpe.tolist(), z["valid_rows"].tolist()):
        assert not fwd["y"][off + v:off + n].any() and not bwd["d_x"][off + v:off + n].any()
        off += n


def test_shared_expert_oracle_reproduces_the_reference_functions(golden_dir):
    z, bf, w = _fixture(golden_dir)
    names = ("gate_shared", "up_shared", "hidden_shared", "y_shared")
    fwd = MO.shared_mlp_ref(bf("x_shared"), bf("w_shared_gate"), bf("w_shared_up"), bf("w_shared_down"))
    for have, name in zip(fwd, names):
        assert O.rel_frobenius(have, bf(name)) < 1e-4, name
    bwd = MO.shared_mlp_bwd_ref(bf("d_y_shared"), bf("x_shared"), bf("gate_shared"), bf("up_shared"), bf("hidden_shared"),
                                bf("w_shared_gate"), bf("w_shared_up"), bf("w_shared_down"))
    for have, name in zip(bwd, ("d_x_shared", "d_gate_shared", "d_up_shared", "d_hidden_shared", "d_w_shared_gate",
                                "d_w_shared_up", "d_w_shared_down")):
        assert O.rel_frobenius(have, bf(name)) < 1e-4, name


def _skewed_topk(W, T, E, k, seed, hot):
    """routing with one hot expert: `hot` percent of the pairs go to expert 0, the rest uniformly anywhere"""
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, E, (W, T, k), generator=g, dtype=torch.int32)
    ids[torch.rand(W, T, k, generator=g) * 100 < hot] = 0
    return ids


def test_schedule_transcription_equals_threads_on_random_shapes():
    # property test over odd shapes: token counts that are no multiple of anything, one to eight source ranks,
    # skewed routing (a hot expert whose list is many rounds long), tables below and above the 1024-entry stride
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=30, deadline=None, derandomize=True)
    @given(W=st.integers(1, 4), T=st.integers(1, 900), k=st.integers(1, 4), E_local=st.integers(1, 5),
           hot=st.sampled_from([0, 30, 90]), seed=st.integers(0, 10 ** 6), data=st.data())
    def check(W, T, k, E_local, hot, seed, data):
        rank = data.draw(st.integers(0, W - 1))
        topk_all = _skewed_topk(W, T, W * E_local, k, seed, hot)
        cap = (W * T * k + 256 * E_local + 255) // 256 * 256
        a = MO.schedule_ref(topk_all, E_local, cap, rank)
        b = MO.schedule_ref_threads(topk_all, E_local, cap, rank)
        n = int(a[2])
        assert int(b[2]) == n and torch.equal(a[3], b[3]) and torch.equal(a[0], b[0])
        assert torch.equal(a[1][a[4]], b[1][a[4]])
        # every pair routed to a local expert appears exactly once, in its expert's segment
        local = (topk_all >= rank * E_local) & (topk_all < (rank + 1) * E_local)
        assert int(a[4].sum()) == int(local.sum())
        seg = torch.repeat_interleave(torch.arange(E_local), a[3].long())
        pr, pt = a[0][:n].long(), a[1][:n].long()
        valid = pr >= 0
        assert torch.equal(topk_all.view(W, -1)[pr[valid], pt[valid]].long() - rank * E_local, seg[valid])
        pairs = pr[valid] * (T * k) + pt[valid]
        assert pairs.unique().numel() == pairs.numel()

    check()
