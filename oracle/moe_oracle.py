"""CPU oracle for the expert-parallel MoE layer built on the MXFP8 path.  TEST INFRASTRUCTURE ONLY
(same rules as mx8_oracle.py: imported by tests, the smoke check and the benchmark's CPU leg only).

Parity status: the quantize and GEMM pieces are pinned through mx8_oracle.py.  The expert MLP (routed
and shared, forward and backward) is pinned by tests/golden/moe_fwd_bwd.npz, which
tests/golden/make_golden.py produces by executing the reference harness's own mlp_swiglu_fwd_ref /
mlp_swiglu_bwd_ref on CPU (with its GPU-only block-scaled GEMM wrapper bound to dequantize -> fp32
product); tests/test_oracle_moe.py requires the functions below to reproduce it.  The routing schedule is
a transcription of the reference's CUDA kernels, which cannot run here; it is checked against a
thread-by-thread execution of the same kernel source logic, not against reference output.  They follow

* schedule ............ blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.cu:34-147
* routed forward ...... blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.py:91-126
* dispatch / combine .. blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.py:386-411
* forward epilogue .... blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.cu:2789-2840
"""
from __future__ import annotations

import numpy as np
import torch

from . import mx8_oracle as O

PAD = 256


SCHED_THREADS = 1024   # scheduler::config::NUM_THREADS, ...-mxfp8-bw.cu:15


def schedule_ref(topk_all: torch.Tensor, num_local_experts: int, capacity: int, rank: int):
    """topk_all int32 [W, T, k] -> (peer_rank[capacity], peer_token_idx[capacity], num_tokens[1],
    tokens_per_expert[E], written[capacity]).

    Transcription of the reference's three scheduler kernels (...-mxfp8-bw.cu:34-147), with the thread
    loops of its placement kernel (:99-146) written out as array operations over a [rows, 1024] view of
    a rank's table: block (expert, peer) has 1024 threads; thread t visits entries t, t + 1024, ...
    (:108, :133); its first hit takes the ordinal `exclusive prefix over threads of the hit counts`
    (:112-131) and later hits of the same thread the following ordinals (:145); ordinal j of peer r
    lands on row base + sum_q min(n_q, j) + #{q < r : n_q > j} (:136-141).  Segments are padded to 256
    rows (:68-71).  `schedule_ref_threads` below is the same thing as plain loops, for small cases."""
    W, T, k = topk_all.shape
    stride = T * k
    flat = topk_all.reshape(W, stride).numpy()
    rows = (stride + SCHED_THREADS - 1) // SCHED_THREADS
    peer_rank = np.full(capacity, -1, np.int32)
    peer_tok = np.zeros(capacity, np.int32)
    tpe = np.zeros(num_local_experts, np.int32)
    written = np.zeros(capacity, bool)
    entry = np.arange(rows * SCHED_THREADS, dtype=np.int64).reshape(rows, SCHED_THREADS)
    base = 0
    for e in range(num_local_experts):
        g = rank * num_local_experts + e
        hits = np.zeros((W, rows * SCHED_THREADS), bool)
        hits[:, :stride] = flat == g
        hits = hits.reshape(W, rows, SCHED_THREADS)
        n_from = hits.sum(axis=(1, 2))                                   # count_kernel
        for r in range(W):
            h = hits[r]
            per_thread = h.sum(axis=0)
            first = np.cumsum(per_thread) - per_thread                   # exclusive prefix over threads
            j = first[None, :] + np.cumsum(h, axis=0) - h                # ordinal of every entry that hits
            jj = j[h]
            dst = base + np.minimum(n_from[None, :], jj[:, None]).sum(axis=1) \
                + (n_from[None, :r] > jj[:, None]).sum(axis=1)
            ok = dst < capacity
            peer_rank[dst[ok]] = r
            peer_tok[dst[ok]] = entry[h][ok]
            written[dst[ok]] = True
        tpe[e] = (int(n_from.sum()) + PAD - 1) // PAD * PAD               # pad_kernel
        base += int(tpe[e])
    return (torch.from_numpy(peer_rank), torch.from_numpy(peer_tok), torch.tensor([base], dtype=torch.int32),
            torch.from_numpy(tpe), torch.from_numpy(written))


def schedule_ref_threads(topk_all: torch.Tensor, num_local_experts: int, capacity: int, rank: int):
    """The reference's placement kernel executed thread by thread in plain Python (small cases only):
    one pass per block (expert, peer) in which every thread counts its hits, then one in which it
    places them.  Same outputs as schedule_ref without `written`."""
    W, T, k = topk_all.shape
    stride = T * k
    flat = topk_all.reshape(W, stride).tolist()
    first_expert = rank * num_local_experts
    n_ep = [[0] * W for _ in range(num_local_experts)]
    for r in range(W):
        for v in flat[r]:
            if first_expert <= v < first_expert + num_local_experts:
                n_ep[v - first_expert][r] += 1
    tpe = [(sum(n_ep[e]) + PAD - 1) // PAD * PAD for e in range(num_local_experts)]
    peer_rank = [-1] * capacity
    peer_tok = [0] * capacity
    for e in range(num_local_experts):
        expert_base = sum(tpe[:e])
        for r in range(W):
            counts = [0] * SCHED_THREADS
            for t in range(SCHED_THREADS):
                for i in range(t, stride, SCHED_THREADS):
                    counts[t] += 1 if flat[r][i] - first_expert == e else 0
            j_of = [0] * SCHED_THREADS
            for t in range(1, SCHED_THREADS):
                j_of[t] = j_of[t - 1] + counts[t - 1]
            for t in range(SCHED_THREADS):
                j = j_of[t]
                for i in range(t, stride, SCHED_THREADS):
                    if flat[r][i] - first_expert == e:
                        dst = expert_base
                        for q in range(W):
                            dst += min(n_ep[e][q], j) + (1 if q < r and n_ep[e][q] > j else 0)
                        if dst < capacity:
                            peer_rank[dst] = r
                            peer_tok[dst] = i
                        j += 1
    return (torch.tensor(peer_rank, dtype=torch.int32), torch.tensor(peer_tok, dtype=torch.int32),
            torch.tensor([sum(tpe)], dtype=torch.int32), torch.tensor(tpe, dtype=torch.int32))


def route(logits: torch.Tensor, k: int):
    """The reference's router: top-k of the logits, softmax over the selected k values
    (blackwell-ultra/022-…-mxfp8-bw.py:270-272)."""
    vals, ids = torch.topk(logits, k, dim=1)
    return ids.to(torch.int32), torch.softmax(vals.float(), dim=-1)


def dispatch_ref(x_all: torch.Tensor, peer_rank, peer_tok, num_tokens: int, k: int) -> torch.Tensor:
    """x_all bf16 [W, T, H] -> x_routed bf16 [num_tokens, H]; padding rows are zero."""
    H = x_all.shape[-1]
    out = torch.zeros(num_tokens, H, dtype=torch.bfloat16)
    pr = peer_rank[:num_tokens].long()
    valid = pr >= 0
    out[valid] = x_all[pr[valid], (peer_tok[:num_tokens].long()[valid]) // k]
    return out


def swiglu_ref(gate_q, gate_sc_tiles, up_q, up_sc_tiles) -> torch.Tensor:
    """hidden = bf16( silu(dequant(gate)) * dequant(up) ), fp32 arithmetic; the dequantized values
    pass through bf16 first, as in the reference's `dequant` (…-mxfp8-bw.py:68-72, 120-122)."""
    g = O.dequantize(gate_q, O.scale_unswizzle(gate_sc_tiles)).to(torch.bfloat16).float()
    u = O.dequantize(up_q, O.scale_unswizzle(up_sc_tiles)).to(torch.bfloat16).float()
    return ((g / (1.0 + torch.exp(-g))) * u).to(torch.bfloat16)


def expert_mlp_ref(x_routed, tokens_per_expert, wg, wu, wd):
    """Routed-expert forward on already dispatched rows.  wg/wu: (fp8 [E, I, H], scale tiles
    [E*I/128, H/128, 512]); wd: (fp8 [E, H, I], scale tiles [E*H/128, I/128, 512]).
    Returns a dict of every intermediate the CUDA path emits."""
    (wg_q, wg_sc), (wu_q, wu_sc), (wd_q, wd_sc) = wg, wu, wd
    E, I, H = wg_q.shape
    R = x_routed.shape[0]
    xq, xsc, xqt, xsct = O.quantize_both(x_routed)
    gate_q = torch.zeros(R, I, dtype=torch.uint8)
    up_q = torch.zeros(R, I, dtype=torch.uint8)
    gate_sc = torch.zeros(R // 128, I // 128, 32, 16, dtype=torch.uint8)
    up_sc = torch.zeros_like(gate_sc)
    hidden = torch.zeros(R, I, dtype=torch.bfloat16)
    y = torch.zeros(R, H, dtype=torch.bfloat16)
    off = 0
    for e, n in enumerate(tokens_per_expert.tolist()):
        if n == 0:
            continue
        rows = slice(off, off + n)
        tiles = slice(off // 128, (off + n) // 128)
        g = O.gemm_ref(xq[rows], xsc[tiles], wg_q[e], wg_sc[e * I // 128:(e + 1) * I // 128])
        u = O.gemm_ref(xq[rows], xsc[tiles], wu_q[e], wu_sc[e * I // 128:(e + 1) * I // 128])
        gate_q[rows], gate_sc[tiles] = O.quantize_tiled(g)
        up_q[rows], up_sc[tiles] = O.quantize_tiled(u)
        hidden[rows] = swiglu_ref(gate_q[rows], gate_sc[tiles], up_q[rows], up_sc[tiles])
        off += n
    hq, hsc, hqt, hsct = O.quantize_both(hidden)
    off = 0
    for e, n in enumerate(tokens_per_expert.tolist()):
        if n == 0:
            continue
        rows = slice(off, off + n)
        tiles = slice(off // 128, (off + n) // 128)
        y[rows] = O.gemm_ref(hq[rows], hsc[tiles], wd_q[e], wd_sc[e * H // 128:(e + 1) * H // 128])
        off += n
    return dict(x_fp8=xq, x_sc=xsc, x_fp8_t=xqt, x_sc_t=xsct, gate_fp8=gate_q, gate_sc=gate_sc, up_fp8=up_q, up_sc=up_sc,
                hidden=hidden, hidden_fp8=hq, hidden_sc=hsc, hidden_fp8_t=hqt, hidden_sc_t=hsct, y=y)


def combine_ref(y_routed_by_rank, peer_rank_by_rank, peer_tok_by_rank, owner: int, T: int, k: int) -> torch.Tensor:
    """combine_buffer [T*k, H] of rank `owner`: row peer_token_idx receives the expert output row."""
    H = y_routed_by_rank[0].shape[-1]
    buf = torch.zeros(T * k, H, dtype=torch.bfloat16)
    for dst in range(len(y_routed_by_rank)):
        n = y_routed_by_rank[dst].shape[0]
        sel = peer_rank_by_rank[dst][:n] == owner
        buf[peer_tok_by_rank[dst][:n][sel].long()] = y_routed_by_rank[dst][sel]
    return buf


def fwd_epilogue_ref(y_shared, combine_buffer, topk_weights) -> torch.Tensor:
    """out[t] = bf16( y_shared[t] + sum_j w[t, j] * combine[t*k + j] ), fp32, products and sums
    rounded separately, j ascending."""
    T, k = topk_weights.shape
    acc = y_shared.float().clone()
    cb = combine_buffer.float().view(T, k, -1)
    for j in range(k):
        acc = acc + cb[:, j] * topk_weights[:, j:j + 1].float()
    return acc.to(torch.bfloat16)


# --------------------------------------------------------------------------------------
# backward (routed experts), following blackwell-ultra/022-…-mxfp8-bw.py:129-215
# --------------------------------------------------------------------------------------
def bwd_prologue_ref(d_output, topk_weights):
    """d_combine[t*k + j] = bf16(d_output[t] * w[t, j])."""
    T, k = topk_weights.shape
    return (d_output.float().unsqueeze(1) * topk_weights.float().unsqueeze(2)).to(torch.bfloat16).reshape(T * k, -1)


def swiglu_bwd_ref(gate_q, gate_sc_tiles, up_q, up_sc_tiles, d_hidden):
    """(d_gate, d_up) in bf16 (…-mxfp8-bw.py:167-171)."""
    g = O.dequantize(gate_q, O.scale_unswizzle(gate_sc_tiles)).to(torch.bfloat16).float()
    u = O.dequantize(up_q, O.scale_unswizzle(up_sc_tiles)).to(torch.bfloat16).float()
    sig = 1.0 / (1.0 + torch.exp(-g))
    silu = g * sig
    d_silu = (1.0 - silu) * sig + silu
    dh = d_hidden.float()
    return ((d_silu * u) * dh).to(torch.bfloat16), (silu * dh).to(torch.bfloat16)


def expert_mlp_bwd_ref(d_y_routed, fwd, tokens_per_expert, wg_T, wu_T, wd_T):
    """Routed-expert backward.  d_y_routed bf16 [R, H] (already dispatched); fwd = the dict returned by
    expert_mlp_ref; w*_T = (fp8, scale tiles) of the transposed weights: gate/up [E, H, I], down [E, I, H]."""
    (wg_q, wg_sc), (wu_q, wu_sc), (wd_q, wd_sc) = wg_T, wu_T, wd_T
    E, H, I = wg_q.shape
    R = d_y_routed.shape[0]
    dyq, dysc, dyqt, dysct = O.quantize_both(d_y_routed)
    d_hidden = torch.zeros(R, I, dtype=torch.bfloat16)
    segs, off = [], 0
    for e, n in enumerate(tokens_per_expert.tolist()):
        segs.append((e, off, n))
        off += n
    for e, off, n in segs:
        if n:
            rows, tiles = slice(off, off + n), slice(off // 128, (off + n) // 128)
            d_hidden[rows] = O.gemm_ref(dyq[rows], dysc[tiles], wd_q[e], wd_sc[e * I // 128:(e + 1) * I // 128])
    d_gate, d_up = swiglu_bwd_ref(fwd["gate_fp8"], fwd["gate_sc"], fwd["up_fp8"], fwd["up_sc"], d_hidden)
    dgq, dgsc, dgqt, dgsct = O.quantize_both(d_gate)
    duq, dusc, duqt, dusct = O.quantize_both(d_up)
    d_x = torch.zeros(R, H, dtype=torch.bfloat16)
    for e, off, n in segs:
        if n:
            rows, tiles = slice(off, off + n), slice(off // 128, (off + n) // 128)
            hs = slice(e * H // 128, (e + 1) * H // 128)
            # one product over the concatenated K dimension [d_gate | d_up] x [Wg^T | Wu^T] (…-mxfp8-bw.py:178-186)
            a = torch.cat((O.dequantize(dgq[rows], O.scale_unswizzle(dgsc[tiles])),
                           O.dequantize(duq[rows], O.scale_unswizzle(dusc[tiles]))), 1)
            b = torch.cat((O.dequantize(wg_q[e], O.scale_unswizzle(wg_sc[hs])), O.dequantize(wu_q[e], O.scale_unswizzle(wu_sc[hs]))), 1)
            d_x[rows] = (a @ b.t()).to(torch.bfloat16)
    deq_t = lambda q, sc: O.dequantize(q, O.scale_unswizzle(sc))          # [cols, R]
    dg_t, du_t, dy_t = deq_t(dgqt, dgsct), deq_t(duqt, dusct), deq_t(dyqt, dysct)
    x_t, h_t = deq_t(fwd["x_fp8_t"], fwd["x_sc_t"]), deq_t(fwd["hidden_fp8_t"], fwd["hidden_sc_t"])
    d_wg = torch.zeros(E, I, H, dtype=torch.bfloat16)
    d_wu = torch.zeros(E, I, H, dtype=torch.bfloat16)
    d_wd = torch.zeros(E, H, I, dtype=torch.bfloat16)
    for e, off, n in segs:
        if n:
            c = slice(off, off + n)
            d_wg[e] = (dg_t[:, c] @ x_t[:, c].t()).to(torch.bfloat16)
            d_wu[e] = (du_t[:, c] @ x_t[:, c].t()).to(torch.bfloat16)
            d_wd[e] = (dy_t[:, c] @ h_t[:, c].t()).to(torch.bfloat16)
    return dict(d_y_fp8=dyq, d_y_sc=dysc, d_hidden=d_hidden, d_gate=d_gate, d_up=d_up, d_gate_fp8=dgq, d_gate_sc=dgsc,
                d_up_fp8=duq, d_up_sc=dusc, d_x=d_x, d_w_gate=d_wg, d_w_up=d_wu, d_w_down=d_wd)


def bwd_epilogue_ref(d_x_shared, d_x_routed_buffer, k):
    T = d_x_routed_buffer.shape[0] // k
    acc = d_x_shared.float().clone() if d_x_shared is not None else torch.zeros(T, d_x_routed_buffer.shape[1])
    rb = d_x_routed_buffer.float().view(T, k, -1)
    for j in range(k):
        acc = acc + rb[:, j]
    return acc.to(torch.bfloat16)


def shared_mlp_ref(x, w_gate, w_up, w_down):
    """Shared (bf16) expert forward: gate = x Wg^T, up = x Wu^T, hidden = bf16(silu(gate) * up) in fp32,
    y = hidden Wd^T; every GEMM accumulates in fp32 and rounds to bf16
    (blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.py:98-102).
    Returns (gate, up, hidden, y)."""
    mm = lambda a, b: (a.float() @ b.float().t()).to(torch.bfloat16)
    gate, up = mm(x, w_gate), mm(x, w_up)
    g = gate.float()
    hidden = ((g / (torch.exp(-g) + 1.0)) * up.float()).to(torch.bfloat16)
    return gate, up, hidden, mm(hidden, w_down)


def shared_mlp_bwd_ref(d_y, x, gate, up, hidden, w_gate, w_up, w_down):
    """Shared expert backward (blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.py:141-151).
    Weights in forward orientation: w_gate, w_up [I, H], w_down [H, I].
    Returns (d_x, d_gate, d_up, d_hidden, d_w_gate, d_w_up, d_w_down)."""
    f = lambda t: t.float()
    bf = lambda t: t.to(torch.bfloat16)
    d_hidden = d_y @ w_down                                  # bf16 products with fp32 accumulation, as in the reference
    den = torch.exp(-f(gate)) + 1.0
    silu = f(gate) / den
    d_silu = (1.0 - silu) / den + silu
    d_gate = bf((f(d_hidden) * d_silu) * f(up))
    d_up = bf(silu * f(d_hidden))
    d_x = torch.cat((d_gate, d_up), 1) @ torch.cat((w_gate, w_up), 0)
    return d_x, d_gate, d_up, d_hidden, d_gate.t() @ x, d_up.t() @ x, d_y.t() @ hidden
