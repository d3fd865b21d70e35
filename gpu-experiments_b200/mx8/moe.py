"""Host-side mirror of the reference's MoE bindings (forward, routed experts) on top of the C ABI.

The reference runs the whole forward as one persistent kernel; here it is a sequence of launches on
the current stream — dispatch+quantize, grouped GEMM (gate, up) with quantizing epilogue,
SwiGLU+quantize, grouped GEMM (down), combine — with the same inputs, outputs and tensor layouts.
Cross-rank ordering (tokens ready before dispatch, combine finished before the epilogue) is the
caller's barrier, exactly where the reference's harness has it
(blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.py:277-301).
"""
import ctypes

import torch

from . import _lib
from .ops import _FP8, _SC, _chk, _stream, gemm_bf16, gemm_grouped, swiglu_bf16, swiglu_bwd_bf16, transpose_bf16


def _ptr_array(ptrs):
    arr = (ctypes.c_void_p * len(ptrs))()
    for i, p in enumerate(ptrs):
        arr[i] = int(p)
    return arr


def dispatch_quantize(x_ptrs, hidden, topk, schedule_peer_rank, schedule_peer_token_idx, num_tokens, capacity=None):
    """Pull the routed token rows from every rank's token matrix (x_ptrs: list of device pointers,
    peer-mapped for other GPUs) and quantize them both ways.
    Returns (x_fp8 [cap, H], x_sc, x_fp8_t [H, cap], x_sc_t); rows beyond num_tokens are not written.
    Stands in for dispatch_quantize_kernel (blackwell-ultra/022-…-mxfp8-bw.cu:717-828)."""
    lib = _lib.load()
    cap = int(capacity if capacity is not None else schedule_peer_rank.numel())
    dev = schedule_peer_rank.device
    x_fp8 = torch.empty(cap, hidden, dtype=torch.float8_e4m3fn, device=dev)
    x_sc = torch.empty(cap // 128, hidden // 128, 32, 16, dtype=torch.uint8, device=dev)
    x_fp8_t = torch.empty(hidden, cap, dtype=torch.float8_e4m3fn, device=dev)
    x_sc_t = torch.empty(hidden // 128, cap // 128, 32, 16, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.mx8_moe_dispatch_quantize(
            _ptr_array(x_ptrs), len(x_ptrs), hidden, topk, _chk(schedule_peer_rank, "schedule_peer_rank", (torch.int32,)),
            _chk(schedule_peer_token_idx, "schedule_peer_token_idx", (torch.int32,)), _chk(num_tokens, "num_tokens", (torch.int32,)),
            cap, x_fp8.data_ptr(), x_sc.data_ptr(), x_fp8_t.data_ptr(), x_sc_t.data_ptr(), _stream()), "dispatch_quantize")
    return x_fp8, x_sc, x_fp8_t, x_sc_t


def swiglu_quantize(gate_fp8, gate_sc, up_fp8, up_sc, num_rows=None, return_bf16=False):
    """hidden = bf16(silu(dequant(gate)) * dequant(up)), re-quantized both ways.
    Returns (hidden_fp8, hidden_sc, hidden_fp8_t, hidden_sc_t[, hidden_bf16]).
    Stands in for swiglu_fwd<false> (blackwell-ultra/022-…-mxfp8-bw.cu:924-1129)."""
    lib = _lib.load()
    R, I = gate_fp8.shape
    dev = gate_fp8.device
    h_fp8 = torch.empty(R, I, dtype=torch.float8_e4m3fn, device=dev)
    h_sc = torch.empty(R // 128, I // 128, 32, 16, dtype=torch.uint8, device=dev)
    h_fp8_t = torch.empty(I, R, dtype=torch.float8_e4m3fn, device=dev)
    h_sc_t = torch.empty(I // 128, R // 128, 32, 16, dtype=torch.uint8, device=dev)
    h_bf16 = torch.empty(R, I, dtype=torch.bfloat16, device=dev) if return_bf16 else None
    with torch.cuda.device(dev):
        _lib.check(lib.mx8_swiglu_quantize(
            _chk(gate_fp8, "gate_fp8", _FP8), _chk(gate_sc, "gate_sc", _SC, (R // 128, I // 128, 512)),
            _chk(up_fp8, "up_fp8", _FP8, (R, I)), _chk(up_sc, "up_sc", _SC, (R // 128, I // 128, 512)), R, I,
            _chk(num_rows, "num_rows", (torch.int32,)) if num_rows is not None else None,
            h_fp8.data_ptr(), h_sc.data_ptr(), h_fp8_t.data_ptr(), h_sc_t.data_ptr(),
            h_bf16.data_ptr() if return_bf16 else None, _stream()), "swiglu_quantize")
    return (h_fp8, h_sc, h_fp8_t, h_sc_t) + ((h_bf16,) if return_bf16 else ())


def combine(y_routed, schedule_peer_rank, schedule_peer_token_idx, num_tokens, combine_buffer_ptrs):
    """Write every routed output row into the combine buffer of the rank that owns the token.
    Stands in for combine_kernel (blackwell-ultra/022-…-mxfp8-bw.cu:830-922)."""
    lib = _lib.load()
    with torch.cuda.device(y_routed.device):
        _lib.check(lib.mx8_moe_combine(
            _chk(y_routed, "y_routed", (torch.bfloat16,)), _chk(schedule_peer_rank, "schedule_peer_rank", (torch.int32,)),
            _chk(schedule_peer_token_idx, "schedule_peer_token_idx", (torch.int32,)), _chk(num_tokens, "num_tokens", (torch.int32,)),
            y_routed.shape[1], _ptr_array(combine_buffer_ptrs), len(combine_buffer_ptrs), _stream()), "combine")


def fwd_epilogue(y_shared, combine_buffer, topk_weights):
    """fwd_epilogue(y_shared, combine_buffer, topk_weights) -> output
    (blackwell-ultra/022-…-mxfp8-bw.cu:2842-2856, bound at :3029-3030).  y_shared may be None."""
    lib = _lib.load()
    T, k = topk_weights.shape
    H = combine_buffer.shape[1]
    out = torch.empty(T, H, dtype=torch.bfloat16, device=combine_buffer.device)
    with torch.cuda.device(combine_buffer.device):
        _lib.check(lib.mx8_moe_fwd_epilogue(
            _chk(y_shared, "y_shared", (torch.bfloat16,), (T, H)) if y_shared is not None else None,
            _chk(combine_buffer, "combine_buffer", (torch.bfloat16,), (T * k, H)),
            _chk(topk_weights, "topk_weights", (torch.float32,)), out.data_ptr(), T, H, k, _stream()), "fwd_epilogue")
    return out


_side_streams = {}
_trace = None       # set to a list to collect (name, start_event, end_event) of every launch of the pipelined layer


def _traced(name, stream, call):
    """run `call()` (one launch on `stream`); with tracing on, bracket it with timing events"""
    if _trace is None:
        return call()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    r = call()
    b.record(stream)
    _trace.append((name, a, b))
    return r



def _streams(dev):
    """two side streams per device for the transfer legs of the pipelined layer (created once)"""
    key = (dev.type, dev.index if dev.index is not None else torch.cuda.current_device())
    if key not in _side_streams:
        _side_streams[key] = (torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev))
    return _side_streams[key]


def _window(bounds, b, max_sms):
    return _lib.Window(bounds.data_ptr() + 4 * b, bounds.data_ptr() + 4 * (b + 1), int(max_sms))


def _routed_fwd_pipelined(x_ptrs, combine_buffer_ptrs, w_routed_gate, w_routed_gate_sc, w_routed_up, w_routed_up_sc,
                          w_routed_down, w_routed_down_sc, schedule_peer_rank, schedule_peer_token_idx, num_tokens,
                          tokens_per_expert, topk, num_comm_sms, minibatches):
    """Routed experts in `minibatches` groups of consecutive local experts.  Dispatch of group b+1 (on
    num_comm_sms multiprocessors, its own stream) and combine of group b-1 (a third stream; a plain copy
    kernel that shares multiprocessors with the GEMMs, held to num_comm_sms / 4 multiprocessors' worth of
    thread blocks: with more, its stores queue up in front of the NVLink ports and slow the GEMMs' operand
    traffic by as much as the overlap gains) run beside the GEMMs of group b, which keep the remaining
    multiprocessors.  Every kernel is the windowed form of the one the unsplit layer launches,
    so all outputs are bit-identical to it.  The stream-and-event counterpart of the reference's
    single-kernel task queue with communication SMs (blackwell-ultra/022-…-mxfp8-bw.cu:1738-2010)."""
    lib = _lib.load()
    E, I, H = w_routed_gate.shape
    cap = schedule_peer_rank.numel()
    dev = schedule_peer_rank.device
    nb = minibatches
    u8 = lambda *shape: torch.empty(*shape, dtype=torch.uint8, device=dev)
    f8 = lambda *shape: torch.empty(*shape, dtype=torch.float8_e4m3fn, device=dev)
    x_fp8, x_sc, x_fp8_t, x_sc_t = f8(cap, H), u8(cap // 128, H // 128, 32, 16), f8(H, cap), u8(H // 128, cap // 128, 32, 16)
    gate_fp8, gate_sc, up_fp8, up_sc = f8(cap, I), u8(cap // 128, I // 128, 32, 16), f8(cap, I), u8(cap // 128, I // 128, 32, 16)
    h_fp8, h_sc, h_fp8_t, h_sc_t = f8(cap, I), u8(cap // 128, I // 128, 32, 16), f8(I, cap), u8(I // 128, cap // 128, 32, 16)
    y_routed = torch.empty(cap, H, dtype=torch.bfloat16, device=dev)
    bounds = torch.empty(nb + 1, dtype=torch.int32, device=dev)
    xp, cp = _ptr_array(x_ptrs), _ptr_array(combine_buffer_ptrs)
    pr, pt, nt, tpe = (schedule_peer_rank.data_ptr(), schedule_peer_token_idx.data_ptr(), num_tokens.data_ptr(),
                       tokens_per_expert.data_ptr())
    wts = [(_chk(w, "w", _FP8), _chk(ws, "w_sc", _SC)) for w, ws in ((w_routed_gate, w_routed_gate_sc), (w_routed_up, w_routed_up_sc),
                                                                      (w_routed_down, w_routed_down_sc))]
    main = torch.cuda.current_stream(dev)
    s_disp, s_comb = _streams(dev)
    with torch.cuda.device(dev):
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        math_sms = max(2, (sms - num_comm_sms) & ~1)
        _lib.check(lib.mx8_moe_minibatch_bounds(tpe, E, nb, bounds.data_ptr(), main.cuda_stream), "minibatch_bounds")
        start = torch.cuda.Event()
        start.record(main)
        s_disp.wait_event(start)
        s_comb.wait_event(start)
        disp_done = []
        for b in range(nb):
            # the first group has the device to itself; later ones run beside the GEMMs
            w = _window(bounds, b, 0 if b == 0 else num_comm_sms)
            _traced("dispatch%d" % b, s_disp, lambda: _lib.check(lib.mx8_moe_dispatch_quantize_window(
                xp, len(x_ptrs), H, topk, pr, pt, nt, cap, x_fp8.data_ptr(), x_sc.data_ptr(), x_fp8_t.data_ptr(), x_sc_t.data_ptr(),
                ctypes.byref(w), s_disp.cuda_stream), "dispatch_quantize (window)"))
            ev = torch.cuda.Event()
            ev.record(s_disp)
            disp_done.append(ev)
        for b in range(nb):
            main.wait_event(disp_done[b])
            w = _window(bounds, b, 0 if b == nb - 1 else math_sms)
            wr = ctypes.byref(w)
            ms = main.cuda_stream
            _traced("gate%d" % b, main, lambda: _lib.check(lib.mx8_gemm_grouped_window(
                x_fp8.data_ptr(), x_sc.data_ptr(), wts[0][0], wts[0][1], gate_fp8.data_ptr(), gate_sc.data_ptr(), cap, I, H, _lib.C_MXFP8,
                nt, tpe, E, wr, ms), "gate gemm (window)"))
            _traced("up%d" % b, main, lambda: _lib.check(lib.mx8_gemm_grouped_window(
                x_fp8.data_ptr(), x_sc.data_ptr(), wts[1][0], wts[1][1], up_fp8.data_ptr(), up_sc.data_ptr(), cap, I, H, _lib.C_MXFP8,
                nt, tpe, E, wr, ms), "up gemm (window)"))
            _traced("swiglu%d" % b, main, lambda: _lib.check(lib.mx8_swiglu_quantize_window(
                gate_fp8.data_ptr(), gate_sc.data_ptr(), up_fp8.data_ptr(), up_sc.data_ptr(), cap, I, nt, h_fp8.data_ptr(), h_sc.data_ptr(),
                h_fp8_t.data_ptr(), h_sc_t.data_ptr(), None, wr, ms), "swiglu_quantize (window)"))
            _traced("down%d" % b, main, lambda: _lib.check(lib.mx8_gemm_grouped_window(
                h_fp8.data_ptr(), h_sc.data_ptr(), wts[2][0], wts[2][1], y_routed.data_ptr(), None, cap, H, I, _lib.C_BF16,
                nt, tpe, E, wr, ms), "down gemm (window)"))
            ev = torch.cuda.Event()
            ev.record(main)
            s_comb.wait_event(ev)
            wc = _window(bounds, b, max(1, num_comm_sms // 4) if b < nb - 1 else 0)
            _traced("combine%d" % b, s_comb, lambda: _lib.check(lib.mx8_moe_combine_window(
                y_routed.data_ptr(), pr, pt, nt, H, cp, len(combine_buffer_ptrs), ctypes.byref(wc), s_comb.cuda_stream), "combine (window)"))
        done = torch.cuda.Event()
        done.record(s_comb)
        main.wait_event(done)
    # the side streams used these tensors; tell the caching allocator so that it does not hand the
    # memory out again before their work has finished
    for t in (x_fp8, x_sc, x_fp8_t, x_sc_t, y_routed, bounds):
        t.record_stream(s_disp)
        t.record_stream(s_comb)
    return x_fp8, x_sc, x_fp8_t, x_sc_t, gate_fp8, gate_sc, up_fp8, up_sc, h_fp8, h_sc, h_fp8_t, h_sc_t, y_routed


def dispatch_mlp_swiglu_combine_fwd(x, x_ptrs, combine_buffer, combine_buffer_ptrs,
                                    w_shared_gate, w_routed_gate, w_routed_gate_sc,
                                    w_shared_up, w_routed_up, w_routed_up_sc,
                                    w_shared_down, w_routed_down, w_routed_down_sc,
                                    schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert,
                                    topk, num_comm_sms=0, macrobatch_size=0, minibatch_size=0, fuse_combine=False):
    """Same arguments and the same 13 return values as the reference's binding
    (blackwell-ultra/022-…-mxfp8-bw.cu:2016-2136, bound at :3001-3010):
      (x_fp8_t_routed, x_sc_t_routed, gate_shared, gate_fp8_routed, gate_sc_routed, up_shared,
       up_fp8_routed, up_sc_routed, hidden_shared, hidden_fp8_t_routed, hidden_sc_t_routed,
       y_shared, y_routed)
    Routed buffers have schedule_capacity rows.  With num_comm_sms > 0 and minibatch_size > 0 the routed
    experts run in ceil(capacity / minibatch_size) groups whose transfers overlap the other groups' GEMMs
    (see _routed_fwd_pipelined); with the defaults the layer is one launch sequence on the current stream.
    macrobatch_size (the backward's replay granularity in the reference) has no effect.  The shared expert (bf16, outside
    the MXFP8 path) runs on the bf16 form of the same GEMM kernel (gemm_bf16) when its weights are given, else
    those outputs are None.
    fuse_combine=True (an addition) lets the down projection's epilogue do the combine; y_routed is then None."""
    E, I, H = w_routed_gate.shape
    cap = schedule_peer_rank.numel()
    dev = x.device
    nb = min(E, -(-cap // minibatch_size)) if (minibatch_size > 0 and num_comm_sms > 0 and not fuse_combine) else 1
    if nb > 1:
        (x_fp8, x_sc, x_fp8_t, x_sc_t, gate_fp8, gate_sc, up_fp8, up_sc, h_fp8, h_sc, h_fp8_t, h_sc_t, y_routed) = _routed_fwd_pipelined(
            x_ptrs, combine_buffer_ptrs, w_routed_gate, w_routed_gate_sc, w_routed_up, w_routed_up_sc, w_routed_down, w_routed_down_sc,
            schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert, topk, num_comm_sms, nb)
        return (x_fp8_t, x_sc_t) + _shared_fwd(x, w_shared_gate, w_shared_up, w_shared_down, gate_fp8, gate_sc, up_fp8, up_sc,
                                                h_fp8_t, h_sc_t, y_routed)
    x_fp8, x_sc, x_fp8_t, x_sc_t = dispatch_quantize(x_ptrs, H, topk, schedule_peer_rank, schedule_peer_token_idx, num_tokens, cap)
    gate_fp8 = torch.empty(cap, I, dtype=torch.float8_e4m3fn, device=dev)
    gate_sc = torch.empty(cap // 128, I // 128, 32, 16, dtype=torch.uint8, device=dev)
    up_fp8 = torch.empty_like(gate_fp8)
    up_sc = torch.empty_like(gate_sc)
    gemm_grouped(x_fp8, x_sc, w_routed_gate, w_routed_gate_sc, gate_fp8, gate_sc, num_tokens, tokens_per_expert)
    gemm_grouped(x_fp8, x_sc, w_routed_up, w_routed_up_sc, up_fp8, up_sc, num_tokens, tokens_per_expert)
    h_fp8, h_sc, h_fp8_t, h_sc_t = swiglu_quantize(gate_fp8, gate_sc, up_fp8, up_sc, num_tokens)
    if fuse_combine:
        # the down projection's epilogue writes every row into its owner's combine buffer; y_routed is None
        y_routed = None
        lib = _lib.load()
        with torch.cuda.device(dev):
            _lib.check(lib.mx8_gemm_grouped_scatter(
                h_fp8.data_ptr(), h_sc.data_ptr(), _chk(w_routed_down, "w_routed_down", _FP8), _chk(w_routed_down_sc, "w_routed_down_sc", _SC),
                cap, H, I, num_tokens.data_ptr(), tokens_per_expert.data_ptr(), E, schedule_peer_rank.data_ptr(),
                schedule_peer_token_idx.data_ptr(), _ptr_array(combine_buffer_ptrs), len(combine_buffer_ptrs), _stream()),
                "grouped gemm + combine")
    else:
        y_routed = torch.empty(cap, H, dtype=torch.bfloat16, device=dev)
        gemm_grouped(h_fp8, h_sc, w_routed_down, w_routed_down_sc, y_routed, None, num_tokens, tokens_per_expert)
        combine(y_routed, schedule_peer_rank, schedule_peer_token_idx, num_tokens, combine_buffer_ptrs)
    return (x_fp8_t, x_sc_t) + _shared_fwd(x, w_shared_gate, w_shared_up, w_shared_down, gate_fp8, gate_sc, up_fp8, up_sc,
                                            h_fp8_t, h_sc_t, y_routed)


def _shared_fwd(x, w_shared_gate, w_shared_up, w_shared_down, gate_fp8, gate_sc, up_fp8, up_sc, h_fp8_t, h_sc_t, y_routed):
    """shared (bf16) expert, when its weights are given; returns outputs 2..12 of the forward binding"""
    gate_shared = up_shared = hidden_shared = y_shared = None
    if w_shared_gate is not None:
        dev = x.device
        Tl, Is, H = x.shape[0], w_shared_gate.shape[0], x.shape[1]
        gate_shared = gemm_bf16(x, w_shared_gate, torch.empty(Tl, Is, dtype=torch.bfloat16, device=dev))
        up_shared = gemm_bf16(x, w_shared_up, torch.empty(Tl, Is, dtype=torch.bfloat16, device=dev))
        hidden_shared = swiglu_bf16(gate_shared, up_shared)
        y_shared = gemm_bf16(hidden_shared, w_shared_down, torch.empty(Tl, H, dtype=torch.bfloat16, device=dev))
    return (gate_shared, gate_fp8, gate_sc, up_shared, up_fp8, up_sc, hidden_shared, h_fp8_t, h_sc_t, y_shared, y_routed)


# ------------------------------------------------------------------------------------------------
# backward (routed experts)
# ------------------------------------------------------------------------------------------------
def swiglu_bwd_quantize(gate_fp8, gate_sc, up_fp8, up_sc, d_hidden, which, num_rows=None, return_bf16=False):
    """Gradient of SwiGLU with respect to gate (which=0) or up (which=1), re-quantized both ways.
    Returns (fp8, sc, fp8_t, sc_t[, bf16])."""
    lib = _lib.load()
    R, I = gate_fp8.shape
    dev = gate_fp8.device
    o_fp8 = torch.empty(R, I, dtype=torch.float8_e4m3fn, device=dev)
    o_sc = torch.empty(R // 128, I // 128, 32, 16, dtype=torch.uint8, device=dev)
    o_fp8_t = torch.empty(I, R, dtype=torch.float8_e4m3fn, device=dev)
    o_sc_t = torch.empty(I // 128, R // 128, 32, 16, dtype=torch.uint8, device=dev)
    o_bf16 = torch.empty(R, I, dtype=torch.bfloat16, device=dev) if return_bf16 else None
    with torch.cuda.device(dev):
        _lib.check(lib.mx8_swiglu_bwd_quantize(
            _chk(gate_fp8, "gate_fp8", _FP8), _chk(gate_sc, "gate_sc", _SC, (R // 128, I // 128, 512)),
            _chk(up_fp8, "up_fp8", _FP8, (R, I)), _chk(up_sc, "up_sc", _SC, (R // 128, I // 128, 512)),
            _chk(d_hidden, "d_hidden", (torch.bfloat16,), (R, I)), R, I,
            _chk(num_rows, "num_rows", (torch.int32,)) if num_rows is not None else None, int(which),
            o_fp8.data_ptr(), o_sc.data_ptr(), o_fp8_t.data_ptr(), o_sc_t.data_ptr(),
            o_bf16.data_ptr() if return_bf16 else None, _stream()), "swiglu_bwd_quantize")
    return (o_fp8, o_sc, o_fp8_t, o_sc_t) + ((o_bf16,) if return_bf16 else ())


def swiglu_bwd_quantize_both(gate_fp8, gate_sc, up_fp8, up_sc, d_hidden, num_rows=None):
    """Both SwiGLU gradients from one pass over the inputs (mx8_swiglu_bwd_quantize_both); same bytes as two
    calls of swiglu_bwd_quantize.  Returns ((d_gate fp8, sc, fp8_t, sc_t), (d_up fp8, sc, fp8_t, sc_t))."""
    lib = _lib.load()
    R, I = gate_fp8.shape
    dev = gate_fp8.device

    def outs():
        return (torch.empty(R, I, dtype=torch.float8_e4m3fn, device=dev), torch.empty(R // 128, I // 128, 32, 16, dtype=torch.uint8, device=dev),
                torch.empty(I, R, dtype=torch.float8_e4m3fn, device=dev), torch.empty(I // 128, R // 128, 32, 16, dtype=torch.uint8, device=dev))
    dg, du = outs(), outs()
    with torch.cuda.device(dev):
        _lib.check(lib.mx8_swiglu_bwd_quantize_both(
            _chk(gate_fp8, "gate_fp8", _FP8), _chk(gate_sc, "gate_sc", _SC, (R // 128, I // 128, 512)),
            _chk(up_fp8, "up_fp8", _FP8, (R, I)), _chk(up_sc, "up_sc", _SC, (R // 128, I // 128, 512)),
            _chk(d_hidden, "d_hidden", (torch.bfloat16,), (R, I)), R, I,
            _chk(num_rows, "num_rows", (torch.int32,)) if num_rows is not None else None,
            *[t.data_ptr() for t in dg], *[t.data_ptr() for t in du], _stream()), "swiglu_bwd_quantize_both")
    return dg, du


def bwd_prologue(d_output, topk_weights, d_combine_buffer):
    """bwd_prologue(d_output, topk_weights, d_combine_buffer) -> d_y_shared (== d_output); fills
    d_combine_buffer[t*topk + j] = d_output[t] * w[t, j] in place
    (blackwell-ultra/022-…-mxfp8-bw.cu:2915-2923)."""
    lib = _lib.load()
    T, k = topk_weights.shape
    H = d_output.shape[1]
    with torch.cuda.device(d_output.device):
        _lib.check(lib.mx8_moe_bwd_prologue(_chk(d_output, "d_output", (torch.bfloat16,), (T, H)),
                                            _chk(topk_weights, "topk_weights", (torch.float32,)),
                                            _chk(d_combine_buffer, "d_combine_buffer", (torch.bfloat16,), (T * k, H)),
                                            T, H, k, _stream()), "bwd_prologue")
    return d_output


def bwd_epilogue(d_x_shared, d_x_routed_buffer):
    """bwd_epilogue(d_x_shared, d_x_routed_buffer) -> d_x = d_x_shared + sum over the topk rows of every
    token (blackwell-ultra/022-…-mxfp8-bw.cu:2982-2993).  d_x_shared may be None; then its shape is taken
    from `d_x_routed_buffer` and the `tokens` it was built for must divide its rows (pass topk via shape)."""
    raise_if = d_x_shared is None
    if raise_if:
        raise ValueError("bwd_epilogue needs d_x_shared (use bwd_epilogue_routed for the routed part alone)")
    return bwd_epilogue_routed(d_x_shared, d_x_routed_buffer, d_x_routed_buffer.shape[0] // d_x_shared.shape[0])


def bwd_epilogue_routed(d_x_shared, d_x_routed_buffer, topk):
    lib = _lib.load()
    H = d_x_routed_buffer.shape[1]
    T = d_x_routed_buffer.shape[0] // topk
    d_x = torch.empty(T, H, dtype=torch.bfloat16, device=d_x_routed_buffer.device)
    with torch.cuda.device(d_x.device):
        _lib.check(lib.mx8_moe_bwd_epilogue(
            _chk(d_x_shared, "d_x_shared", (torch.bfloat16,), (T, H)) if d_x_shared is not None else None,
            _chk(d_x_routed_buffer, "d_x_routed_buffer", (torch.bfloat16,), (T * topk, H)), d_x.data_ptr(), T, H, topk,
            _stream()), "bwd_epilogue")
    return d_x


def _routed_bwd_pipelined(d_combine_buffer_ptrs, d_x_routed_buffer_ptrs, w_routed_gate_T, w_routed_gate_T_sc, w_routed_up_T,
                          w_routed_up_T_sc, w_routed_down_T, w_routed_down_T_sc, gate_fp8_routed, gate_sc_routed, up_fp8_routed,
                          up_sc_routed, schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert,
                          num_comm_sms, minibatches):
    """Gradient dispatch, data-gradient GEMMs, SwiGLU backward and gradient combine in minibatches of
    experts on three streams, like _routed_fwd_pipelined; the weight-gradient GEMMs follow unsplit.
    Returns the tensors of the one-stream sequence, bit-identical to it."""
    lib = _lib.load()
    E, H, I = w_routed_gate_T.shape
    cap = schedule_peer_rank.numel()
    dev = schedule_peer_rank.device
    nb = minibatches
    u8 = lambda *shape: torch.empty(*shape, dtype=torch.uint8, device=dev)
    f8 = lambda *shape: torch.empty(*shape, dtype=torch.float8_e4m3fn, device=dev)
    quad = lambda r, c: (f8(r, c), u8(r // 128, c // 128, 32, 16), f8(c, r), u8(c // 128, r // 128, 32, 16))
    d_y = quad(cap, H)
    d_gate, d_up = quad(cap, I), quad(cap, I)
    d_hidden = torch.empty(cap, I, dtype=torch.bfloat16, device=dev)
    d_x_routed = torch.empty(cap, H, dtype=torch.bfloat16, device=dev)
    bounds = torch.empty(nb + 1, dtype=torch.int32, device=dev)
    src, dst = _ptr_array(d_combine_buffer_ptrs), _ptr_array(d_x_routed_buffer_ptrs)
    pr, pt, nt, tpe = (schedule_peer_rank.data_ptr(), schedule_peer_token_idx.data_ptr(), num_tokens.data_ptr(),
                       tokens_per_expert.data_ptr())
    wts = [(_chk(w, "w", _FP8), _chk(ws, "w_sc", _SC)) for w, ws in ((w_routed_gate_T, w_routed_gate_T_sc), (w_routed_up_T, w_routed_up_T_sc),
                                                                      (w_routed_down_T, w_routed_down_T_sc))]
    main = torch.cuda.current_stream(dev)
    s_disp, s_comb = _streams(dev)
    with torch.cuda.device(dev):
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        math_sms = max(2, (sms - num_comm_sms) & ~1)
        _lib.check(lib.mx8_moe_minibatch_bounds(tpe, E, nb, bounds.data_ptr(), main.cuda_stream), "minibatch_bounds")
        start = torch.cuda.Event()
        start.record(main)
        s_disp.wait_event(start)
        s_comb.wait_event(start)
        disp_done = []
        for b in range(nb):
            w = _window(bounds, b, 0 if b == 0 else num_comm_sms)
            # one gradient row per (token, k) pair, hence topk = 1 for the index
            _lib.check(lib.mx8_moe_dispatch_quantize_window(src, len(d_combine_buffer_ptrs), H, 1, pr, pt, nt, cap, d_y[0].data_ptr(),
                                                            d_y[1].data_ptr(), d_y[2].data_ptr(), d_y[3].data_ptr(), ctypes.byref(w),
                                                            s_disp.cuda_stream), "gradient dispatch (window)")
            ev = torch.cuda.Event()
            ev.record(s_disp)
            disp_done.append(ev)
        for b in range(nb):
            main.wait_event(disp_done[b])
            # the weight-gradient GEMMs follow the last group, so no group has the whole device for its data gradients
            w = _window(bounds, b, math_sms if b < nb - 1 else 0)
            wr, ms = ctypes.byref(w), main.cuda_stream
            _lib.check(lib.mx8_gemm_grouped_window(d_y[0].data_ptr(), d_y[1].data_ptr(), wts[2][0], wts[2][1], d_hidden.data_ptr(), None,
                                                   cap, I, H, _lib.C_BF16, nt, tpe, E, wr, ms), "d_hidden gemm (window)")
            _lib.check(lib.mx8_swiglu_bwd_quantize_both_window(
                _chk(gate_fp8_routed, "gate_fp8", _FP8), _chk(gate_sc_routed, "gate_sc", _SC), _chk(up_fp8_routed, "up_fp8", _FP8),
                _chk(up_sc_routed, "up_sc", _SC), d_hidden.data_ptr(), cap, I, nt, *[t.data_ptr() for t in d_gate],
                *[t.data_ptr() for t in d_up], wr, ms), "swiglu backward (window)")
            _lib.check(lib.mx8_gemm_grouped_dual_window(d_gate[0].data_ptr(), d_gate[1].data_ptr(), wts[0][0], wts[0][1], d_up[0].data_ptr(),
                                                        d_up[1].data_ptr(), wts[1][0], wts[1][1], d_x_routed.data_ptr(), cap, H, I, I,
                                                        nt, tpe, E, wr, ms), "data-gradient gemm (window)")
            ev = torch.cuda.Event()
            ev.record(main)
            s_comb.wait_event(ev)
            wc = _window(bounds, b, max(1, num_comm_sms // 4) if b < nb - 1 else 0)
            _lib.check(lib.mx8_moe_combine_window(d_x_routed.data_ptr(), pr, pt, nt, H, dst, len(d_x_routed_buffer_ptrs), ctypes.byref(wc),
                                                  s_comb.cuda_stream), "gradient combine (window)")
        done = torch.cuda.Event()
        done.record(s_comb)
    for t in d_y + (d_x_routed, bounds):
        t.record_stream(s_disp)
        t.record_stream(s_comb)
    return d_y, d_hidden, d_gate, d_up, d_x_routed, done


def dispatch_mlp_swiglu_combine_bwd(d_y_shared, d_combine_buffer, d_combine_buffer_ptrs, d_x_routed_buffer, d_x_routed_buffer_ptrs,
                                    w_shared_gate_T, w_routed_gate_T, w_routed_gate_T_sc,
                                    w_shared_up_T, w_routed_up_T, w_routed_up_T_sc,
                                    w_shared_down_T, w_routed_down_T, w_routed_down_T_sc,
                                    x_fp8_t_routed, x_sc_t_routed,
                                    gate_shared, gate_fp8_routed, gate_sc_routed,
                                    up_shared, up_fp8_routed, up_sc_routed,
                                    hidden_shared, hidden_fp8_t_routed, hidden_sc_t_routed,
                                    x_buffer, x_buffer_ptrs,
                                    w_routed_gate, w_routed_gate_sc, w_routed_up, w_routed_up_sc,
                                    schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert,
                                    topk, num_comm_sms=0, macrobatch_size=0, minibatch_size=0):
    """Same arguments and the same 18 return values as the reference's backward binding
    (blackwell-ultra/022-…-mxfp8-bw.cu:2556-2760, bound at :3011-3028):
      (d_x_shared, d_x_routed, d_gate_shared, d_gate_fp8_routed, d_gate_sc_routed, d_up_shared,
       d_up_fp8_routed, d_up_sc_routed, d_hidden_shared, d_hidden_routed, d_y_routed_fp8_routed,
       d_y_routed_sc_routed, d_w_shared_gate, d_w_routed_gate, d_w_shared_up, d_w_routed_up,
       d_w_shared_down, d_w_routed_down)
    The routed part runs on the MXFP8 kernels; it uses the transposed activations the forward returned
    (x_fp8_t_routed, hidden_fp8_t_routed), so the arguments the reference needs only to replay its
    forward (x_buffer, x_buffer_ptrs, w_routed_gate/up) are accepted and unused.  The shared expert
    (bf16) runs on gemm_bf16 / swiglu_bwd_bf16 when its inputs are given, else those outputs are None."""
    E, H, I = w_routed_gate_T.shape                      # transposed weights: [E, H, I]
    cap = schedule_peer_rank.numel()
    dev = d_combine_buffer.device
    from .ops import gemm_grouped_dual, gemm_wgrad
    nb = min(E, -(-cap // minibatch_size)) if (minibatch_size > 0 and num_comm_sms > 0) else 1
    combine_done = None
    if nb > 1:
        ((d_y_fp8, d_y_sc, d_y_fp8_t, d_y_sc_t), d_hidden, (d_gate_fp8, d_gate_sc, d_gate_fp8_t, d_gate_sc_t),
         (d_up_fp8, d_up_sc, d_up_fp8_t, d_up_sc_t), d_x_routed, combine_done) = _routed_bwd_pipelined(
            d_combine_buffer_ptrs, d_x_routed_buffer_ptrs, w_routed_gate_T, w_routed_gate_T_sc, w_routed_up_T, w_routed_up_T_sc,
            w_routed_down_T, w_routed_down_T_sc, gate_fp8_routed, gate_sc_routed, up_fp8_routed, up_sc_routed,
            schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert, num_comm_sms, nb)
    else:
        # gradient rows of the routed outputs, pulled from the owners' buffers (one row per (token, k) pair)
        d_y_fp8, d_y_sc, d_y_fp8_t, d_y_sc_t = dispatch_quantize(d_combine_buffer_ptrs, H, 1, schedule_peer_rank,
                                                                   schedule_peer_token_idx, num_tokens, cap)
        d_hidden = torch.empty(cap, I, dtype=torch.bfloat16, device=dev)
        gemm_grouped(d_y_fp8, d_y_sc, w_routed_down_T, w_routed_down_T_sc, d_hidden, None, num_tokens, tokens_per_expert)
        (d_gate_fp8, d_gate_sc, d_gate_fp8_t, d_gate_sc_t), (d_up_fp8, d_up_sc, d_up_fp8_t, d_up_sc_t) = swiglu_bwd_quantize_both(
            gate_fp8_routed, gate_sc_routed, up_fp8_routed, up_sc_routed, d_hidden, num_tokens)
        d_x_routed = torch.empty(cap, H, dtype=torch.bfloat16, device=dev)
        gemm_grouped_dual(d_gate_fp8, d_gate_sc, w_routed_gate_T, w_routed_gate_T_sc, d_up_fp8, d_up_sc, w_routed_up_T,
                          w_routed_up_T_sc, d_x_routed, num_tokens, tokens_per_expert)
        combine(d_x_routed, schedule_peer_rank, schedule_peer_token_idx, num_tokens, d_x_routed_buffer_ptrs)
    d_w_gate = torch.empty(E, I, H, dtype=torch.bfloat16, device=dev)
    d_w_up = torch.empty(E, I, H, dtype=torch.bfloat16, device=dev)
    d_w_down = torch.empty(E, H, I, dtype=torch.bfloat16, device=dev)
    gemm_wgrad(d_gate_fp8_t, d_gate_sc_t, x_fp8_t_routed, x_sc_t_routed, d_w_gate, tokens_per_expert)
    gemm_wgrad(d_up_fp8_t, d_up_sc_t, x_fp8_t_routed, x_sc_t_routed, d_w_up, tokens_per_expert)
    gemm_wgrad(d_y_fp8_t, d_y_sc_t, hidden_fp8_t_routed, hidden_sc_t_routed, d_w_down, tokens_per_expert)
    if combine_done is not None:
        torch.cuda.current_stream(dev).wait_event(combine_done)     # the last gradient combine ran beside the weight gradients
    d_x_shared = d_gate_shared = d_up_shared = d_hidden_shared = d_w_sg = d_w_su = d_w_sd = None
    if w_shared_gate_T is not None and d_y_shared is not None:
        x = x_buffer
        Tl, Hs, Is = d_y_shared.shape[0], d_y_shared.shape[1], gate_shared.shape[1]
        mk = lambda r, c: torch.empty(r, c, dtype=torch.bfloat16, device=dev)
        d_hidden_shared = gemm_bf16(d_y_shared, w_shared_down_T, mk(Tl, Is))
        d_gate_shared, d_up_shared = swiglu_bwd_bf16(d_hidden_shared, gate_shared, up_shared)
        # dgrad: two products accumulated in one tile pass
        d_x_shared = gemm_bf16(d_gate_shared, w_shared_gate_T, mk(Tl, Hs), d_up_shared, w_shared_up_T)
        # wgrad: K runs over the tokens, so both operands are transposed to K-major first
        x_t = transpose_bf16(x)
        d_w_sg = gemm_bf16(transpose_bf16(d_gate_shared), x_t, mk(Is, Hs))
        d_w_su = gemm_bf16(transpose_bf16(d_up_shared), x_t, mk(Is, Hs))
        d_w_sd = gemm_bf16(transpose_bf16(d_y_shared), transpose_bf16(hidden_shared), mk(Hs, Is))
    return (d_x_shared, d_x_routed, d_gate_shared, d_gate_fp8, d_gate_sc, d_up_shared, d_up_fp8, d_up_sc,
            d_hidden_shared, d_hidden, d_y_fp8, d_y_sc, d_w_sg, d_w_gate, d_w_su, d_w_up, d_w_sd, d_w_down)
