"""Host-side mirror of the reference's MoE bindings on top of the C ABI.

The reference runs the forward (and the backward) as one persistent kernel; behind the C ABI it is one call,
mx8_moe_fwd (mx8_moe_bwd), that queues dispatch+quantize, grouped GEMMs (gate, up) with quantizing epilogue,
SwiGLU+quantize, grouped GEMM (down) and combine, in minibatches on three streams when the reference's
num_comm_sms / minibatch_size arguments ask for it, with the same inputs, outputs and tensor layouts.  This
module only allocates the outputs and the workspace and checks arguments.  Cross-rank ordering (tokens ready
before dispatch, combine finished before the epilogue) is the caller's barrier, exactly where the reference's
harness has it (blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.py:277-301).
"""
import ctypes

import torch

from . import _lib
from .ops import _FP8, _SC, _chk, _stream


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


def combine(y_routed, schedule_peer_rank, schedule_peer_token_idx, num_tokens, combine_buffer_ptrs, combine_rows):
    """Write every routed output row into the combine buffer of the rank that owns the token; combine_rows =
    rows of every rank's buffer (tokens * topk).  Stands in for combine_kernel
    (blackwell-ultra/022-…-mxfp8-bw.cu:830-922)."""
    lib = _lib.load()
    with torch.cuda.device(y_routed.device):
        _lib.check(lib.mx8_moe_combine(
            _chk(y_routed, "y_routed", (torch.bfloat16,)), _chk(schedule_peer_rank, "schedule_peer_rank", (torch.int32,)),
            _chk(schedule_peer_token_idx, "schedule_peer_token_idx", (torch.int32,)), _chk(num_tokens, "num_tokens", (torch.int32,)),
            min(y_routed.shape[0], schedule_peer_rank.numel()), y_routed.shape[1], _ptr_array(combine_buffer_ptrs),
            len(combine_buffer_ptrs), int(combine_rows), _stream()), "combine")


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


def _dims(world, tokens, hidden, intermediate, shared_intermediate, experts, topk, capacity, num_comm_sms, minibatch_size, tuning):
    d = _lib.MoeDims(world=world, tokens=tokens, hidden=hidden, intermediate=intermediate, shared_intermediate=shared_intermediate,
                     num_local_experts=experts, topk=topk, capacity=capacity, num_comm_sms=int(num_comm_sms),
                     minibatch_size=int(minibatch_size))
    for key, val in (tuning or {}).items():
        setattr(d, key, int(val))
    return d


_workspaces = {}


def _workspace(dev, nbytes):
    """one grow-only workspace per device: the layer's internal tensors live here between the launches of a call"""
    key = (dev.type, dev.index if dev.index is not None else torch.cuda.current_device())
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        _workspaces[key] = ws
    return ws


def _opt(t, name, dtypes, shape=None):
    return _chk(t, name, dtypes, shape) if t is not None else None


def dispatch_mlp_swiglu_combine_fwd(x, x_ptrs, combine_buffer, combine_buffer_ptrs,
                                    w_shared_gate, w_routed_gate, w_routed_gate_sc,
                                    w_shared_up, w_routed_up, w_routed_up_sc,
                                    w_shared_down, w_routed_down, w_routed_down_sc,
                                    schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert,
                                    topk, num_comm_sms=0, macrobatch_size=0, minibatch_size=0, fuse_combine=False, tuning=None):
    """Same arguments and the same 13 return values as the reference's binding
    (blackwell-ultra/022-…-mxfp8-bw.cu:2016-2136, bound at :3001-3010):
      (x_fp8_t_routed, x_sc_t_routed, gate_shared, gate_fp8_routed, gate_sc_routed, up_shared,
       up_fp8_routed, up_sc_routed, hidden_shared, hidden_fp8_t_routed, hidden_sc_t_routed,
       y_shared, y_routed)
    Routed buffers have schedule_capacity rows.  With num_comm_sms > 0 and minibatch_size > 0 the routed
    experts run in ceil(capacity / minibatch_size) minibatches whose transfers overlap the other minibatches'
    GEMMs (mx8_moe_fwd); with the defaults the layer is one launch sequence on the current stream.
    macrobatch_size (the backward's replay granularity in the reference) has no effect.  The shared expert
    (bf16) runs when its weights are given, else those outputs are None.
    fuse_combine=True (an addition) lets the down projection's epilogue do the combine; y_routed is then None.
    tuning (an addition): dict of mx8_moe_dims fields minibatches / ramp / combine_sms / combine_own_sms."""
    lib = _lib.load()
    E, I, H = w_routed_gate.shape
    cap = schedule_peer_rank.numel()
    T = x.shape[0]
    dev = x.device
    shared = w_shared_gate is not None and w_shared_up is not None and w_shared_down is not None
    Is = w_shared_gate.shape[0] if shared else 0
    d = _dims(len(x_ptrs), T, H, I, Is, E, topk, cap, num_comm_sms, minibatch_size, tuning)
    u8 = lambda *shape: torch.empty(*shape, dtype=torch.uint8, device=dev)
    f8 = lambda *shape: torch.empty(*shape, dtype=torch.float8_e4m3fn, device=dev)
    bf = lambda *shape: torch.empty(*shape, dtype=torch.bfloat16, device=dev)
    out = dict(x_fp8_t=f8(H, cap), x_sc_t=u8(H // 128, cap // 128, 32, 16), gate_fp8=f8(cap, I), gate_sc=u8(cap // 128, I // 128, 32, 16),
               up_fp8=f8(cap, I), up_sc=u8(cap // 128, I // 128, 32, 16), hidden_fp8_t=f8(I, cap), hidden_sc_t=u8(I // 128, cap // 128, 32, 16),
               y_routed=None if fuse_combine else bf(cap, H), gate_shared=None, up_shared=None, hidden_shared=None, y_shared=None)
    if shared:
        out.update(gate_shared=bf(T, Is), up_shared=bf(T, Is), hidden_shared=bf(T, Is), y_shared=bf(T, H))
    a = _lib.MoeFwdArgs()
    a.dims = d
    a.fuse_combine = 1 if fuse_combine else 0
    a.x = _chk(x, "x", (torch.bfloat16,), (T, H))
    xp, cp = _ptr_array(x_ptrs), _ptr_array(combine_buffer_ptrs)
    a.x_ptrs, a.combine_ptrs = xp, cp
    a.w_shared_gate = _opt(w_shared_gate if shared else None, "w_shared_gate", (torch.bfloat16,), (Is, H))
    a.w_shared_up = _opt(w_shared_up if shared else None, "w_shared_up", (torch.bfloat16,), (Is, H))
    a.w_shared_down = _opt(w_shared_down if shared else None, "w_shared_down", (torch.bfloat16,), (H, Is))
    a.w_gate, a.w_gate_sc = _chk(w_routed_gate, "w_routed_gate", _FP8, (E, I, H)), _chk(w_routed_gate_sc, "w_routed_gate_sc", _SC)
    a.w_up, a.w_up_sc = _chk(w_routed_up, "w_routed_up", _FP8, (E, I, H)), _chk(w_routed_up_sc, "w_routed_up_sc", _SC)
    a.w_down, a.w_down_sc = _chk(w_routed_down, "w_routed_down", _FP8, (E, H, I)), _chk(w_routed_down_sc, "w_routed_down_sc", _SC)
    a.peer_rank = _chk(schedule_peer_rank, "schedule_peer_rank", (torch.int32,))
    a.peer_token_idx = _chk(schedule_peer_token_idx, "schedule_peer_token_idx", (torch.int32,), (cap,))
    a.num_tokens = _chk(num_tokens, "num_tokens", (torch.int32,))
    a.tokens_per_expert = _chk(tokens_per_expert, "tokens_per_expert", (torch.int32,), (E,))
    for name in _lib.FWD_OUT:
        setattr(a, name, out[name].data_ptr() if out[name] is not None else None)
    need = lib.mx8_moe_fwd_workspace_bytes(ctypes.byref(d))
    if need == 0:
        raise _lib.Mx8Error(_lib.ERR_SHAPE, "dispatch_mlp_swiglu_combine_fwd (dimensions)")
    ws = _workspace(dev, need)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    with torch.cuda.device(dev):
        _lib.check(lib.mx8_moe_fwd(ctypes.byref(a), _stream()), "dispatch_mlp_swiglu_combine_fwd")
    return tuple(out[name] for name in _lib.FWD_OUT)


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
                                    topk, num_comm_sms=0, macrobatch_size=0, minibatch_size=0, tuning=None):
    """Same arguments and the same 18 return values as the reference's backward binding
    (blackwell-ultra/022-…-mxfp8-bw.cu:2556-2760, bound at :3011-3028):
      (d_x_shared, d_x_routed, d_gate_shared, d_gate_fp8_routed, d_gate_sc_routed, d_up_shared,
       d_up_fp8_routed, d_up_sc_routed, d_hidden_shared, d_hidden_routed, d_y_routed_fp8_routed,
       d_y_routed_sc_routed, d_w_shared_gate, d_w_routed_gate, d_w_shared_up, d_w_routed_up,
       d_w_shared_down, d_w_routed_down)
    The routed part runs on the MXFP8 kernels; it uses the transposed activations the forward returned
    (x_fp8_t_routed, hidden_fp8_t_routed), so the arguments the reference needs only to replay its
    forward (x_buffer_ptrs, w_routed_gate/up) are accepted and unused.  The shared expert (bf16) runs when
    its inputs are given, else those outputs are None."""
    lib = _lib.load()
    E, H, I = w_routed_gate_T.shape                      # transposed weights: [E, H, I]
    cap = schedule_peer_rank.numel()
    dev = d_combine_buffer.device
    shared = (w_shared_gate_T is not None and w_shared_up_T is not None and w_shared_down_T is not None and d_y_shared is not None
              and gate_shared is not None and up_shared is not None and hidden_shared is not None and x_buffer is not None)
    T = d_combine_buffer.shape[0] // topk
    Is = gate_shared.shape[1] if shared else 0
    d = _dims(len(d_combine_buffer_ptrs), T, H, I, Is, E, topk, cap, num_comm_sms, minibatch_size, tuning)
    u8 = lambda *shape: torch.empty(*shape, dtype=torch.uint8, device=dev)
    f8 = lambda *shape: torch.empty(*shape, dtype=torch.float8_e4m3fn, device=dev)
    bf = lambda *shape: torch.empty(*shape, dtype=torch.bfloat16, device=dev)
    out = dict(d_x_routed=bf(cap, H), d_gate_fp8=f8(cap, I), d_gate_sc=u8(cap // 128, I // 128, 32, 16), d_up_fp8=f8(cap, I),
               d_up_sc=u8(cap // 128, I // 128, 32, 16), d_hidden_routed=bf(cap, I), d_y_fp8=f8(cap, H), d_y_sc=u8(cap // 128, H // 128, 32, 16),
               d_w_gate=bf(E, I, H), d_w_up=bf(E, I, H), d_w_down=bf(E, H, I))
    for name in ("d_x_shared", "d_gate_shared", "d_up_shared", "d_hidden_shared", "d_w_shared_gate", "d_w_shared_up", "d_w_shared_down"):
        out[name] = None
    if shared:
        out.update(d_x_shared=bf(T, H), d_gate_shared=bf(T, Is), d_up_shared=bf(T, Is), d_hidden_shared=bf(T, Is),
                   d_w_shared_gate=bf(Is, H), d_w_shared_up=bf(Is, H), d_w_shared_down=bf(H, Is))
    a = _lib.MoeBwdArgs()
    a.dims = d
    a.d_y_shared = _opt(d_y_shared if shared else None, "d_y_shared", (torch.bfloat16,), (T, H))
    src, dst = _ptr_array(d_combine_buffer_ptrs), _ptr_array(d_x_routed_buffer_ptrs)
    a.d_combine_ptrs, a.d_x_routed_ptrs = src, dst
    ins = dict(w_shared_gate_T=w_shared_gate_T, w_shared_up_T=w_shared_up_T, w_shared_down_T=w_shared_down_T, gate_shared=gate_shared,
               up_shared=up_shared, hidden_shared=hidden_shared, x=x_buffer)
    for name, t in ins.items():
        setattr(a, name, _opt(t if shared else None, name, (torch.bfloat16,)))
    a.w_gate_T, a.w_gate_T_sc = _chk(w_routed_gate_T, "w_routed_gate_T", _FP8, (E, H, I)), _chk(w_routed_gate_T_sc, "w_routed_gate_T_sc", _SC)
    a.w_up_T, a.w_up_T_sc = _chk(w_routed_up_T, "w_routed_up_T", _FP8, (E, H, I)), _chk(w_routed_up_T_sc, "w_routed_up_T_sc", _SC)
    a.w_down_T, a.w_down_T_sc = _chk(w_routed_down_T, "w_routed_down_T", _FP8, (E, I, H)), _chk(w_routed_down_T_sc, "w_routed_down_T_sc", _SC)
    a.x_fp8_t, a.x_sc_t = _chk(x_fp8_t_routed, "x_fp8_t_routed", _FP8, (H, cap)), _chk(x_sc_t_routed, "x_sc_t_routed", _SC)
    a.gate_fp8, a.gate_sc = _chk(gate_fp8_routed, "gate_fp8_routed", _FP8, (cap, I)), _chk(gate_sc_routed, "gate_sc_routed", _SC)
    a.up_fp8, a.up_sc = _chk(up_fp8_routed, "up_fp8_routed", _FP8, (cap, I)), _chk(up_sc_routed, "up_sc_routed", _SC)
    a.hidden_fp8_t = _chk(hidden_fp8_t_routed, "hidden_fp8_t_routed", _FP8, (I, cap))
    a.hidden_sc_t = _chk(hidden_sc_t_routed, "hidden_sc_t_routed", _SC)
    a.peer_rank = _chk(schedule_peer_rank, "schedule_peer_rank", (torch.int32,))
    a.peer_token_idx = _chk(schedule_peer_token_idx, "schedule_peer_token_idx", (torch.int32,), (cap,))
    a.num_tokens = _chk(num_tokens, "num_tokens", (torch.int32,))
    a.tokens_per_expert = _chk(tokens_per_expert, "tokens_per_expert", (torch.int32,), (E,))
    for name in _lib.BWD_OUT:
        setattr(a, name, out[name].data_ptr() if out[name] is not None else None)
    need = lib.mx8_moe_bwd_workspace_bytes(ctypes.byref(d))
    if need == 0:
        raise _lib.Mx8Error(_lib.ERR_SHAPE, "dispatch_mlp_swiglu_combine_bwd (dimensions)")
    ws = _workspace(dev, need)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    with torch.cuda.device(dev):
        _lib.check(lib.mx8_moe_bwd(ctypes.byref(a), _stream()), "dispatch_mlp_swiglu_combine_bwd")
    return tuple(out[name] for name in _lib.BWD_OUT)
