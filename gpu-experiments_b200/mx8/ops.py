"""Host-side mirror of the reference's pybind11 module `_C` for the MXFP8 path.

Function names, argument order and argument meaning follow the reference's harness-facing
bindings; each docstring cites the binding it stands in for.  Tensors stay owned by the caller,
launches go to torch's current CUDA stream and are asynchronous, exactly as in the reference.
Unlike the reference (which prints and exits), errors raise `Mx8Error`.
"""
import torch

from . import _lib
from ._lib import SCALE_FLOOR, SCALE_RCEIL, Mx8Error  # noqa: F401

_SCALE_MODES = {"rceil": SCALE_RCEIL, "floor": SCALE_FLOOR, SCALE_RCEIL: SCALE_RCEIL, SCALE_FLOOR: SCALE_FLOOR}
_FP8 = (torch.float8_e4m3fn, torch.uint8)
_SC = (torch.uint8, getattr(torch, "float8_e8m0fnu", torch.uint8))


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _chk(t, name, dtypes, shape=None):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if t.dtype not in dtypes:
        raise ValueError(f"{name} has dtype {t.dtype}, expected one of {dtypes}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if shape is not None and t.numel() != _numel(shape):
        raise ValueError(f"{name} has {t.numel()} elements, expected shape {tuple(shape)}")
    return t.data_ptr()


def _numel(shape):
    n = 1
    for s in shape:
        n *= s
    return n


def mxfp8_quantize(x_bf16, *args, scale_mode="rceil"):
    """Two call forms, as in the reference:

    mxfp8_quantize(x_bf16, x_fp8, x_sc, x_fp8_t, x_sc_t, return_normal, return_transposed) -> None
        caller-allocated outputs (blackwell-ultra/019-mxfp8-quantize.cu:185-219); an output pair
        that is not requested is ignored and may be any tensor.
    mxfp8_quantize(x_bf16, return_normal, return_transposed) -> (x_fp8, x_sc, x_fp8_t, x_sc_t)
        outputs allocated here; x_bf16 is [M, N] or [E, M, N]; outputs not requested are None
        (blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.cu:404-448).

    x_sc is uint8 [rows/128, cols/128, 32, 16] in the tcgen05 scale tile layout.
    `scale_mode` ("rceil" = the reference's rule, "floor" = OCP) is an addition.
    """
    lib = _lib.load()
    if x_bf16.dim() not in (2, 3):
        raise ValueError("x_bf16 must be [M, N] or [E, M, N]")
    E = x_bf16.shape[0] if x_bf16.dim() == 3 else 1
    M, N = x_bf16.shape[-2], x_bf16.shape[-1]
    xp = _chk(x_bf16, "x_bf16", (torch.bfloat16,))
    mode = _SCALE_MODES[scale_mode]
    if len(args) == 2:
        rn, rt = bool(args[0]), bool(args[1])
        lead = (E,) if x_bf16.dim() == 3 else ()
        dev = x_bf16.device
        x_fp8 = torch.empty(lead + (M, N), dtype=torch.float8_e4m3fn, device=dev) if rn else None
        x_sc = torch.empty(E * M // 128, N // 128, 32, 16, dtype=torch.uint8, device=dev) if rn else None
        x_fp8_t = torch.empty(lead + (N, M), dtype=torch.float8_e4m3fn, device=dev) if rt else None
        x_sc_t = torch.empty(E * N // 128, M // 128, 32, 16, dtype=torch.uint8, device=dev) if rt else None
        ret = (x_fp8, x_sc, x_fp8_t, x_sc_t)
    elif len(args) == 6:
        x_fp8, x_sc, x_fp8_t, x_sc_t = args[:4]
        rn, rt = bool(args[4]), bool(args[5])
        ret = None
    else:
        raise TypeError("mxfp8_quantize takes (x, rn, rt) or (x, x_fp8, x_sc, x_fp8_t, x_sc_t, rn, rt)")
    if not (rn or rt):
        raise ValueError("at least one of return_normal / return_transposed must be set")
    p = [None, None, None, None]
    if rn:
        p[0] = _chk(x_fp8, "x_fp8", _FP8, (E, M, N))
        p[1] = _chk(x_sc, "x_sc", _SC, (E * M // 128, N // 128, 512))
    if rt:
        p[2] = _chk(x_fp8_t, "x_fp8_t", _FP8, (E, N, M))
        p[3] = _chk(x_sc_t, "x_sc_t", _SC, (E * N // 128, M // 128, 512))
    with torch.cuda.device(x_bf16.device):
        _lib.check(lib.mx8_quantize(xp, E, M, N, p[0], p[1], p[2], p[3], mode, _stream()), "mxfp8_quantize")
    return ret


def _chk_host(t, name, dtypes, shape):
    if not isinstance(t, torch.Tensor) or t.is_cuda:
        raise ValueError(f"{name} must be a host tensor")
    if t.dtype not in dtypes:
        raise ValueError(f"{name} has dtype {t.dtype}, expected one of {dtypes}")
    if not t.is_contiguous() or t.numel() != _numel(shape):
        raise ValueError(f"{name} must be contiguous with shape {tuple(shape)}")
    return t.data_ptr()


def _workspace(workspace, need, device):
    if workspace is None:
        return torch.empty(need, dtype=torch.uint8, device=device)
    if not workspace.is_cuda or workspace.numel() * workspace.element_size() < need:
        raise ValueError(f"workspace must be a CUDA tensor of at least {need} bytes")
    return workspace


def mxfp8_quantize_host(x_bf16, x_fp8, x_sc, x_fp8_t, x_sc_t, return_normal, return_transposed, *,
                        band_rows=2048, workspace=None, device=None, scale_mode="rceil"):
    """mxfp8_quantize for a matrix that lives in HOST memory: x_bf16 [M, N] and the requested outputs
    are host tensors (page-locked for the copies to overlap) with the layouts of `mxfp8_quantize`.
    Bands of `band_rows` rows flow through copy-in, kernel and copy-out on three streams
    (mx8_quantize_host).  `workspace` is a CUDA byte tensor of `quantize_host_workspace(N, band_rows)`
    bytes, allocated per call when omitted.  Returns the workspace so that a caller can keep it."""
    lib = _lib.load()
    M, N = x_bf16.shape
    xp = _chk_host(x_bf16, "x_bf16", (torch.bfloat16,), (M, N))
    p = [None, None, None, None]
    if return_normal:
        p[0] = _chk_host(x_fp8, "x_fp8", _FP8, (M, N))
        p[1] = _chk_host(x_sc, "x_sc", _SC, (M // 128, N // 128, 512))
    if return_transposed:
        p[2] = _chk_host(x_fp8_t, "x_fp8_t", _FP8, (N, M))
        p[3] = _chk_host(x_sc_t, "x_sc_t", _SC, (N // 128, M // 128, 512))
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        rows = min(band_rows, M)
        need = lib.mx8_quantize_host_workspace(N, rows)
        ws = _workspace(workspace, need, dev)
        _lib.check(lib.mx8_quantize_host(xp, M, N, p[0], p[1], p[2], p[3], _SCALE_MODES[scale_mode], band_rows,
                                         ws.data_ptr(), ws.numel() * ws.element_size(), _stream()), "mxfp8_quantize_host")
    return ws


def quantize_host_workspace(N, band_rows):
    return _lib.load().mx8_quantize_host_workspace(N, band_rows)


def kernel_host(A, A_sc, B, B_sc, C, *, band_rows=2048, workspace=None, device=None):
    """`kernel(A_fp8, A_sc, B_fp8, B_sc, C)` for operands and result in HOST memory (mx8_gemm_host):
    B and its scales are copied once, then bands of `band_rows` rows of A and C are pipelined."""
    lib = _lib.load()
    M, K = A.shape
    N = B.shape[0]
    ap = _chk_host(A, "A", _FP8, (M, K))
    bp = _chk_host(B, "B", _FP8, (N, K))
    asp = _chk_host(A_sc, "A_sc", _SC, (M // 128, K // 128, 512))
    bsp = _chk_host(B_sc, "B_sc", _SC, (N // 128, K // 128, 512))
    cp = _chk_host(C, "C", (torch.bfloat16, torch.float32), (M, N))
    c_dtype = _lib.C_F32 if C.dtype == torch.float32 else _lib.C_BF16
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        rows = min(band_rows, M)
        need = lib.mx8_gemm_host_workspace(N, K, rows, c_dtype)
        ws = _workspace(workspace, need, dev)
        _lib.check(lib.mx8_gemm_host(ap, asp, bp, bsp, cp, M, N, K, c_dtype, band_rows, ws.data_ptr(),
                                     ws.numel() * ws.element_size(), _stream()), "kernel_host")
    return ws


def kernel_a_bf16(A_bf16, B, B_sc, C, workspace=None, fused=False):
    """`kernel` for an A operand that is still bf16 [M, K]: quantized row-wise into `workspace` (a CUDA byte
    tensor of mx8_gemm_a_bf16_workspace(M, K) bytes, allocated here when omitted), then the block-scaled GEMM
    (mx8_gemm_a_bf16).  Returns the workspace: its first M*K bytes are A's E4M3 bytes, the scale tiles follow.
    fused=True quantizes inside the GEMM's main loop instead (mx8_gemm_a_bf16_fused): one launch, no workspace,
    same bits; returns None."""
    lib = _lib.load()
    M, K = A_bf16.shape
    N = B.shape[0]
    ap = _chk(A_bf16, "A_bf16", (torch.bfloat16,), (M, K))
    bp, bsp = _chk(B, "B", _FP8, (N, K)), _chk(B_sc, "B_sc", _SC, (N // 128, K // 128, 512))
    cp = _chk(C, "C", (torch.bfloat16, torch.float32), (M, N))
    cd = _lib.C_F32 if C.dtype == torch.float32 else _lib.C_BF16
    if fused:
        with torch.cuda.device(A_bf16.device):
            _lib.check(lib.mx8_gemm_a_bf16_fused(ap, bp, bsp, cp, M, N, K, cd, _stream()), "kernel_a_bf16 (fused)")
        return None
    with torch.cuda.device(A_bf16.device):
        ws = _workspace(workspace, lib.mx8_gemm_a_bf16_workspace(M, K), A_bf16.device)
        _lib.check(lib.mx8_gemm_a_bf16(ap, bp, bsp, cp, M, N, K, cd, ws.data_ptr(), ws.numel() * ws.element_size(), _stream()),
                   "kernel_a_bf16")
    return ws


def kernel(A, A_sc, B, B_sc, C, *, cta_group=0, max_ctas=0):
    """kernel(A_fp8, A_sc, B_fp8, B_sc, C) -> None:  C = dequant(A) . dequant(B)^T.

    A [M, K], B [N, K] E4M3; A_sc [M/128, K/128, 512] (or [.., 32, 16]) and B_sc likewise, uint8 in
    the scale tile layout; C [M, N] preallocated, bf16 (blackwell/047-mxfp8-mma-2cta-MNK128-
    polished.cu:532-541, also 045/046) or float32 (blackwell/009-mxfp8-mm.cu:225-234, 010-017).
    """
    lib = _lib.load()
    M, K = A.shape
    N = B.shape[0]
    if B.shape[1] != K or tuple(C.shape) != (M, N):
        raise ValueError("shape mismatch: A [M,K], B [N,K], C [M,N]")
    ap = _chk(A, "A", _FP8)
    bp = _chk(B, "B", _FP8)
    asp = _chk(A_sc, "A_sc", _SC, (M // 128, K // 128, 512))
    bsp = _chk(B_sc, "B_sc", _SC, (N // 128, K // 128, 512))
    cp = _chk(C, "C", (torch.bfloat16, torch.float32))
    cd = _lib.C_F32 if C.dtype == torch.float32 else _lib.C_BF16
    with torch.cuda.device(A.device):
        _lib.check(lib.mx8_gemm_ex(ap, asp, bp, bsp, cp, M, N, K, cd, cta_group, max_ctas, _stream()), "kernel")


def quantize_kernel(A, A_fp8, A_sc, A_t_fp8=None, A_t_sc=None):
    """Legacy quantize entry points of the older harnesses, which call the binding `kernel`:
    kernel(A, A_fp8, A_sc) (blackwell/018-mxfp8-quantize.cu:288-300, 036) and
    kernel(A, A_fp8, A_sc, A_t_fp8, A_t_sc) (blackwell/038-mxfp8-quantize-combined.cu:397-399).
    A_sc is [M/128, N/128, 512]."""
    both = A_t_fp8 is not None
    mxfp8_quantize(A, A_fp8, A_sc, A_t_fp8, A_t_sc, True, both)


def kernel_transpose(A, A_fp8, A_sc):
    """kernel_transpose(A, A_t_fp8, A_t_sc): transposed-only quantize
    (blackwell/018-mxfp8-quantize.cu:294-300, blackwell/037-mxfp8-transpose-quantize.cu)."""
    mxfp8_quantize(A, None, None, A_fp8, A_sc, False, True)


def device_status():
    """Synchronize the current stream and return the device status word (0 = healthy); raises
    Mx8Error if a kernel's bounded wait expired."""
    import ctypes
    lib = _lib.load()
    v = ctypes.c_int(0)
    rc = lib.mx8_device_status(ctypes.byref(v), _stream())
    if rc != _lib.OK:
        raise Mx8Error(rc, f"device_status (device word = {v.value})")
    return v.value


def schedule(topk_all, num_local_experts, schedule_capacity, rank):
    """schedule(topk_all, num_local_experts, schedule_capacity, rank)
        -> (schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert)

    topk_all int32 [world, tokens, topk] on the device.  Outputs are int32 CUDA tensors, allocated
    here like the reference does (blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.cu:149-183,
    bound at :2996-2997)."""
    lib = _lib.load()
    tp = _chk(topk_all, "topk_all", (torch.int32,))
    if topk_all.dim() != 3:
        raise ValueError("topk_all must be [world, tokens, topk]")
    W, T, k = topk_all.shape
    dev = topk_all.device
    peer_rank = torch.empty(schedule_capacity, dtype=torch.int32, device=dev)
    peer_tok = torch.empty(schedule_capacity, dtype=torch.int32, device=dev)
    num_tokens = torch.empty(1, dtype=torch.int32, device=dev)
    tpe = torch.empty(num_local_experts, dtype=torch.int32, device=dev)
    scratch = torch.empty(lib.mx8_moe_schedule_scratch_bytes(W, T, k, num_local_experts), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.mx8_moe_schedule(tp, W, T, k, num_local_experts, schedule_capacity, rank, peer_rank.data_ptr(),
                                        peer_tok.data_ptr(), num_tokens.data_ptr(), tpe.data_ptr(), scratch.data_ptr(),
                                        scratch.numel(), _stream()), "schedule")
    return peer_rank, peer_tok, num_tokens, tpe


def gemm_grouped(A, A_sc, B, B_sc, C, C_sc=None, num_rows=None, group_rows=None):
    """Grouped / quantizing GEMM (mx8_gemm_grouped).

    A [M, K] E4M3 rows of all groups back to back, A_sc its scale tiles; B [G, N, K] (or [N, K] when
    group_rows is None) with B_sc [G*N/128, K/128, 512]; C [M, N] bf16/float32, or E4M3/uint8 together
    with C_sc [M/128, N/128, 32, 16] for the quantizing epilogue.  num_rows: int32 device tensor with
    the rows present; group_rows: int32 device tensor [G], multiples of 256.
    Stands in for expert_grouped_gemm<false> inside the reference's MoE kernel
    (blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.cu:1399-1736)."""
    lib = _lib.load()
    M, K = A.shape
    G = 0
    if group_rows is not None:
        G, N = B.shape[0], B.shape[1]
        if B.dim() != 3 or B.shape[2] != K:
            raise ValueError("grouped B must be [G, N, K]")
    else:
        N = B.shape[0]
    if tuple(C.shape) != (M, N):
        raise ValueError("C must be [M, N]")
    ap, bp = _chk(A, "A", _FP8), _chk(B, "B", _FP8)
    asp = _chk(A_sc, "A_sc", _SC, (M // 128, K // 128, 512))
    bsp = _chk(B_sc, "B_sc", _SC, (max(G, 1) * N // 128, K // 128, 512))
    if C_sc is not None:
        cp = _chk(C, "C", _FP8)
        csp = _chk(C_sc, "C_sc", _SC, (M // 128, N // 128, 512))
        cd = _lib.C_MXFP8
    else:
        cp = _chk(C, "C", (torch.bfloat16, torch.float32))
        csp = None
        cd = _lib.C_F32 if C.dtype == torch.float32 else _lib.C_BF16
    nr = _chk(num_rows, "num_rows", (torch.int32,)) if num_rows is not None else None
    grp = _chk(group_rows, "group_rows", (torch.int32,)) if group_rows is not None else None
    with torch.cuda.device(A.device):
        _lib.check(lib.mx8_gemm_grouped(ap, asp, bp, bsp, cp, csp, M, N, K, cd, nr, grp, G, _stream()), "gemm_grouped")


def gemm_grouped_dual(A1, A1_sc, B1, B1_sc, A2, A2_sc, B2, B2_sc, C, num_rows=None, group_rows=None):
    """C = dequant(A1) . dequant(B1_g)^T + dequant(A2) . dequant(B2_g)^T (bf16), grouped like gemm_grouped.
    The data-gradient GEMM of the MoE backward (two operand pairs instead of concatenated tensors;
    blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.cu:1399-1736, second GEMM of expert_grouped_gemm)."""
    lib = _lib.load()
    M, K1 = A1.shape
    K2 = A2.shape[1]
    G = B1.shape[0] if group_rows is not None else 0
    N = B1.shape[1] if group_rows is not None else B1.shape[0]
    ptrs = [_chk(A1, "A1", _FP8), _chk(A1_sc, "A1_sc", _SC), _chk(B1, "B1", _FP8), _chk(B1_sc, "B1_sc", _SC),
            _chk(A2, "A2", _FP8), _chk(A2_sc, "A2_sc", _SC), _chk(B2, "B2", _FP8), _chk(B2_sc, "B2_sc", _SC),
            _chk(C, "C", (torch.bfloat16,), (M, N))]
    nr = _chk(num_rows, "num_rows", (torch.int32,)) if num_rows is not None else None
    grp = _chk(group_rows, "group_rows", (torch.int32,)) if group_rows is not None else None
    with torch.cuda.device(A1.device):
        _lib.check(lib.mx8_gemm_grouped_dual(*ptrs, M, N, K1, K2, nr, grp, G, _stream()), "gemm_grouped_dual")


def gemm_wgrad(A_t, A_t_sc, B_t, B_t_sc, C, group_rows):
    """C[g] = dequant(A_t[:, rows_g]) . dequant(B_t[:, rows_g])^T for every group g (bf16 [G, M, N]);
    A_t [M, R] and B_t [N, R] are transposed quantizer outputs (blocks along R).  The weight-gradient
    form of the reference's expert_grouped_gemm (IS_WGRAD)."""
    lib = _lib.load()
    M, R = A_t.shape
    N = B_t.shape[0]
    G = group_rows.numel()
    with torch.cuda.device(A_t.device):
        _lib.check(lib.mx8_gemm_wgrad(_chk(A_t, "A_t", _FP8), _chk(A_t_sc, "A_t_sc", _SC, (M // 128, R // 128, 512)),
                                      _chk(B_t, "B_t", _FP8, (N, R)), _chk(B_t_sc, "B_t_sc", _SC, (N // 128, R // 128, 512)),
                                      _chk(C, "C", (torch.bfloat16,), (G, M, N)), M, N, R,
                                      _chk(group_rows, "group_rows", (torch.int32,)), G, _stream()), "gemm_wgrad")


def gemm_bf16(A, B, C, A2=None, B2=None):
    """C[M, N] = A[M, K] @ B[N, K].T (+ A2[M, K2] @ B2[N, K2].T), bf16 operands, fp32 accumulation on the
    tensor cores, C bf16 or float32 (mx8_gemm_bf16 / mx8_gemm_bf16_dual): the shared expert's GEMMs,
    expert_grouped_gemm<true> of blackwell-ultra/022-…-mxfp8-bw.cu:1399-1736."""
    lib = _lib.load()
    M, K = A.shape
    N = B.shape[0]
    bf = (torch.bfloat16,)
    ap, bp = _chk(A, "A", bf, (M, K)), _chk(B, "B", bf, (N, K))
    cp = _chk(C, "C", (torch.bfloat16, torch.float32), (M, N))
    cd = _lib.C_F32 if C.dtype == torch.float32 else _lib.C_BF16
    K2, a2p, b2p = 0, None, None
    if A2 is not None:
        K2 = A2.shape[1]
        a2p, b2p = _chk(A2, "A2", bf, (M, K2)), _chk(B2, "B2", bf, (N, K2))
    with torch.cuda.device(A.device):
        _lib.check(lib.mx8_gemm_bf16_dual(ap, bp, a2p, b2p, cp, M, N, K, K2, cd, _stream()), "gemm_bf16")
    return C


def swiglu_bf16(gate, up, hidden=None):
    """hidden = silu(gate) * up on bf16 tensors (swiglu_fwd<true>, blackwell-ultra/022-…-mxfp8-bw.cu:1097-1110)."""
    lib = _lib.load()
    bf = (torch.bfloat16,)
    hidden = torch.empty_like(gate) if hidden is None else hidden
    n = gate.numel()
    with torch.cuda.device(gate.device):
        _lib.check(lib.mx8_swiglu_bf16(_chk(gate, "gate", bf), _chk(up, "up", bf, gate.shape), _chk(hidden, "hidden", bf, gate.shape),
                                       n, _stream()), "swiglu_bf16")
    return hidden


def swiglu_bwd_bf16(d_hidden, gate, up):
    """(d_gate, d_up) of hidden = silu(gate) * up (swiglu_bwd<true>, blackwell-ultra/022-…-mxfp8-bw.cu:1354-1375)."""
    lib = _lib.load()
    bf = (torch.bfloat16,)
    d_gate, d_up = torch.empty_like(gate), torch.empty_like(gate)
    with torch.cuda.device(gate.device):
        _lib.check(lib.mx8_swiglu_bwd_bf16(_chk(d_hidden, "d_hidden", bf, gate.shape), _chk(gate, "gate", bf), _chk(up, "up", bf, gate.shape),
                                           d_gate.data_ptr(), d_up.data_ptr(), gate.numel(), _stream()), "swiglu_bwd_bf16")
    return d_gate, d_up


def transpose_bf16(x):
    """x[rows, cols] -> new contiguous [cols, rows] (mx8_transpose_bf16)."""
    lib = _lib.load()
    rows, cols = x.shape
    out = torch.empty(cols, rows, dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(lib.mx8_transpose_bf16(_chk(x, "x", (torch.bfloat16,)), out.data_ptr(), rows, cols, _stream()), "transpose_bf16")
    return out
