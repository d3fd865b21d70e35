"""ctypes binding of libmx8.so (declared in include/mx8.h).  Fails loudly when the library is
missing or a call returns a non-zero status: there is no fallback path."""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libmx8.so")

OK, ERR_ARG, ERR_SHAPE, ERR_ALIGN, ERR_CUDA, ERR_UNSUPPORTED, ERR_DEVICE_TIMEOUT, ERR_LIMIT = range(8)
SCALE_RCEIL, SCALE_FLOOR = 0, 1
C_BF16, C_F32, C_MXFP8 = 0, 1, 2

# every symbol include/mx8.h declares, with its ctypes signature
_vp, _i = ctypes.c_void_p, ctypes.c_int
class Window(ctypes.Structure):
    """mx8_window: rows [*row_begin, *row_end) (device ints) on at most max_sms multiprocessors."""
    _fields_ = [("row_begin", ctypes.c_void_p), ("row_end", ctypes.c_void_p), ("max_sms", ctypes.c_int), ("own_sms", ctypes.c_int)]


_wp = ctypes.POINTER(Window)
_pp = ctypes.POINTER(ctypes.c_void_p)


class MoeDims(ctypes.Structure):
    """mx8_moe_dims"""
    _fields_ = [(n, ctypes.c_int) for n in ("world", "tokens", "hidden", "intermediate", "shared_intermediate", "num_local_experts",
                                            "topk", "capacity", "num_comm_sms", "minibatch_size", "minibatches", "ramp", "combine_sms", "split_gate_up", "split_swiglu", "combine_own_sms")]


FWD_IN = ("w_shared_gate", "w_shared_up", "w_shared_down", "w_gate", "w_gate_sc", "w_up", "w_up_sc", "w_down", "w_down_sc",
          "peer_rank", "peer_token_idx", "num_tokens", "tokens_per_expert")
FWD_OUT = ("x_fp8_t", "x_sc_t", "gate_shared", "gate_fp8", "gate_sc", "up_shared", "up_fp8", "up_sc", "hidden_shared", "hidden_fp8_t",
           "hidden_sc_t", "y_shared", "y_routed")


class MoeFwdArgs(ctypes.Structure):
    """mx8_moe_fwd_args"""
    _fields_ = ([("dims", MoeDims), ("fuse_combine", ctypes.c_int), ("x", ctypes.c_void_p), ("x_ptrs", _pp), ("combine_ptrs", _pp)]
                + [(n, ctypes.c_void_p) for n in FWD_IN + FWD_OUT] + [("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t)])


BWD_IN = ("w_shared_gate_T", "w_shared_up_T", "w_shared_down_T", "w_gate_T", "w_gate_T_sc", "w_up_T", "w_up_T_sc", "w_down_T", "w_down_T_sc",
          "x_fp8_t", "x_sc_t", "gate_shared", "gate_fp8", "gate_sc", "up_shared", "up_fp8", "up_sc", "hidden_shared", "hidden_fp8_t",
          "hidden_sc_t", "x", "peer_rank", "peer_token_idx", "num_tokens", "tokens_per_expert")
BWD_OUT = ("d_x_shared", "d_x_routed", "d_gate_shared", "d_gate_fp8", "d_gate_sc", "d_up_shared", "d_up_fp8", "d_up_sc", "d_hidden_shared",
           "d_hidden_routed", "d_y_fp8", "d_y_sc", "d_w_shared_gate", "d_w_gate", "d_w_shared_up", "d_w_up", "d_w_shared_down", "d_w_down")


class MoeBwdArgs(ctypes.Structure):
    """mx8_moe_bwd_args"""
    _fields_ = ([("dims", MoeDims), ("d_y_shared", ctypes.c_void_p), ("d_combine_ptrs", _pp), ("d_x_routed_ptrs", _pp)]
                + [(n, ctypes.c_void_p) for n in BWD_IN + BWD_OUT] + [("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t)])


SIGNATURES = {
    "mx8_quantize": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _vp]),
    "mx8_gemm": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "mx8_gemm_ex": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "mx8_gemm_grouped": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _i, _vp]),
    "mx8_moe_dispatch_quantize": (_i, [ctypes.POINTER(_vp), _i, _i, _i, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp]),
    "mx8_swiglu_quantize": (_i, [_vp, _vp, _vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "mx8_moe_combine": (_i, [_vp, _vp, _vp, _vp, _i, _i, ctypes.POINTER(_vp), _i, ctypes.c_longlong, _vp]),
    "mx8_moe_fwd_epilogue": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "mx8_gemm_grouped_scatter": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _i, _vp, _vp, ctypes.POINTER(_vp), _i, _vp]),
    "mx8_gemm_grouped_dual": (_i, [_vp] * 9 + [_i, _i, _i, _i, _vp, _vp, _i, _vp]),
    "mx8_gemm_wgrad": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _i, _vp]),
    "mx8_swiglu_bwd_quantize": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "mx8_swiglu_bwd_quantize_both": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _vp] + [_vp] * 8 + [_vp]),
    "mx8_moe_bwd_prologue": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "mx8_moe_bwd_epilogue": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "mx8_moe_schedule": (_i, [_vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, ctypes.c_size_t, _vp]),
    "mx8_moe_schedule_scratch_bytes": (ctypes.c_size_t, [_i, _i, _i, _i]),
    "mx8_moe_schedule_static": (_i, [_vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "mx8_gemm_bf16": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "mx8_gemm_bf16_dual": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "mx8_swiglu_bf16": (_i, [_vp, _vp, _vp, ctypes.c_longlong, _vp]),
    "mx8_swiglu_bwd_bf16": (_i, [_vp, _vp, _vp, _vp, _vp, ctypes.c_longlong, _vp]),
    "mx8_transpose_bf16": (_i, [_vp, _vp, _i, _i, _vp]),
    "mx8_moe_minibatch_bounds": (_i, [_vp, _i, _i, _vp, _vp]),
    "mx8_moe_dispatch_quantize_window": (_i, [ctypes.POINTER(_vp), _i, _i, _i, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _wp, _vp]),
    "mx8_gemm_grouped_window": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _i, _wp, _vp]),
    "mx8_gemm_grouped_pair_window": (_i, [_vp] * 10 + [_i, _i, _i, _i, _vp, _vp, _i, _wp, _vp]),
    "mx8_gemm_grouped_swiglu_window": (_i, [_vp] * 14 + [_i, _i, _i, _vp, _vp, _i, _wp, _vp]),
    "mx8_swiglu_quantize_window": (_i, [_vp, _vp, _vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _wp, _vp]),
    "mx8_swiglu_bwd_quantize_both_window": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _vp] + [_vp] * 8 + [_wp, _vp]),
    "mx8_gemm_grouped_dual_window": (_i, [_vp] * 9 + [_i, _i, _i, _i, _vp, _vp, _i, _wp, _vp]),
    "mx8_moe_combine_window": (_i, [_vp, _vp, _vp, _vp, _i, _i, ctypes.POINTER(_vp), _i, ctypes.c_longlong, _wp, _vp]),
    "mx8_moe_minibatch_bounds_split": (_i, [_vp, _i, _i, ctypes.POINTER(_i), _vp, _vp]),
    "mx8_moe_fwd_workspace_bytes": (ctypes.c_size_t, [ctypes.POINTER(MoeDims)]),
    "mx8_moe_fwd": (_i, [ctypes.POINTER(MoeFwdArgs), _vp]),
    "mx8_moe_bwd_workspace_bytes": (ctypes.c_size_t, [ctypes.POINTER(MoeDims)]),
    "mx8_moe_bwd": (_i, [ctypes.POINTER(MoeBwdArgs), _vp]),
    "mx8_quantize_host_workspace": (ctypes.c_size_t, [_i, _i]),
    "mx8_quantize_host": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _i, _i, _vp, ctypes.c_size_t, _vp]),
    "mx8_gemm_host_workspace": (ctypes.c_size_t, [_i, _i, _i, _i]),
    "mx8_gemm_host": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, ctypes.c_size_t, _vp]),
    "mx8_gemm_a_bf16_workspace": (ctypes.c_size_t, [_i, _i]),
    "mx8_gemm_a_bf16_fused": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "mx8_gemm_a_bf16": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, ctypes.c_size_t, _vp]),
    "mx8_probe_mma_peak": (_i, [_i, ctypes.POINTER(ctypes.c_double), _vp]),
    "mx8_selftest_bounded_wait": (_i, [ctypes.c_uint, _vp]),
    "mx8_device_status": (_i, [ctypes.POINTER(_i), _vp]),
    "mx8_strerror": (ctypes.c_char_p, [_i]),
    "mx8_last_cuda_error": (ctypes.c_char_p, []),
    "mx8_version": (ctypes.c_char_p, []),
}

_lib = None


class Mx8Error(RuntimeError):
    def __init__(self, code, where):
        self.code = code
        lib = load()
        msg = lib.mx8_strerror(code).decode()
        detail = lib.mx8_last_cuda_error().decode() if code in (ERR_CUDA, ERR_LIMIT) else ""
        super().__init__(f"{where}: mx8 status {code}: {msg}" + (f" [{detail}]" if detail else ""))


def load():
    """Load libmx8.so once.  torch is imported first so that its CUDA runtime is the one in the
    process."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python gpu-experiments_b200/build.py` "
                "(the mx8 operators have no fallback implementation)")
        import torch  # noqa: F401  (loads libcudart)
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(code, where):
    if code != OK:
        raise Mx8Error(code, where)
