"""mx8: B200-native MXFP8 quantize + block-scaled GEMM behind the C ABI in include/mx8.h."""
from ._lib import LIB_PATH, Mx8Error, load  # noqa: F401
from .ops import (device_status, gemm_grouped, gemm_grouped_dual, gemm_wgrad, kernel, kernel_transpose, mxfp8_quantize, schedule,  # noqa: F401
                  quantize_kernel, gemm_bf16, swiglu_bf16, swiglu_bwd_bf16, transpose_bf16, kernel_a_bf16, kernel_host, mxfp8_quantize_host, quantize_host_workspace)
from .moe import (bwd_epilogue, bwd_epilogue_routed, bwd_prologue, combine, dispatch_mlp_swiglu_combine_bwd,  # noqa: F401
                  dispatch_mlp_swiglu_combine_fwd, dispatch_quantize, fwd_epilogue, swiglu_bwd_quantize, swiglu_bwd_quantize_both, swiglu_quantize)
