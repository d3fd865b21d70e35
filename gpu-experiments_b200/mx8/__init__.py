"""mx8: B200-native MXFP8 quantize + block-scaled GEMM behind the C ABI in include/mx8.h."""
from ._lib import LIB_PATH, Mx8Error, load  # noqa: F401
from .ops import (device_status, gemm_grouped, gemm_grouped_dual, gemm_wgrad, kernel, kernel_transpose, mxfp8_quantize, schedule,  # noqa: F401
                  quantize_kernel)
from .moe import (combine, dispatch_mlp_swiglu_combine_fwd, dispatch_quantize, fwd_epilogue,  # noqa: F401
                  swiglu_quantize)
