"""CPU-side checks of the C-ABI library: it loads, exports every declared symbol, and validates
arguments before touching a device."""
import ctypes
import os
import re

import pytest

import mx8
from mx8 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(_lib.LIB_PATH):
        import importlib.util
        spec = importlib.util.spec_from_file_location("mx8_build", os.path.join(ROOT, "gpu-experiments_b200", "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()
    return mx8.load()


def test_header_and_binding_agree(lib):
    hdr = open(os.path.join(ROOT, "include", "mx8.h")).read()
    declared = set(re.findall(r"MX8_API\s+[\w\s\*]+?\b(mx8_\w+)\s*\(", hdr))
    assert declared == set(_lib.SIGNATURES), (declared, set(_lib.SIGNATURES))
    for name in declared:
        assert hasattr(lib, name)


def test_status_codes_have_text(lib):
    hdr = open(os.path.join(ROOT, "include", "mx8.h")).read()
    codes = dict((n, int(v)) for n, v in re.findall(r"(MX8_(?:OK|ERR_\w+))\s*=\s*(\d+)", hdr))
    assert codes["MX8_OK"] == _lib.OK and codes["MX8_ERR_DEVICE_TIMEOUT"] == _lib.ERR_DEVICE_TIMEOUT
    for v in codes.values():
        assert b"unknown" not in lib.mx8_strerror(v)
    assert b"unknown" in lib.mx8_strerror(99)
    assert lib.mx8_version().startswith(b"mx8")


def test_argument_validation_needs_no_device(lib):
    p = ctypes.c_void_p(4096)      # never dereferenced: validation fails first
    odd = ctypes.c_void_p(4100)
    q = lib.mx8_quantize
    assert q(None, 1, 128, 128, p, p, p, p, 0, None) == _lib.ERR_ARG
    assert q(p, 1, 128, 128, None, None, None, None, 0, None) == _lib.ERR_ARG       # nothing requested
    assert q(p, 1, 128, 128, p, None, None, None, 0, None) == _lib.ERR_ARG          # half a pair
    assert q(p, 1, 128, 128, p, p, None, None, 7, None) == _lib.ERR_ARG             # bad scale mode
    assert q(p, 1, 100, 128, p, p, None, None, 0, None) == _lib.ERR_SHAPE
    assert q(p, 1, 128, 0, p, p, None, None, 0, None) == _lib.ERR_SHAPE
    assert q(p, 0, 128, 128, p, p, None, None, 0, None) == _lib.ERR_SHAPE
    assert q(odd, 1, 128, 128, p, p, None, None, 0, None) == _lib.ERR_ALIGN
    g = lib.mx8_gemm
    assert g(None, p, p, p, p, 128, 128, 128, 0, None) == _lib.ERR_ARG
    assert g(p, p, p, p, p, 128, 128, 128, 5, None) == _lib.ERR_ARG
    assert g(p, p, p, p, p, 128, 192, 128, 0, None) == _lib.ERR_SHAPE
    assert g(p, p, p, p, p, 128, 128, 64, 0, None) == _lib.ERR_SHAPE
    assert g(p, p, odd, p, p, 128, 128, 128, 0, None) == _lib.ERR_ALIGN
    assert lib.mx8_gemm_ex(p, p, p, p, p, 128, 128, 128, 0, 3, 0, None) == _lib.ERR_ARG


def test_no_device_means_error_not_fallback(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    p = ctypes.c_void_p(4096)
    rc = lib.mx8_quantize(p, 1, 128, 128, p, p, None, None, 0, None)
    assert rc in (_lib.ERR_CUDA, _lib.ERR_UNSUPPORTED)
    with pytest.raises(ValueError):
        mx8.mxfp8_quantize(torch.zeros(128, 128, dtype=torch.bfloat16), True, False)   # CPU tensor rejected


def test_torch_module_mirrors_reference_bindings(lib):
    """mx8._C is the pybind11/torch module with the reference's function names."""
    import importlib.util
    import torch
    spec = importlib.util.spec_from_file_location("mx8_build", os.path.join(ROOT, "gpu-experiments_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    if not os.path.exists(mod.torch_binding_path()):
        mod.build_torch_binding()
    from mx8 import _C
    for name in ("mxfp8_quantize", "kernel", "kernel_transpose", "schedule", "dispatch_mlp_swiglu_combine_fwd", "fwd_epilogue",
                 "device_status", "version"):
        assert hasattr(_C, name)
    assert _C.version().startswith("mx8")
    x = torch.zeros(128, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        _C.mxfp8_quantize(x, True, False)          # CPU tensor: rejected, never computed on the host


def test_moe_layer_structs_match_the_header_layout(lib):
    # the argument structs of mx8_moe_fwd / mx8_moe_bwd as ctypes declares them against what the library reads:
    # every pointer field set to a (never dereferenced) address and an undersized workspace in the LAST field must get
    # past the null checks and stop at the size check; clearing any one pointer must stop at the null check
    fake = 4096
    dims = _lib.MoeDims(world=2, tokens=256, hidden=512, intermediate=256, shared_intermediate=0, num_local_experts=4, topk=2,
                        capacity=1024, num_comm_sms=0, minibatch_size=0)
    need = lib.mx8_moe_fwd_workspace_bytes(ctypes.byref(dims))
    assert need >= 1024 * 512 + 1024 * 256
    bad = _lib.MoeDims(world=2, tokens=256, hidden=500, intermediate=256, num_local_experts=4, topk=2, capacity=1024)
    assert lib.mx8_moe_fwd_workspace_bytes(ctypes.byref(bad)) == 0
    ptrs = (ctypes.c_void_p * 2)(fake, fake)
    shared_only = {"w_shared_gate", "w_shared_up", "w_shared_down", "gate_shared", "up_shared", "hidden_shared", "y_shared"}

    def fwd_args():
        a = _lib.MoeFwdArgs()
        a.dims = dims
        a.x, a.x_ptrs, a.combine_ptrs = fake, ptrs, ptrs
        for name in _lib.FWD_IN + _lib.FWD_OUT:
            setattr(a, name, None if name in shared_only else fake)
        a.workspace, a.workspace_bytes = fake, 1
        return a

    assert lib.mx8_moe_fwd(ctypes.byref(fwd_args()), None) == _lib.ERR_LIMIT
    for name in ("w_gate", "tokens_per_expert", "x_fp8_t", "hidden_sc_t", "y_routed", "workspace"):
        a = fwd_args()
        setattr(a, name, None)
        assert lib.mx8_moe_fwd(ctypes.byref(a), None) == _lib.ERR_ARG, name

    def bwd_args():
        a = _lib.MoeBwdArgs()
        a.dims = dims
        a.d_combine_ptrs, a.d_x_routed_ptrs = ptrs, ptrs
        shared = {"w_shared_gate_T", "w_shared_up_T", "w_shared_down_T", "gate_shared", "up_shared", "hidden_shared", "x", "d_x_shared",
                  "d_gate_shared", "d_up_shared", "d_hidden_shared", "d_w_shared_gate", "d_w_shared_up", "d_w_shared_down"}
        for name in _lib.BWD_IN + _lib.BWD_OUT:
            setattr(a, name, None if name in shared else fake)
        a.workspace, a.workspace_bytes = fake, 1
        return a

    assert lib.mx8_moe_bwd_workspace_bytes(ctypes.byref(dims)) > 0
    assert lib.mx8_moe_bwd(ctypes.byref(bwd_args()), None) == _lib.ERR_LIMIT
    for name in ("w_down_T_sc", "hidden_sc_t", "d_w_down", "d_y_sc"):
        a = bwd_args()
        setattr(a, name, None)
        assert lib.mx8_moe_bwd(ctypes.byref(a), None) == _lib.ERR_ARG, name
