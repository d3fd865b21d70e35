// C++ host layer over the mx8 C ABI: a pybind11/torch extension module named `_C` with the call
// signatures of the reference's harness-facing bindings.  It only validates tensors, picks the
// current CUDA stream and forwards raw pointers to libmx8.so; all arithmetic lives behind the C ABI.
//
//   mxfp8_quantize(x_bf16, x_fp8, x_sc, x_fp8_t, x_sc_t, return_normal, return_transposed) -> None
//       blackwell-ultra/019-mxfp8-quantize.cu:185-219
//   mxfp8_quantize(x_bf16, return_normal, return_transposed) -> (x_fp8, x_sc, x_fp8_t, x_sc_t)
//       blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.cu:404-448
//   kernel(A_fp8, A_sc, B_fp8, B_sc, C) -> None          blackwell/047-mxfp8-mma-2cta-MNK128-polished.cu:532-541
//   kernel(A, A_fp8, A_sc[, A_t_fp8, A_t_sc]) -> None     blackwell/018-mxfp8-quantize.cu:288-293,
//                                                         blackwell/038-mxfp8-quantize-combined.cu:397-399
//   kernel_transpose(A, A_t_fp8, A_t_sc) -> None          blackwell/018-mxfp8-quantize.cu:294-300
// Errors raise RuntimeError (the reference prints and exits).
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <optional>
#include <string>
#include <tuple>

#include "../../include/mx8.h"

namespace {

void check(int rc, const char* where) {
    if (rc == MX8_OK) return;
    std::string msg = std::string(where) + ": mx8 status " + std::to_string(rc) + ": " + mx8_strerror(rc);
    if (rc == MX8_ERR_CUDA) msg += std::string(" [") + mx8_last_cuda_error() + "]";
    throw std::runtime_error(msg);
}

void* stream() { return static_cast<void*>(c10::cuda::getCurrentCUDAStream().stream()); }

const void* dptr(const at::Tensor& t, const char* name, int64_t numel = -1) {
    TORCH_CHECK(t.defined() && t.is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
    TORCH_CHECK(numel < 0 || t.numel() == numel, name, " has ", t.numel(), " elements, expected ", numel);
    return t.data_ptr();
}

bool is_fp8_or_u8(const at::Tensor& t) { return t.element_size() == 1; }

void quantize_into(const at::Tensor& x, const at::Tensor& x_fp8, const at::Tensor& x_sc, const at::Tensor& x_fp8_t,
                   const at::Tensor& x_sc_t, bool rn, bool rt, int mode) {
    TORCH_CHECK(x.dim() == 2 || x.dim() == 3, "x_bf16 must be [M, N] or [E, M, N]");
    TORCH_CHECK(x.scalar_type() == at::kBFloat16, "x_bf16 must be bfloat16");
    TORCH_CHECK(rn || rt, "at least one of return_normal / return_transposed must be set");
    const int64_t E = x.dim() == 3 ? x.size(0) : 1, M = x.size(-2), N = x.size(-1);
    c10::cuda::CUDAGuard guard(x.device());
    const void* xp = dptr(x, "x_bf16");
    void *p0 = nullptr, *p1 = nullptr, *p2 = nullptr, *p3 = nullptr;
    if (rn) {
        TORCH_CHECK(is_fp8_or_u8(x_fp8) && is_fp8_or_u8(x_sc), "x_fp8 / x_sc must be 1-byte types");
        p0 = const_cast<void*>(dptr(x_fp8, "x_fp8", E * M * N));
        p1 = const_cast<void*>(dptr(x_sc, "x_sc", E * M * N / 32));
    }
    if (rt) {
        TORCH_CHECK(is_fp8_or_u8(x_fp8_t) && is_fp8_or_u8(x_sc_t), "x_fp8_t / x_sc_t must be 1-byte types");
        p2 = const_cast<void*>(dptr(x_fp8_t, "x_fp8_t", E * M * N));
        p3 = const_cast<void*>(dptr(x_sc_t, "x_sc_t", E * M * N / 32));
    }
    check(mx8_quantize(xp, static_cast<int>(E), static_cast<int>(M), static_cast<int>(N), p0, p1, p2, p3, mode, stream()),
          "mxfp8_quantize");
}

void mxfp8_quantize_out(const at::Tensor& x, const at::Tensor& x_fp8, const at::Tensor& x_sc, const at::Tensor& x_fp8_t,
                        const at::Tensor& x_sc_t, bool rn, bool rt, int scale_mode) {
    quantize_into(x, x_fp8, x_sc, x_fp8_t, x_sc_t, rn, rt, scale_mode);
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> mxfp8_quantize_alloc(const at::Tensor& x, bool rn, bool rt,
                                                                                int scale_mode) {
    TORCH_CHECK(x.dim() == 2 || x.dim() == 3, "x_bf16 must be [M, N] or [E, M, N]");
    const int64_t E = x.dim() == 3 ? x.size(0) : 1, M = x.size(-2), N = x.size(-1);
    TORCH_CHECK(M % 128 == 0 && N % 128 == 0, "M and N must be multiples of 128");
    auto fp8 = x.options().dtype(at::kFloat8_e4m3fn);
    auto u8 = x.options().dtype(at::kByte);
    at::Tensor q, sc, qt, sct;      // outputs that are not requested stay undefined (None in Python)
    if (rn) {
        q = x.dim() == 3 ? at::empty({E, M, N}, fp8) : at::empty({M, N}, fp8);
        sc = at::empty({E * M / 128, N / 128, 32, 16}, u8);
    }
    if (rt) {
        qt = x.dim() == 3 ? at::empty({E, N, M}, fp8) : at::empty({N, M}, fp8);
        sct = at::empty({E * N / 128, M / 128, 32, 16}, u8);
    }
    quantize_into(x, q, sc, qt, sct, rn, rt, scale_mode);
    return {q, sc, qt, sct};
}

void gemm(const at::Tensor& A, const at::Tensor& A_sc, const at::Tensor& B, const at::Tensor& B_sc, const at::Tensor& C) {
    TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && C.dim() == 2, "A [M,K], B [N,K], C [M,N]");
    const int64_t M = A.size(0), K = A.size(1), N = B.size(0);
    TORCH_CHECK(B.size(1) == K && C.size(0) == M && C.size(1) == N, "shape mismatch: A [M,K], B [N,K], C [M,N]");
    TORCH_CHECK(is_fp8_or_u8(A) && is_fp8_or_u8(B) && is_fp8_or_u8(A_sc) && is_fp8_or_u8(B_sc), "operands must be 1-byte types");
    TORCH_CHECK(C.scalar_type() == at::kBFloat16 || C.scalar_type() == at::kFloat, "C must be bfloat16 or float32");
    c10::cuda::CUDAGuard guard(A.device());
    check(mx8_gemm(dptr(A, "A"), dptr(A_sc, "A_sc", M * K / 32), dptr(B, "B"), dptr(B_sc, "B_sc", N * K / 32),
                   const_cast<void*>(dptr(C, "C")), static_cast<int>(M), static_cast<int>(N), static_cast<int>(K),
                   C.scalar_type() == at::kFloat ? MX8_C_F32 : MX8_C_BF16, stream()),
          "kernel");
}

// `kernel` is the name of both the GEMM binding and the older quantize bindings in the reference;
// a bf16 first argument selects the quantizer.
void kernel(const at::Tensor& a0, const at::Tensor& a1, const at::Tensor& a2, const std::optional<at::Tensor>& a3,
            const std::optional<at::Tensor>& a4) {
    if (a0.scalar_type() == at::kBFloat16) {
        if (a3.has_value() && a4.has_value()) quantize_into(a0, a1, a2, *a3, *a4, true, true, MX8_SCALE_RCEIL);
        else quantize_into(a0, a1, a2, at::Tensor(), at::Tensor(), true, false, MX8_SCALE_RCEIL);
        return;
    }
    TORCH_CHECK(a3.has_value() && a4.has_value(), "kernel(A_fp8, A_sc, B_fp8, B_sc, C) takes five tensors");
    gemm(a0, a1, a2, *a3, *a4);
}

void kernel_transpose(const at::Tensor& A, const at::Tensor& A_t_fp8, const at::Tensor& A_t_sc) {
    quantize_into(A, at::Tensor(), at::Tensor(), A_t_fp8, A_t_sc, false, true, MX8_SCALE_RCEIL);
}

int device_status() {
    int v = 0;
    int rc = mx8_device_status(&v, stream());
    if (rc != MX8_OK && rc != MX8_ERR_DEVICE_TIMEOUT) check(rc, "device_status");
    return v;
}

}  // namespace

PYBIND11_MODULE(_C, m) {
    m.doc() = "mx8: MXFP8 quantize and block-scaled GEMM for sm_100a (host layer over the C ABI in include/mx8.h)";
    m.def("mxfp8_quantize", &mxfp8_quantize_out, "", pybind11::arg("x_bf16"), pybind11::arg("x_fp8"), pybind11::arg("x_sc"),
          pybind11::arg("x_fp8_t"), pybind11::arg("x_sc_t"), pybind11::arg("return_normal"), pybind11::arg("return_transposed"),
          pybind11::arg("scale_mode") = static_cast<int>(MX8_SCALE_RCEIL));
    m.def("mxfp8_quantize", &mxfp8_quantize_alloc, "", pybind11::arg("x_bf16"), pybind11::arg("return_normal"),
          pybind11::arg("return_transposed"), pybind11::arg("scale_mode") = static_cast<int>(MX8_SCALE_RCEIL));
    m.def("kernel", &kernel, "", pybind11::arg("a0"), pybind11::arg("a1"), pybind11::arg("a2"),
          pybind11::arg("a3") = std::nullopt, pybind11::arg("a4") = std::nullopt);
    m.def("kernel_transpose", &kernel_transpose);
    m.def("device_status", &device_status);
    m.def("version", []() { return std::string(mx8_version()); });
}
