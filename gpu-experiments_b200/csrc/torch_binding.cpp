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
//   schedule(...), dispatch_mlp_swiglu_combine_fwd(...), fwd_epilogue(...)
//                                                         blackwell-ultra/022-…-mxfp8-bw.cu:2996-3030 (forward, routed experts)
// Errors raise RuntimeError (the reference prints and exits).
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <optional>
#include <string>
#include <tuple>
#include <vector>

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

// ---------------------------------------------------------------------------------------------
// MoE forward (routed experts) with the reference's binding signatures
// (blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.cu:2996-3030)

const void* iptr(const at::Tensor& t, const char* name) {
    TORCH_CHECK(t.defined() && t.is_cuda() && t.scalar_type() == at::kInt && t.is_contiguous(), name, " must be a contiguous int32 CUDA tensor");
    return t.data_ptr();
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> schedule(const at::Tensor& topk_all, int num_local_experts,
                                                                    int schedule_capacity, int rank) {
    TORCH_CHECK(topk_all.dim() == 3, "topk_all must be [world, tokens, topk]");
    c10::cuda::CUDAGuard guard(topk_all.device());
    const int world = static_cast<int>(topk_all.size(0));
    auto opt = topk_all.options().dtype(at::kInt);
    at::Tensor peer_rank = at::empty({schedule_capacity}, opt), peer_tok = at::empty({schedule_capacity}, opt);
    at::Tensor num_tokens = at::empty({1}, opt), tpe = at::empty({num_local_experts}, opt);
    const size_t scratch_bytes = mx8_moe_schedule_scratch_bytes(world, static_cast<int>(topk_all.size(1)), static_cast<int>(topk_all.size(2)),
                                                                num_local_experts);
    at::Tensor scratch = at::empty({static_cast<int64_t>(scratch_bytes)}, topk_all.options().dtype(at::kByte));
    check(mx8_moe_schedule(iptr(topk_all, "topk_all"), world, static_cast<int>(topk_all.size(1)), static_cast<int>(topk_all.size(2)),
                           num_local_experts, schedule_capacity, rank, peer_rank.data_ptr(), peer_tok.data_ptr(),
                           num_tokens.data_ptr(), tpe.data_ptr(), scratch.data_ptr(), scratch_bytes, stream()),
          "schedule");
    return {peer_rank, peer_tok, num_tokens, tpe};
}

// pointer of an optional / possibly undefined tensor
const void* optr(const std::optional<at::Tensor>& t) { return (t.has_value() && t->defined()) ? t->data_ptr() : nullptr; }
void* mptr(const at::Tensor& t) { return t.defined() ? t.data_ptr() : nullptr; }

mx8_moe_dims moe_dims(int world, int64_t tokens, int64_t H, int64_t I, int64_t Is, int64_t E, int topk, int64_t cap, int num_comm_sms,
                      int minibatch_size) {
    mx8_moe_dims d{};
    d.world = world;
    d.tokens = static_cast<int>(tokens);
    d.hidden = static_cast<int>(H);
    d.intermediate = static_cast<int>(I);
    d.shared_intermediate = static_cast<int>(Is);
    d.num_local_experts = static_cast<int>(E);
    d.topk = topk;
    d.capacity = static_cast<int>(cap);
    d.num_comm_sms = num_comm_sms;
    d.minibatch_size = minibatch_size;
    return d;
}

// The layer itself is one C-ABI call (mx8_moe_fwd); this function allocates what the reference's host function
// allocates (blackwell-ultra/022-…-mxfp8-bw.cu:2040-2075) and returns its thirteen tensors.
std::vector<at::Tensor> dispatch_mlp_swiglu_combine_fwd(
    const at::Tensor& x, const std::vector<int64_t>& x_ptrs, const at::Tensor& combine_buffer,
    const std::vector<int64_t>& combine_buffer_ptrs, const std::optional<at::Tensor>& w_shared_gate, const at::Tensor& w_routed_gate,
    const at::Tensor& w_routed_gate_sc, const std::optional<at::Tensor>& w_shared_up, const at::Tensor& w_routed_up,
    const at::Tensor& w_routed_up_sc, const std::optional<at::Tensor>& w_shared_down, const at::Tensor& w_routed_down,
    const at::Tensor& w_routed_down_sc, const at::Tensor& schedule_peer_rank, const at::Tensor& schedule_peer_token_idx,
    const at::Tensor& num_tokens, const at::Tensor& tokens_per_expert, int topk, int num_comm_sms, int /*macrobatch_size*/,
    int minibatch_size) {
    TORCH_CHECK(w_routed_gate.dim() == 3 && w_routed_down.dim() == 3, "routed weights must be [E, rows, cols]");
    TORCH_CHECK(x_ptrs.size() == combine_buffer_ptrs.size() && !x_ptrs.empty() && x_ptrs.size() <= 16, "1..16 ranks");
    TORCH_CHECK(x.dim() == 2 && x.scalar_type() == at::kBFloat16, "x must be bf16 [tokens, hidden]");
    (void)combine_buffer;
    c10::cuda::CUDAGuard guard(x.device());
    const int64_t E = w_routed_gate.size(0), I = w_routed_gate.size(1), H = w_routed_gate.size(2), cap = schedule_peer_rank.size(0);
    const int64_t T = x.size(0);
    const bool shared = optr(w_shared_gate) && optr(w_shared_up) && optr(w_shared_down);
    const int64_t Is = shared ? w_shared_gate->size(0) : 0;
    auto fp8 = x.options().dtype(at::kFloat8_e4m3fn);
    auto u8 = x.options().dtype(at::kByte);
    at::Tensor x_fp8_t = at::empty({H, cap}, fp8), x_sc_t = at::empty({H / 128, cap / 128, 32, 16}, u8);
    at::Tensor gate_fp8 = at::empty({cap, I}, fp8), gate_sc = at::empty({cap / 128, I / 128, 32, 16}, u8);
    at::Tensor up_fp8 = at::empty({cap, I}, fp8), up_sc = at::empty({cap / 128, I / 128, 32, 16}, u8);
    at::Tensor h_fp8_t = at::empty({I, cap}, fp8), h_sc_t = at::empty({I / 128, cap / 128, 32, 16}, u8);
    at::Tensor y_routed = at::empty({cap, H}, x.options());
    at::Tensor gate_shared, up_shared, hidden_shared, y_shared;
    if (shared) {
        gate_shared = at::empty({T, Is}, x.options());
        up_shared = at::empty({T, Is}, x.options());
        hidden_shared = at::empty({T, Is}, x.options());
        y_shared = at::empty({T, H}, x.options());
    }
    std::vector<const void*> xp(x_ptrs.size());
    std::vector<void*> cp(x_ptrs.size());
    for (size_t i = 0; i < x_ptrs.size(); ++i) {
        xp[i] = reinterpret_cast<const void*>(x_ptrs[i]);
        cp[i] = reinterpret_cast<void*>(combine_buffer_ptrs[i]);
    }
    mx8_moe_fwd_args a{};
    a.dims = moe_dims(static_cast<int>(x_ptrs.size()), T, H, I, Is, E, topk, cap, num_comm_sms, minibatch_size);
    a.x = dptr(x, "x");
    a.x_ptrs = xp.data();
    a.combine_ptrs = cp.data();
    a.w_shared_gate = shared ? optr(w_shared_gate) : nullptr;
    a.w_shared_up = shared ? optr(w_shared_up) : nullptr;
    a.w_shared_down = shared ? optr(w_shared_down) : nullptr;
    a.w_gate = dptr(w_routed_gate, "w_routed_gate");
    a.w_gate_sc = dptr(w_routed_gate_sc, "w_routed_gate_sc", E * I * H / 32);
    a.w_up = dptr(w_routed_up, "w_routed_up", E * I * H);
    a.w_up_sc = dptr(w_routed_up_sc, "w_routed_up_sc", E * I * H / 32);
    a.w_down = dptr(w_routed_down, "w_routed_down", E * I * H);
    a.w_down_sc = dptr(w_routed_down_sc, "w_routed_down_sc", E * I * H / 32);
    a.peer_rank = iptr(schedule_peer_rank, "schedule_peer_rank");
    a.peer_token_idx = iptr(schedule_peer_token_idx, "schedule_peer_token_idx");
    a.num_tokens = iptr(num_tokens, "num_tokens");
    a.tokens_per_expert = iptr(tokens_per_expert, "tokens_per_expert");
    a.x_fp8_t = x_fp8_t.data_ptr(); a.x_sc_t = x_sc_t.data_ptr();
    a.gate_shared = mptr(gate_shared); a.gate_fp8 = gate_fp8.data_ptr(); a.gate_sc = gate_sc.data_ptr();
    a.up_shared = mptr(up_shared); a.up_fp8 = up_fp8.data_ptr(); a.up_sc = up_sc.data_ptr();
    a.hidden_shared = mptr(hidden_shared); a.hidden_fp8_t = h_fp8_t.data_ptr(); a.hidden_sc_t = h_sc_t.data_ptr();
    a.y_shared = mptr(y_shared); a.y_routed = y_routed.data_ptr();
    const size_t need = mx8_moe_fwd_workspace_bytes(&a.dims);
    TORCH_CHECK(need > 0, "dispatch_mlp_swiglu_combine_fwd: hidden, intermediate and capacity must be multiples of 256");
    at::Tensor ws = at::empty({static_cast<int64_t>(need)}, u8);
    a.workspace = ws.data_ptr();
    a.workspace_bytes = need;
    check(mx8_moe_fwd(&a, stream()), "dispatch_mlp_swiglu_combine_fwd");
    return {x_fp8_t, x_sc_t, gate_shared, gate_fp8, gate_sc, up_shared, up_fp8, up_sc, hidden_shared, h_fp8_t, h_sc_t, y_shared, y_routed};
}

at::Tensor fwd_epilogue(const std::optional<at::Tensor>& y_shared, const at::Tensor& combine_buffer, const at::Tensor& topk_weights) {
    TORCH_CHECK(topk_weights.dim() == 2 && topk_weights.scalar_type() == at::kFloat && topk_weights.is_contiguous(), "topk_weights float32 [tokens, topk]");
    TORCH_CHECK(combine_buffer.scalar_type() == at::kBFloat16 && combine_buffer.is_contiguous(), "combine_buffer must be contiguous bf16");
    c10::cuda::CUDAGuard guard(combine_buffer.device());
    const int64_t T = topk_weights.size(0), k = topk_weights.size(1), H = combine_buffer.size(1);
    TORCH_CHECK(combine_buffer.size(0) == T * k, "combine_buffer must be [tokens * topk, hidden]");
    at::Tensor out = at::empty({T, H}, combine_buffer.options());
    const void* ys = nullptr;
    if (y_shared.has_value() && y_shared->defined()) ys = dptr(*y_shared, "y_shared", T * H);
    check(mx8_moe_fwd_epilogue(ys, combine_buffer.data_ptr(), topk_weights.data_ptr(), out.data_ptr(), static_cast<int>(T),
                               static_cast<int>(H), static_cast<int>(k), stream()),
          "fwd_epilogue");
    return out;
}

// ---------------------------------------------------------------------------------------------
// MoE backward (routed experts), blackwell-ultra/022-…-mxfp8-bw.cu:3011-3034

at::Tensor bwd_prologue(const at::Tensor& d_output, const at::Tensor& topk_weights, const at::Tensor& d_combine_buffer) {
    TORCH_CHECK(topk_weights.dim() == 2 && topk_weights.scalar_type() == at::kFloat && topk_weights.is_contiguous(), "topk_weights float32 [tokens, topk]");
    c10::cuda::CUDAGuard guard(d_output.device());
    const int64_t T = topk_weights.size(0), k = topk_weights.size(1), H = d_output.size(1);
    check(mx8_moe_bwd_prologue(dptr(d_output, "d_output", T * H), topk_weights.data_ptr(),
                               const_cast<void*>(dptr(d_combine_buffer, "d_combine_buffer", T * k * H)), static_cast<int>(T),
                               static_cast<int>(H), static_cast<int>(k), stream()),
          "bwd_prologue");
    return d_output;   // == d_y_shared; the combine buffer is filled in place
}

at::Tensor bwd_epilogue(const at::Tensor& d_x_shared, const at::Tensor& d_x_routed_buffer) {
    c10::cuda::CUDAGuard guard(d_x_shared.device());
    const int64_t T = d_x_shared.size(0), H = d_x_shared.size(1), k = d_x_routed_buffer.size(0) / T;
    at::Tensor d_x = at::empty_like(d_x_shared);
    check(mx8_moe_bwd_epilogue(dptr(d_x_shared, "d_x_shared", T * H), dptr(d_x_routed_buffer, "d_x_routed_buffer", T * k * H),
                               d_x.data_ptr(), static_cast<int>(T), static_cast<int>(H), static_cast<int>(k), stream()),
          "bwd_epilogue");
    return d_x;
}

using OptT = std::optional<at::Tensor>;

// One C-ABI call (mx8_moe_bwd); allocates and returns the eighteen tensors of the reference's backward binding.
std::vector<at::Tensor> dispatch_mlp_swiglu_combine_bwd(
    const OptT& d_y_shared, const at::Tensor& d_combine_buffer, const std::vector<int64_t>& d_combine_buffer_ptrs,
    const at::Tensor& d_x_routed_buffer, const std::vector<int64_t>& d_x_routed_buffer_ptrs, const OptT& w_shared_gate_T,
    const at::Tensor& w_routed_gate_T, const at::Tensor& w_routed_gate_T_sc, const OptT& w_shared_up_T, const at::Tensor& w_routed_up_T,
    const at::Tensor& w_routed_up_T_sc, const OptT& w_shared_down_T, const at::Tensor& w_routed_down_T,
    const at::Tensor& w_routed_down_T_sc, const at::Tensor& x_fp8_t_routed, const at::Tensor& x_sc_t_routed, const OptT& gate_shared,
    const at::Tensor& gate_fp8_routed, const at::Tensor& gate_sc_routed, const OptT& up_shared, const at::Tensor& up_fp8_routed,
    const at::Tensor& up_sc_routed, const OptT& hidden_shared, const at::Tensor& hidden_fp8_t_routed,
    const at::Tensor& hidden_sc_t_routed, const OptT& x_buffer, const std::vector<int64_t>& /*x_buffer_ptrs*/,
    const OptT& /*w_routed_gate*/, const OptT& /*w_routed_gate_sc*/, const OptT& /*w_routed_up*/, const OptT& /*w_routed_up_sc*/,
    const at::Tensor& schedule_peer_rank, const at::Tensor& schedule_peer_token_idx, const at::Tensor& num_tokens,
    const at::Tensor& tokens_per_expert, int topk, int num_comm_sms, int /*macrobatch_size*/, int minibatch_size) {
    TORCH_CHECK(w_routed_gate_T.dim() == 3, "transposed routed weights must be [E, H, I]");
    TORCH_CHECK(!d_combine_buffer_ptrs.empty() && d_combine_buffer_ptrs.size() == d_x_routed_buffer_ptrs.size() &&
                d_combine_buffer_ptrs.size() <= 16, "1..16 ranks");
    TORCH_CHECK(topk > 0 && d_combine_buffer.dim() == 2 && d_combine_buffer.size(0) % topk == 0, "d_combine_buffer must be [tokens * topk, hidden]");
    (void)d_x_routed_buffer;
    c10::cuda::CUDAGuard guard(d_combine_buffer.device());
    const int64_t E = w_routed_gate_T.size(0), H = w_routed_gate_T.size(1), I = w_routed_gate_T.size(2), cap = schedule_peer_rank.size(0);
    const int64_t T = d_combine_buffer.size(0) / topk;
    const int world = static_cast<int>(d_combine_buffer_ptrs.size());
    const bool shared = optr(d_y_shared) && optr(w_shared_gate_T) && optr(w_shared_up_T) && optr(w_shared_down_T) && optr(gate_shared) &&
                        optr(up_shared) && optr(hidden_shared) && optr(x_buffer);
    const int64_t Is = shared ? gate_shared->size(1) : 0;
    auto bf = d_combine_buffer.options();
    auto fp8 = bf.dtype(at::kFloat8_e4m3fn);
    auto u8 = bf.dtype(at::kByte);
    at::Tensor d_y_fp8 = at::empty({cap, H}, fp8), d_y_sc = at::empty({cap / 128, H / 128, 32, 16}, u8);
    at::Tensor d_gate_fp8 = at::empty({cap, I}, fp8), d_gate_sc = at::empty({cap / 128, I / 128, 32, 16}, u8);
    at::Tensor d_up_fp8 = at::empty({cap, I}, fp8), d_up_sc = at::empty({cap / 128, I / 128, 32, 16}, u8);
    at::Tensor d_hidden = at::empty({cap, I}, bf), d_x_routed = at::empty({cap, H}, bf);
    at::Tensor d_w_gate = at::empty({E, I, H}, bf), d_w_up = at::empty({E, I, H}, bf), d_w_down = at::empty({E, H, I}, bf);
    at::Tensor d_x_shared, d_gate_shared, d_up_shared, d_hidden_shared, d_w_sg, d_w_su, d_w_sd;
    if (shared) {
        d_x_shared = at::empty({T, H}, bf);
        d_gate_shared = at::empty({T, Is}, bf);
        d_up_shared = at::empty({T, Is}, bf);
        d_hidden_shared = at::empty({T, Is}, bf);
        d_w_sg = at::empty({Is, H}, bf);
        d_w_su = at::empty({Is, H}, bf);
        d_w_sd = at::empty({H, Is}, bf);
    }
    std::vector<const void*> src(world);
    std::vector<void*> dst(world);
    for (int i = 0; i < world; ++i) {
        src[i] = reinterpret_cast<const void*>(d_combine_buffer_ptrs[i]);
        dst[i] = reinterpret_cast<void*>(d_x_routed_buffer_ptrs[i]);
    }
    mx8_moe_bwd_args a{};
    a.dims = moe_dims(world, T, H, I, Is, E, topk, cap, num_comm_sms, minibatch_size);
    a.d_y_shared = shared ? optr(d_y_shared) : nullptr;
    a.d_combine_ptrs = src.data();
    a.d_x_routed_ptrs = dst.data();
    a.w_shared_gate_T = shared ? optr(w_shared_gate_T) : nullptr;
    a.w_shared_up_T = shared ? optr(w_shared_up_T) : nullptr;
    a.w_shared_down_T = shared ? optr(w_shared_down_T) : nullptr;
    a.w_gate_T = dptr(w_routed_gate_T, "w_routed_gate_T"); a.w_gate_T_sc = dptr(w_routed_gate_T_sc, "w_routed_gate_T_sc", E * I * H / 32);
    a.w_up_T = dptr(w_routed_up_T, "w_routed_up_T", E * I * H); a.w_up_T_sc = dptr(w_routed_up_T_sc, "w_routed_up_T_sc", E * I * H / 32);
    a.w_down_T = dptr(w_routed_down_T, "w_routed_down_T", E * I * H); a.w_down_T_sc = dptr(w_routed_down_T_sc, "w_routed_down_T_sc", E * I * H / 32);
    a.x_fp8_t = dptr(x_fp8_t_routed, "x_fp8_t_routed", cap * H); a.x_sc_t = dptr(x_sc_t_routed, "x_sc_t_routed", cap * H / 32);
    a.gate_shared = shared ? optr(gate_shared) : nullptr;
    a.gate_fp8 = dptr(gate_fp8_routed, "gate_fp8_routed", cap * I); a.gate_sc = dptr(gate_sc_routed, "gate_sc_routed", cap * I / 32);
    a.up_shared = shared ? optr(up_shared) : nullptr;
    a.up_fp8 = dptr(up_fp8_routed, "up_fp8_routed", cap * I); a.up_sc = dptr(up_sc_routed, "up_sc_routed", cap * I / 32);
    a.hidden_shared = shared ? optr(hidden_shared) : nullptr;
    a.hidden_fp8_t = dptr(hidden_fp8_t_routed, "hidden_fp8_t_routed", cap * I);
    a.hidden_sc_t = dptr(hidden_sc_t_routed, "hidden_sc_t_routed", cap * I / 32);
    a.x = shared ? optr(x_buffer) : nullptr;
    a.peer_rank = iptr(schedule_peer_rank, "schedule_peer_rank");
    a.peer_token_idx = iptr(schedule_peer_token_idx, "schedule_peer_token_idx");
    a.num_tokens = iptr(num_tokens, "num_tokens");
    a.tokens_per_expert = iptr(tokens_per_expert, "tokens_per_expert");
    a.d_x_shared = mptr(d_x_shared); a.d_x_routed = d_x_routed.data_ptr();
    a.d_gate_shared = mptr(d_gate_shared); a.d_gate_fp8 = d_gate_fp8.data_ptr(); a.d_gate_sc = d_gate_sc.data_ptr();
    a.d_up_shared = mptr(d_up_shared); a.d_up_fp8 = d_up_fp8.data_ptr(); a.d_up_sc = d_up_sc.data_ptr();
    a.d_hidden_shared = mptr(d_hidden_shared); a.d_hidden_routed = d_hidden.data_ptr();
    a.d_y_fp8 = d_y_fp8.data_ptr(); a.d_y_sc = d_y_sc.data_ptr();
    a.d_w_shared_gate = mptr(d_w_sg); a.d_w_gate = d_w_gate.data_ptr();
    a.d_w_shared_up = mptr(d_w_su); a.d_w_up = d_w_up.data_ptr();
    a.d_w_shared_down = mptr(d_w_sd); a.d_w_down = d_w_down.data_ptr();
    const size_t need = mx8_moe_bwd_workspace_bytes(&a.dims);
    TORCH_CHECK(need > 0, "dispatch_mlp_swiglu_combine_bwd: hidden, intermediate and capacity must be multiples of 256");
    at::Tensor ws = at::empty({static_cast<int64_t>(need)}, u8);
    a.workspace = ws.data_ptr();
    a.workspace_bytes = need;
    check(mx8_moe_bwd(&a, stream()), "dispatch_mlp_swiglu_combine_bwd");
    return {d_x_shared, d_x_routed, d_gate_shared, d_gate_fp8, d_gate_sc, d_up_shared, d_up_fp8, d_up_sc, d_hidden_shared, d_hidden,
            d_y_fp8, d_y_sc, d_w_sg, d_w_gate, d_w_su, d_w_up, d_w_sd, d_w_down};
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
    m.def("schedule", &schedule, "", pybind11::arg("topk_all"), pybind11::arg("num_local_experts"), pybind11::arg("schedule_capacity"),
          pybind11::arg("rank"));
    m.def("dispatch_mlp_swiglu_combine_fwd", &dispatch_mlp_swiglu_combine_fwd, "", pybind11::arg("x"), pybind11::arg("x_ptrs"),
          pybind11::arg("combine_buffer"), pybind11::arg("combine_buffer_ptrs"), pybind11::arg("w_shared_gate"),
          pybind11::arg("w_routed_gate"), pybind11::arg("w_routed_gate_sc"), pybind11::arg("w_shared_up"), pybind11::arg("w_routed_up"),
          pybind11::arg("w_routed_up_sc"), pybind11::arg("w_shared_down"), pybind11::arg("w_routed_down"),
          pybind11::arg("w_routed_down_sc"), pybind11::arg("schedule_peer_rank"), pybind11::arg("schedule_peer_token_idx"),
          pybind11::arg("num_tokens"), pybind11::arg("tokens_per_expert"), pybind11::arg("topk"), pybind11::arg("num_comm_sms") = 0,
          pybind11::arg("macrobatch_size") = 0, pybind11::arg("minibatch_size") = 0);
    m.def("fwd_epilogue", &fwd_epilogue, "", pybind11::arg("y_shared"), pybind11::arg("combine_buffer"), pybind11::arg("topk_weights"));
    m.def("bwd_prologue", &bwd_prologue);
    m.def("bwd_epilogue", &bwd_epilogue);
    m.def("dispatch_mlp_swiglu_combine_bwd", &dispatch_mlp_swiglu_combine_bwd);
    m.def("device_status", &device_status);
    m.def("version", []() { return std::string(mx8_version()); });
}
