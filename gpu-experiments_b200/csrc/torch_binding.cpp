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
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDACachingAllocator.h>
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

void grouped(const at::Tensor& A, const at::Tensor& A_sc, const at::Tensor& B, const at::Tensor& B_sc, const at::Tensor& C,
             const at::Tensor& C_sc, const at::Tensor& num_tokens, const at::Tensor& tokens_per_expert) {
    const bool q = C_sc.defined();
    check(mx8_gemm_grouped(A.data_ptr(), A_sc.data_ptr(), B.data_ptr(), B_sc.data_ptr(), C.data_ptr(), q ? C_sc.data_ptr() : nullptr,
                           static_cast<int>(A.size(0)), static_cast<int>(B.size(1)), static_cast<int>(A.size(1)),
                           q ? MX8_C_MXFP8 : MX8_C_BF16, num_tokens.data_ptr(), tokens_per_expert.data_ptr(),
                           static_cast<int>(B.size(0)), stream()),
          "expert grouped gemm");
}

// ---- shared (bf16) expert: the kind::f16 form of the GEMM kernel and its element-wise companions
at::Tensor bf16_gemm(const at::Tensor& a, const at::Tensor& b, const at::Tensor* a2 = nullptr, const at::Tensor* b2 = nullptr) {
    const int64_t M = a.size(0), K = a.size(1), N = b.size(0), K2 = a2 ? a2->size(1) : 0;
    at::Tensor c = at::empty({M, N}, a.options().dtype(at::kBFloat16));
    check(mx8_gemm_bf16_dual(dptr(a, "A", M * K), dptr(b, "B", N * K), a2 ? dptr(*a2, "A2", M * K2) : nullptr,
                             b2 ? dptr(*b2, "B2", N * K2) : nullptr, c.data_ptr(), static_cast<int>(M), static_cast<int>(N),
                             static_cast<int>(K), static_cast<int>(K2), MX8_C_BF16, stream()),
          "bf16 gemm");
    return c;
}

at::Tensor bf16_transpose(const at::Tensor& x) {
    at::Tensor out = at::empty({x.size(1), x.size(0)}, x.options());
    check(mx8_transpose_bf16(dptr(x, "x"), out.data_ptr(), static_cast<int>(x.size(0)), static_cast<int>(x.size(1)), stream()),
          "bf16 transpose");
    return out;
}

// two side streams per device for the transfer legs of the pipelined layer, taken from torch's pool once
std::pair<c10::cuda::CUDAStream, c10::cuda::CUDAStream> side_streams(c10::DeviceIndex dev) {
    static std::vector<std::optional<std::pair<c10::cuda::CUDAStream, c10::cuda::CUDAStream>>> cache(64);
    auto& slot = cache[static_cast<size_t>(dev) & 63];
    if (!slot.has_value()) slot.emplace(c10::cuda::getStreamFromPool(false, dev), c10::cuda::getStreamFromPool(false, dev));
    return *slot;
}

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
    c10::cuda::CUDAGuard guard(x.device());
    const int64_t I = w_routed_gate.size(1), H = w_routed_gate.size(2), cap = schedule_peer_rank.size(0);
    auto fp8 = x.options().dtype(at::kFloat8_e4m3fn);
    auto u8 = x.options().dtype(at::kByte);
    at::Tensor x_fp8 = at::empty({cap, H}, fp8), x_sc = at::empty({cap / 128, H / 128, 32, 16}, u8);
    at::Tensor x_fp8_t = at::empty({H, cap}, fp8), x_sc_t = at::empty({H / 128, cap / 128, 32, 16}, u8);
    at::Tensor gate_fp8 = at::empty({cap, I}, fp8), gate_sc = at::empty({cap / 128, I / 128, 32, 16}, u8);
    at::Tensor up_fp8 = at::empty({cap, I}, fp8), up_sc = at::empty({cap / 128, I / 128, 32, 16}, u8);
    at::Tensor h_fp8 = at::empty({cap, I}, fp8), h_sc = at::empty({cap / 128, I / 128, 32, 16}, u8);
    at::Tensor h_fp8_t = at::empty({I, cap}, fp8), h_sc_t = at::empty({I / 128, cap / 128, 32, 16}, u8);
    at::Tensor y_routed = at::empty({cap, H}, x.options());
    std::vector<const void*> xp(x_ptrs.size());
    std::vector<void*> cp(x_ptrs.size());
    for (size_t i = 0; i < x_ptrs.size(); ++i) {
        xp[i] = reinterpret_cast<const void*>(x_ptrs[i]);
        cp[i] = reinterpret_cast<void*>(combine_buffer_ptrs[i]);
    }
    const int world = static_cast<int>(x_ptrs.size());
    const int E = static_cast<int>(w_routed_gate.size(0));
    int nb = 1;
    if (num_comm_sms > 0 && minibatch_size > 0) nb = static_cast<int>(std::min<int64_t>(E, (cap + minibatch_size - 1) / minibatch_size));
    if (nb > 1) {
        // Minibatches of consecutive experts: dispatch of group b+1 (num_comm_sms multiprocessors, own stream) and
        // combine of group b-1 (third stream) run beside the GEMMs of group b.  Same kernels on row windows, so the
        // outputs are bit-identical to the single sequence below.
        const c10::cuda::CUDAStream main = c10::cuda::getCurrentCUDAStream();
        const auto [s_disp, s_comb] = side_streams(main.device_index());
        at::Tensor bounds = at::empty({nb + 1}, schedule_peer_rank.options());
        int sms = 0;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, main.device_index());
        const int math_sms = std::max(2, (sms - num_comm_sms) & ~1);
        check(mx8_moe_minibatch_bounds(iptr(tokens_per_expert, "tokens_per_expert"), E, nb, bounds.data_ptr(), main.stream()), "minibatch bounds");
        const int* bp = static_cast<const int*>(bounds.data_ptr());
        at::cuda::CUDAEvent start;
        start.record(main);
        start.block(s_disp);
        start.block(s_comb);
        std::vector<at::cuda::CUDAEvent> disp_done(nb);
        for (int b = 0; b < nb; ++b) {
            const mx8_window w{bp + b, bp + b + 1, b == 0 ? 0 : num_comm_sms};
            check(mx8_moe_dispatch_quantize_window(xp.data(), world, static_cast<int>(H), topk, iptr(schedule_peer_rank, "schedule_peer_rank"),
                                                   iptr(schedule_peer_token_idx, "schedule_peer_token_idx"), iptr(num_tokens, "num_tokens"),
                                                   static_cast<int>(cap), x_fp8.data_ptr(), x_sc.data_ptr(), x_fp8_t.data_ptr(),
                                                   x_sc_t.data_ptr(), &w, s_disp.stream()),
                  "dispatch + quantize (window)");
            disp_done[b].record(s_disp);
        }
        auto gemm_w = [&](const at::Tensor& a, const at::Tensor& a_sc, const at::Tensor& wt, const at::Tensor& wt_sc, const at::Tensor& c,
                          const at::Tensor& c_sc, const mx8_window& w) {
            const bool q = c_sc.defined();
            check(mx8_gemm_grouped_window(a.data_ptr(), a_sc.data_ptr(), dptr(wt, "w"), dptr(wt_sc, "w_sc"), c.data_ptr(),
                                          q ? c_sc.data_ptr() : nullptr, static_cast<int>(a.size(0)), static_cast<int>(wt.size(1)),
                                          static_cast<int>(a.size(1)), q ? MX8_C_MXFP8 : MX8_C_BF16, num_tokens.data_ptr(),
                                          tokens_per_expert.data_ptr(), E, &w, main.stream()),
                  "grouped gemm (window)");
        };
        for (int b = 0; b < nb; ++b) {
            disp_done[b].block(main);
            const mx8_window w{bp + b, bp + b + 1, b == nb - 1 ? 0 : math_sms};
            gemm_w(x_fp8, x_sc, w_routed_gate, w_routed_gate_sc, gate_fp8, gate_sc, w);
            gemm_w(x_fp8, x_sc, w_routed_up, w_routed_up_sc, up_fp8, up_sc, w);
            check(mx8_swiglu_quantize_window(gate_fp8.data_ptr(), gate_sc.data_ptr(), up_fp8.data_ptr(), up_sc.data_ptr(), static_cast<int>(cap),
                                             static_cast<int>(I), num_tokens.data_ptr(), h_fp8.data_ptr(), h_sc.data_ptr(), h_fp8_t.data_ptr(),
                                             h_sc_t.data_ptr(), nullptr, &w, main.stream()),
                  "swiglu + quantize (window)");
            gemm_w(h_fp8, h_sc, w_routed_down, w_routed_down_sc, y_routed, at::Tensor(), w);
            at::cuda::CUDAEvent math_done;
            math_done.record(main);
            math_done.block(s_comb);
            // beside GEMMs the combine is held to a few thread blocks: more only queue stores in front of the NVLink ports
            const mx8_window wc{bp + b, bp + b + 1, b < nb - 1 ? std::max(1, num_comm_sms / 4) : 0};
            check(mx8_moe_combine_window(y_routed.data_ptr(), schedule_peer_rank.data_ptr(), schedule_peer_token_idx.data_ptr(),
                                         num_tokens.data_ptr(), static_cast<int>(H), cp.data(), world, &wc, s_comb.stream()),
                  "combine (window)");
        }
        at::cuda::CUDAEvent done;
        done.record(s_comb);
        done.block(main);
        // memory touched by the side streams must not be handed out again before their work has finished
        for (const at::Tensor* t : {&x_fp8, &x_sc, &x_fp8_t, &x_sc_t, &y_routed, &bounds}) {
            c10::cuda::CUDACachingAllocator::recordStream(t->storage().data_ptr(), s_disp);
            c10::cuda::CUDACachingAllocator::recordStream(t->storage().data_ptr(), s_comb);
        }
    } else {
        check(mx8_moe_dispatch_quantize(xp.data(), world, static_cast<int>(H), topk, iptr(schedule_peer_rank, "schedule_peer_rank"),
                                        iptr(schedule_peer_token_idx, "schedule_peer_token_idx"), iptr(num_tokens, "num_tokens"),
                                        static_cast<int>(cap), x_fp8.data_ptr(), x_sc.data_ptr(), x_fp8_t.data_ptr(), x_sc_t.data_ptr(), stream()),
              "dispatch + quantize");
        grouped(x_fp8, x_sc, w_routed_gate, w_routed_gate_sc, gate_fp8, gate_sc, num_tokens, tokens_per_expert);
        grouped(x_fp8, x_sc, w_routed_up, w_routed_up_sc, up_fp8, up_sc, num_tokens, tokens_per_expert);
        check(mx8_swiglu_quantize(gate_fp8.data_ptr(), gate_sc.data_ptr(), up_fp8.data_ptr(), up_sc.data_ptr(), static_cast<int>(cap),
                                  static_cast<int>(I), num_tokens.data_ptr(), h_fp8.data_ptr(), h_sc.data_ptr(), h_fp8_t.data_ptr(),
                                  h_sc_t.data_ptr(), nullptr, stream()),
              "swiglu + quantize");
        grouped(h_fp8, h_sc, w_routed_down, w_routed_down_sc, y_routed, at::Tensor(), num_tokens, tokens_per_expert);
        check(mx8_moe_combine(y_routed.data_ptr(), schedule_peer_rank.data_ptr(), schedule_peer_token_idx.data_ptr(), num_tokens.data_ptr(),
                              static_cast<int>(H), cp.data(), world, stream()),
              "combine");
    }
    // shared expert (bf16), when its weights are given
    at::Tensor gate_shared, up_shared, hidden_shared, y_shared;
    if (w_shared_gate.has_value() && w_shared_up.has_value() && w_shared_down.has_value()) {
        gate_shared = bf16_gemm(x, *w_shared_gate);
        up_shared = bf16_gemm(x, *w_shared_up);
        hidden_shared = at::empty_like(gate_shared);
        check(mx8_swiglu_bf16(gate_shared.data_ptr(), up_shared.data_ptr(), hidden_shared.data_ptr(), gate_shared.numel(), stream()),
              "shared swiglu");
        y_shared = bf16_gemm(hidden_shared, *w_shared_down);
    }
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
    const at::Tensor& tokens_per_expert, int /*topk*/, int num_comm_sms, int /*macrobatch_size*/, int minibatch_size) {
    TORCH_CHECK(w_routed_gate_T.dim() == 3, "transposed routed weights must be [E, H, I]");
    TORCH_CHECK(!d_combine_buffer_ptrs.empty() && d_combine_buffer_ptrs.size() == d_x_routed_buffer_ptrs.size() &&
                d_combine_buffer_ptrs.size() <= 16, "1..16 ranks");
    c10::cuda::CUDAGuard guard(d_combine_buffer.device());
    const int64_t E = w_routed_gate_T.size(0), H = w_routed_gate_T.size(1), I = w_routed_gate_T.size(2), cap = schedule_peer_rank.size(0);
    const int world = static_cast<int>(d_combine_buffer_ptrs.size());
    auto bf = d_combine_buffer.options();
    auto fp8 = bf.dtype(at::kFloat8_e4m3fn);
    auto u8 = bf.dtype(at::kByte);
    auto q = [&](int64_t r, int64_t c) { return std::make_tuple(at::empty({r, c}, fp8), at::empty({r / 128, c / 128, 32, 16}, u8)); };
    auto [d_y_fp8, d_y_sc] = q(cap, H);
    auto [d_y_fp8_t, d_y_sc_t] = q(H, cap);
    auto [d_gate_fp8, d_gate_sc] = q(cap, I);
    auto [d_gate_fp8_t, d_gate_sc_t] = q(I, cap);
    auto [d_up_fp8, d_up_sc] = q(cap, I);
    auto [d_up_fp8_t, d_up_sc_t] = q(I, cap);
    at::Tensor d_hidden = at::empty({cap, I}, bf), d_x_routed = at::empty({cap, H}, bf);
    at::Tensor d_w_gate = at::empty({E, I, H}, bf), d_w_up = at::empty({E, I, H}, bf), d_w_down = at::empty({E, H, I}, bf);
    std::vector<const void*> src(world);
    std::vector<void*> dst(world);
    for (int i = 0; i < world; ++i) {
        src[i] = reinterpret_cast<const void*>(d_combine_buffer_ptrs[i]);
        dst[i] = reinterpret_cast<void*>(d_x_routed_buffer_ptrs[i]);
    }
    // With num_comm_sms and minibatch_size set, the experts are cut into minibatches: gradient dispatch of group b+1
    // (own stream, num_comm_sms multiprocessors) and gradient combine of group b-1 (third stream) run beside the data-
    // gradient GEMMs of group b; otherwise everything is one sequence on the current stream.  Same kernels, same bytes.
    int nb = 1;
    if (num_comm_sms > 0 && minibatch_size > 0) nb = static_cast<int>(std::min<int64_t>(E, (cap + minibatch_size - 1) / minibatch_size));
    const bool pipe = nb > 1;
    const c10::cuda::CUDAStream main = c10::cuda::getCurrentCUDAStream();
    c10::cuda::CUDAStream s_disp = main, s_comb = main;
    at::Tensor bounds;
    const int* bp = nullptr;
    int math_sms = 0;
    if (pipe) {
        std::tie(s_disp, s_comb) = side_streams(main.device_index());
        bounds = at::empty({nb + 1}, schedule_peer_rank.options());
        bp = static_cast<const int*>(bounds.data_ptr());
        int sms = 0;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, main.device_index());
        math_sms = std::max(2, (sms - num_comm_sms) & ~1);
        check(mx8_moe_minibatch_bounds(iptr(tokens_per_expert, "tokens_per_expert"), static_cast<int>(E), nb, bounds.data_ptr(), main.stream()),
              "minibatch bounds");
        at::cuda::CUDAEvent start;
        start.record(main);
        start.block(s_disp);
        start.block(s_comb);
    }
    std::vector<at::cuda::CUDAEvent> disp_done(nb);
    for (int b = 0; b < nb; ++b) {
        const mx8_window w{pipe ? bp + b : nullptr, pipe ? bp + b + 1 : nullptr, (pipe && b > 0) ? num_comm_sms : 0};
        // gradient rows of the routed outputs: one row per (token, k) pair, hence topk = 1 for the index
        check(mx8_moe_dispatch_quantize_window(src.data(), world, static_cast<int>(H), 1, iptr(schedule_peer_rank, "schedule_peer_rank"),
                                               iptr(schedule_peer_token_idx, "schedule_peer_token_idx"), iptr(num_tokens, "num_tokens"),
                                               static_cast<int>(cap), d_y_fp8.data_ptr(), d_y_sc.data_ptr(), d_y_fp8_t.data_ptr(),
                                               d_y_sc_t.data_ptr(), &w, s_disp.stream()),
              "gradient dispatch + quantize");
        if (pipe) disp_done[b].record(s_disp);
    }
    for (int b = 0; b < nb; ++b) {
        if (pipe) disp_done[b].block(main);
        const mx8_window w{pipe ? bp + b : nullptr, pipe ? bp + b + 1 : nullptr, (pipe && b < nb - 1) ? math_sms : 0};
        check(mx8_gemm_grouped_window(d_y_fp8.data_ptr(), d_y_sc.data_ptr(), dptr(w_routed_down_T, "w_routed_down_T"),
                                      dptr(w_routed_down_T_sc, "w_routed_down_T_sc"), d_hidden.data_ptr(), nullptr, static_cast<int>(cap),
                                      static_cast<int>(I), static_cast<int>(H), MX8_C_BF16, num_tokens.data_ptr(), tokens_per_expert.data_ptr(),
                                      static_cast<int>(E), &w, main.stream()),
              "d_hidden gemm");
        check(mx8_swiglu_bwd_quantize_both_window(gate_fp8_routed.data_ptr(), gate_sc_routed.data_ptr(), up_fp8_routed.data_ptr(),
                                                  up_sc_routed.data_ptr(), d_hidden.data_ptr(), static_cast<int>(cap), static_cast<int>(I),
                                                  num_tokens.data_ptr(), d_gate_fp8.data_ptr(), d_gate_sc.data_ptr(), d_gate_fp8_t.data_ptr(),
                                                  d_gate_sc_t.data_ptr(), d_up_fp8.data_ptr(), d_up_sc.data_ptr(), d_up_fp8_t.data_ptr(),
                                                  d_up_sc_t.data_ptr(), &w, main.stream()),
              "swiglu backward + quantize");
        check(mx8_gemm_grouped_dual_window(d_gate_fp8.data_ptr(), d_gate_sc.data_ptr(), w_routed_gate_T.data_ptr(), w_routed_gate_T_sc.data_ptr(),
                                           d_up_fp8.data_ptr(), d_up_sc.data_ptr(), w_routed_up_T.data_ptr(), w_routed_up_T_sc.data_ptr(),
                                           d_x_routed.data_ptr(), static_cast<int>(cap), static_cast<int>(H), static_cast<int>(I),
                                           static_cast<int>(I), num_tokens.data_ptr(), tokens_per_expert.data_ptr(), static_cast<int>(E), &w,
                                           main.stream()),
              "data-gradient gemm");
        if (pipe) {
            at::cuda::CUDAEvent math_done;
            math_done.record(main);
            math_done.block(s_comb);
        }
        const mx8_window wc{pipe ? bp + b : nullptr, pipe ? bp + b + 1 : nullptr, (pipe && b < nb - 1) ? std::max(1, num_comm_sms / 4) : 0};
        check(mx8_moe_combine_window(d_x_routed.data_ptr(), schedule_peer_rank.data_ptr(), schedule_peer_token_idx.data_ptr(),
                                     num_tokens.data_ptr(), static_cast<int>(H), dst.data(), world, &wc, s_comb.stream()),
              "gradient combine");
    }
    auto wgrad = [&](const at::Tensor& at_, const at::Tensor& ats, const at::Tensor& bt, const at::Tensor& bts, at::Tensor& c) {
        check(mx8_gemm_wgrad(at_.data_ptr(), ats.data_ptr(), bt.data_ptr(), bts.data_ptr(), c.data_ptr(), static_cast<int>(at_.size(0)),
                             static_cast<int>(bt.size(0)), static_cast<int>(cap), tokens_per_expert.data_ptr(), static_cast<int>(E), stream()),
              "weight-gradient gemm");
    };
    wgrad(d_gate_fp8_t, d_gate_sc_t, x_fp8_t_routed, x_sc_t_routed, d_w_gate);
    wgrad(d_up_fp8_t, d_up_sc_t, x_fp8_t_routed, x_sc_t_routed, d_w_up);
    wgrad(d_y_fp8_t, d_y_sc_t, hidden_fp8_t_routed, hidden_sc_t_routed, d_w_down);
    if (pipe) {
        at::cuda::CUDAEvent done;                 // the last gradient combine ran beside the weight gradients
        done.record(s_comb);
        done.block(main);
        for (const at::Tensor* t : {&d_y_fp8, &d_y_sc, &d_y_fp8_t, &d_y_sc_t, &d_x_routed, &bounds}) {
            c10::cuda::CUDACachingAllocator::recordStream(t->storage().data_ptr(), s_disp);
            c10::cuda::CUDACachingAllocator::recordStream(t->storage().data_ptr(), s_comb);
        }
    }
    // shared expert (bf16), only when its tensors are given
    at::Tensor d_x_shared, d_gate_shared, d_up_shared, d_hidden_shared, d_w_sg, d_w_su, d_w_sd;
    if (d_y_shared && w_shared_gate_T && w_shared_up_T && w_shared_down_T && gate_shared && up_shared && hidden_shared && x_buffer) {
        d_hidden_shared = bf16_gemm(*d_y_shared, *w_shared_down_T);
        d_gate_shared = at::empty_like(*gate_shared);
        d_up_shared = at::empty_like(*gate_shared);
        check(mx8_swiglu_bwd_bf16(dptr(d_hidden_shared, "d_hidden_shared"), dptr(*gate_shared, "gate_shared"), dptr(*up_shared, "up_shared"),
                                  d_gate_shared.data_ptr(), d_up_shared.data_ptr(), gate_shared->numel(), stream()),
              "shared swiglu backward");
        d_x_shared = bf16_gemm(d_gate_shared, *w_shared_gate_T, &d_up_shared, &*w_shared_up_T);
        // weight gradients: K runs over the tokens, so both operands are transposed to K-major first
        at::Tensor x_t = bf16_transpose(*x_buffer);
        d_w_sg = bf16_gemm(bf16_transpose(d_gate_shared), x_t);
        d_w_su = bf16_gemm(bf16_transpose(d_up_shared), x_t);
        d_w_sd = bf16_gemm(bf16_transpose(*d_y_shared), bf16_transpose(*hidden_shared));
    }
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
