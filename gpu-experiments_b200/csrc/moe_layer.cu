// The expert-parallel MoE layer as one call behind the C ABI: dispatch + quantize, grouped GEMMs (gate, up) with
// quantizing epilogue, SwiGLU + quantize, grouped GEMM (down), combine, and the shared (bf16) expert; and its
// backward.  Stands in for the reference's two host functions that launch its persistent kernels,
// dispatch_mlp_swiglu_combine_fwd (blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.cu:2016-2136)
// and dispatch_mlp_swiglu_combine_bwd (:2556-2760).
//
// The reference overlaps transfers and GEMMs inside one kernel (communication CTAs beside a task queue,
// :1738-2011).  Here the same overlap comes from kernels on three streams: the local experts are cut into
// minibatches; the dispatch of minibatch b+1 runs on its own stream on `num_comm_sms` multiprocessors, the
// combine of minibatch b-1 on a third stream, the GEMMs and SwiGLU of minibatch b on the caller's stream on the
// remaining multiprocessors.  Events order the three legs of a minibatch; no kernel waits on another kernel.
// Every kernel is the row-window form of the one the unsplit layer launches, so the outputs do not depend on
// the split.  No device memory is allocated: intermediates live in the caller's workspace; the two side streams are
// created once per device and kept, the events of a call live as long as the call.
#include <cstdio>
#include <mutex>

#include "mx8_host.cuh"

namespace mx8 {
namespace layer {

constexpr int MAX_MINIBATCHES = 64;

struct DeviceCtx {
    cudaStream_t disp = nullptr, comb = nullptr;
    bool ready = false;
};

// Events of one call: created at its start, destroyed when it returns (the runtime keeps an event alive until the
// work that references it has finished), so concurrent calls never share one.
struct CallEvents {
    cudaEvent_t ev[2 * MAX_MINIBATCHES + 2] = {};
    int n = 0;
    cudaError_t err = cudaSuccess;
    explicit CallEvents(int count) {
        for (; n < count && err == cudaSuccess; ++n) err = cudaEventCreateWithFlags(&ev[n], cudaEventDisableTiming);
        if (err != cudaSuccess) --n;
    }
    ~CallEvents() {
        for (int i = 0; i < n; ++i) cudaEventDestroy(ev[i]);
    }
};

// side streams of the current device (created on first use, kept until the process exits)
static int device_ctx(DeviceCtx** out) {
    static DeviceCtx per_device[64];
    static std::mutex mu;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        note_cuda_error("cudaGetDevice", cudaGetErrorString(e));
        return MX8_ERR_CUDA;
    }
    std::lock_guard<std::mutex> lock(mu);
    DeviceCtx& c = per_device[dev];
    if (!c.ready) {
        e = cudaStreamCreateWithFlags(&c.disp, cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c.comb, cudaStreamNonBlocking);
        if (e != cudaSuccess) {
            note_cuda_error("moe layer: stream creation", cudaGetErrorString(e));
            return MX8_ERR_CUDA;
        }
        c.ready = true;
    }
    *out = &c;
    return MX8_OK;
}

struct Check {
    int rc = MX8_OK;
    void operator()(int r) { if (rc == MX8_OK && r != MX8_OK) rc = r; }
    void cuda(cudaError_t e, const char* what) {
        if (rc == MX8_OK && e != cudaSuccess) {
            note_cuda_error(what, cudaGetErrorString(e));
            rc = MX8_ERR_CUDA;
        }
    }
    bool ok() const { return rc == MX8_OK; }
};

#ifdef MX8_TRACE
// Timing study only (a build with -DMX8_TRACE): timed events around every launch of the minibatch forward, read back
// by mx8_debug_moe_trace_dump after the caller has synchronized.  Not part of the shipped library.
struct TraceRec { const char* name; int b; int stream; cudaEvent_t a, e; };
static TraceRec g_trace[8 * MAX_MINIBATCHES + 8];
static int g_trace_n = 0;
static cudaEvent_t g_trace_t0 = nullptr;
struct TraceScope {
    TraceRec* r = nullptr;
    cudaStream_t st;
    TraceScope(const char* name, int b, int stream_id, cudaStream_t s) : st(s) {
        if (g_trace_n >= static_cast<int>(sizeof(g_trace) / sizeof(g_trace[0]))) return;
        r = &g_trace[g_trace_n++];
        r->name = name; r->b = b; r->stream = stream_id;
        cudaEventCreate(&r->a); cudaEventCreate(&r->e);
        cudaEventRecord(r->a, st);
    }
    ~TraceScope() { if (r) cudaEventRecord(r->e, st); }
};
#define MX8_TRACE_SCOPE(name, b, id, s) TraceScope trace_scope_(name, b, id, s)
#else
#define MX8_TRACE_SCOPE(name, b, id, s) do {} while (0)
#endif

inline size_t up256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

// carve consecutive 256-byte aligned pieces out of the caller's workspace
struct Carver {
    uint8_t* p;
    size_t used = 0;
    explicit Carver(void* base) : p(static_cast<uint8_t*>(base)) {}
    void* take(size_t bytes) {
        void* r = p ? p + used : nullptr;
        used += up256(bytes);
        return r;
    }
};

// Minibatches: ceil(capacity / minibatch_size) groups of consecutive local experts (the reference's argument),
// at most one per expert.  `ramp` makes the first and the last groups smaller than the middle ones:
// the first dispatch and the last combine are the two transfers nothing can hide.
static int plan_minibatches(const mx8_moe_dims& d, int first_expert[MAX_MINIBATCHES + 1]) {
    int nb = 1;
    if (d.num_comm_sms > 0 && d.minibatch_size > 0) nb = (d.capacity + d.minibatch_size - 1) / d.minibatch_size;
    if (d.minibatches > 0) nb = d.minibatches;
    if (nb > d.num_local_experts) nb = d.num_local_experts;
    if (nb > MAX_MINIBATCHES) nb = MAX_MINIBATCHES;
    if (nb < 1) nb = 1;
    // weight of group b: 1 (equal groups); ramp = 1: the two end groups half; ramp > 100: groups grow by ramp percent
    // from either end toward the middle (a transfer hides behind the GEMMs of the group before it as long as the
    // growth stays below the ratio of GEMM time to transfer time)
    double w[MAX_MINIBATCHES], total = 0.0;
    for (int b = 0; b < nb; ++b) {
        w[b] = 1.0;
        if (d.ramp == 1 && nb >= 3 && (b == 0 || b == nb - 1)) w[b] = 0.5;
        if (d.ramp > 100 && nb >= 3) {
            const int steps = b < nb - 1 - b ? b : nb - 1 - b;
            for (int i = 0; i < steps; ++i) w[b] *= d.ramp / 100.0;
        }
        total += w[b];
    }
    double acc = 0.0;
    first_expert[0] = 0;
    for (int b = 0; b < nb; ++b) {
        acc += w[b];
        int e = static_cast<int>(d.num_local_experts * acc / total + 0.5);
        if (e <= first_expert[b]) e = first_expert[b] + 1;            // every group has an expert
        if (e > d.num_local_experts - (nb - 1 - b)) e = d.num_local_experts - (nb - 1 - b);
        first_expert[b + 1] = e;
    }
    first_expert[nb] = d.num_local_experts;
    return nb;
}

static int check_dims(const mx8_moe_dims& d) {
    if (d.world <= 0 || d.world > 16 || d.tokens <= 0 || d.topk <= 0 || d.num_local_experts <= 0) return MX8_ERR_ARG;
    if (d.num_local_experts > 256) {
        note_cuda_error("mx8_moe", "more than 256 local experts");
        return MX8_ERR_LIMIT;
    }
    if (d.hidden <= 0 || d.intermediate <= 0 || d.capacity <= 0 || d.hidden % 256 || d.intermediate % 256 || d.capacity % 256)
        return MX8_ERR_SHAPE;
    if (d.shared_intermediate < 0 || d.shared_intermediate % 128 || (d.shared_intermediate > 0 && d.tokens % 128)) return MX8_ERR_SHAPE;
    return MX8_OK;
}

}  // namespace layer
}  // namespace mx8

using mx8::layer::Carver;

extern "C" size_t mx8_moe_fwd_workspace_bytes(const mx8_moe_dims* d) {
    if (!d || mx8::layer::check_dims(*d) != MX8_OK) return 0;
    const size_t cap = d->capacity, H = d->hidden, I = d->intermediate;
    Carver c(nullptr);
    c.take(cap * H); c.take(cap * H / 32);          // row-wise MXFP8 of the dispatched tokens
    c.take(cap * I); c.take(cap * I / 32);          // row-wise MXFP8 of the activation
    c.take((mx8::layer::MAX_MINIBATCHES + 1) * sizeof(int));
    return c.used;
}

extern "C" int mx8_moe_fwd(const mx8_moe_fwd_args* a, void* stream) {
    using namespace mx8;
    using namespace mx8::layer;
    if (!a) return MX8_ERR_ARG;
    const mx8_moe_dims& d = a->dims;
    int rc = check_dims(d);
    if (rc != MX8_OK) return rc;
    if (!a->x_ptrs || !a->combine_ptrs || !a->w_gate || !a->w_gate_sc || !a->w_up || !a->w_up_sc || !a->w_down || !a->w_down_sc ||
        !a->peer_rank || !a->peer_token_idx || !a->num_tokens || !a->tokens_per_expert || !a->x_fp8_t || !a->x_sc_t || !a->gate_fp8 ||
        !a->gate_sc || !a->up_fp8 || !a->up_sc || !a->hidden_fp8_t || !a->hidden_sc_t || !a->workspace)
        return MX8_ERR_ARG;
    if (!a->fuse_combine && !a->y_routed) return MX8_ERR_ARG;
    const bool shared = d.shared_intermediate > 0;
    if (shared && (!a->x || !a->w_shared_gate || !a->w_shared_up || !a->w_shared_down || !a->gate_shared || !a->up_shared ||
                   !a->hidden_shared || !a->y_shared))
        return MX8_ERR_ARG;
    if (a->workspace_bytes < mx8_moe_fwd_workspace_bytes(&d)) {
        note_cuda_error("mx8_moe_fwd", "workspace smaller than mx8_moe_fwd_workspace_bytes");
        return MX8_ERR_LIMIT;
    }
    if (!aligned16(a->workspace)) return MX8_ERR_ALIGN;
    if ((rc = check_device_sm100()) != MX8_OK) return rc;

    const int cap = d.capacity, H = d.hidden, I = d.intermediate, E = d.num_local_experts;
    Carver ws(a->workspace);
    void* x_fp8 = ws.take(static_cast<size_t>(cap) * H);
    void* x_sc = ws.take(static_cast<size_t>(cap) * H / 32);
    void* h_fp8 = ws.take(static_cast<size_t>(cap) * I);
    void* h_sc = ws.take(static_cast<size_t>(cap) * I / 32);
    int* bounds = static_cast<int*>(ws.take((MAX_MINIBATCHES + 1) * sizeof(int)));

    cudaStream_t main = static_cast<cudaStream_t>(stream);
    int first_expert[MAX_MINIBATCHES + 1];
    const int nb = a->fuse_combine ? 1 : plan_minibatches(d, first_expert);
    Check ck;

    // shared expert (bf16, outside the MXFP8 path): queued first, so that with minibatches its GEMMs fill the time
    // the first dispatch needs (the reference's task queue starts with the shared expert's tasks as well)
    auto shared_expert = [&]() {
        if (!shared) return;
        const int T = d.tokens, Is = d.shared_intermediate;
        ck(mx8_gemm_bf16(a->x, a->w_shared_gate, a->gate_shared, T, Is, H, MX8_C_BF16, main));
        ck(mx8_gemm_bf16(a->x, a->w_shared_up, a->up_shared, T, Is, H, MX8_C_BF16, main));
        ck(mx8_swiglu_bf16(a->gate_shared, a->up_shared, a->hidden_shared, static_cast<long long>(T) * Is, main));
        ck(mx8_gemm_bf16(a->hidden_shared, a->w_shared_down, a->y_shared, T, H, Is, MX8_C_BF16, main));
    };

    // gate and up projections and SwiGLU.  Default: one launch whose epilogue holds gate and up of the same columns,
    // writes both as MXFP8 and the activation as MXFP8 in both orientations.  split_swiglu: the projections as one
    // pair launch (or two launches with split_gate_up) followed by the stand-alone SwiGLU kernel.  Same bytes in all forms.
    auto gate_up = [&](const mx8_window* w) {
        if (!d.split_swiglu) {
            ck(mx8_gemm_grouped_swiglu_window(x_fp8, x_sc, a->w_gate, a->w_gate_sc, a->w_up, a->w_up_sc, a->gate_fp8, a->gate_sc, a->up_fp8,
                                              a->up_sc, h_fp8, h_sc, a->hidden_fp8_t, a->hidden_sc_t, cap, I, H, a->num_tokens,
                                              a->tokens_per_expert, E, w, main));
            return;
        }
        if (d.split_gate_up) {
            ck(mx8_gemm_grouped_window(x_fp8, x_sc, a->w_gate, a->w_gate_sc, a->gate_fp8, a->gate_sc, cap, I, H, MX8_C_MXFP8,
                                       a->num_tokens, a->tokens_per_expert, E, w, main));
            ck(mx8_gemm_grouped_window(x_fp8, x_sc, a->w_up, a->w_up_sc, a->up_fp8, a->up_sc, cap, I, H, MX8_C_MXFP8, a->num_tokens,
                                       a->tokens_per_expert, E, w, main));
        } else {
            ck(mx8_gemm_grouped_pair_window(x_fp8, x_sc, a->w_gate, a->w_gate_sc, a->w_up, a->w_up_sc, a->gate_fp8, a->gate_sc, a->up_fp8,
                                            a->up_sc, cap, I, H, MX8_C_MXFP8, a->num_tokens, a->tokens_per_expert, E, w, main));
        }
        ck(mx8_swiglu_quantize_window(a->gate_fp8, a->gate_sc, a->up_fp8, a->up_sc, cap, I, a->num_tokens, h_fp8, h_sc, a->hidden_fp8_t,
                                      a->hidden_sc_t, nullptr, w, main));
    };

    if (nb <= 1) {
        ck(mx8_moe_dispatch_quantize(a->x_ptrs, d.world, H, d.topk, a->peer_rank, a->peer_token_idx, a->num_tokens, cap, x_fp8, x_sc,
                                     a->x_fp8_t, a->x_sc_t, main));
        gate_up(nullptr);
        if (a->fuse_combine) {
            ck(mx8_gemm_grouped_scatter(h_fp8, h_sc, a->w_down, a->w_down_sc, cap, H, I, a->num_tokens, a->tokens_per_expert, E,
                                        a->peer_rank, a->peer_token_idx, a->combine_ptrs, d.world, main));
        } else {
            ck(mx8_gemm_grouped(h_fp8, h_sc, a->w_down, a->w_down_sc, a->y_routed, nullptr, cap, H, I, MX8_C_BF16, a->num_tokens,
                                a->tokens_per_expert, E, main));
            ck(mx8_moe_combine(a->y_routed, a->peer_rank, a->peer_token_idx, a->num_tokens, cap, H, a->combine_ptrs, d.world,
                               static_cast<long long>(d.tokens) * d.topk, main));
        }
        shared_expert();
        return ck.rc;
    }

    DeviceCtx* cx = nullptr;
    if ((rc = device_ctx(&cx)) != MX8_OK) return rc;
    const int sms = sm_count();
    if (sms <= 0) return MX8_ERR_CUDA;
    const int math_sms = (sms - d.num_comm_sms) & ~1;
    if (math_sms < 2) return MX8_ERR_ARG;
    // A combine that runs beside GEMMs either shares their multiprocessors, held to combine_sms multiprocessors' worth of
    // copy blocks, or (combine_own_sms > 0) gets multiprocessors of its own, which the GEMMs beside it then leave free.
    const int own_sms = d.combine_own_sms > 0 ? ((d.combine_own_sms + 1) & ~1) : 0;
    const int combine_sms = own_sms ? own_sms : (d.combine_sms > 0 ? d.combine_sms : (d.num_comm_sms / 4 > 0 ? d.num_comm_sms / 4 : 1));
    if (math_sms - own_sms < 2) return MX8_ERR_ARG;
    ck(mx8_moe_minibatch_bounds_split(a->tokens_per_expert, E, nb, first_expert, bounds, main));
    CallEvents evs(2 * nb + 2);
    ck.cuda(evs.err, "cudaEventCreateWithFlags");
    if (!ck.ok()) return ck.rc;
    cudaEvent_t start = evs.ev[0], done = evs.ev[1];
    cudaEvent_t* disp_done = evs.ev + 2;
    cudaEvent_t* math_done = evs.ev + 2 + nb;
    ck.cuda(cudaEventRecord(start, main), "cudaEventRecord");
#ifdef MX8_TRACE
    for (int i = 0; i < g_trace_n; ++i) { cudaEventDestroy(g_trace[i].a); cudaEventDestroy(g_trace[i].e); }
    g_trace_n = 0;
    if (!g_trace_t0) cudaEventCreate(&g_trace_t0);
    cudaEventRecord(g_trace_t0, main);
#endif
    ck.cuda(cudaStreamWaitEvent(cx->disp, start, 0), "cudaStreamWaitEvent");
    ck.cuda(cudaStreamWaitEvent(cx->comb, start, 0), "cudaStreamWaitEvent");
    for (int b = 0; b < nb && ck.ok(); ++b) {
        // the first minibatch has the device to itself; later ones run beside the GEMMs
        const mx8_window w{bounds + b, bounds + b + 1, b == 0 ? 0 : d.num_comm_sms};
        {
            MX8_TRACE_SCOPE("dispatch", b, 1, cx->disp);
            ck(mx8_moe_dispatch_quantize_window(a->x_ptrs, d.world, H, d.topk, a->peer_rank, a->peer_token_idx, a->num_tokens, cap,
                                                x_fp8, x_sc, a->x_fp8_t, a->x_sc_t, &w, cx->disp));
        }
        ck.cuda(cudaEventRecord(disp_done[b], cx->disp), "cudaEventRecord");
    }
    shared_expert();
    for (int b = 0; b < nb && ck.ok(); ++b) {
        ck.cuda(cudaStreamWaitEvent(main, disp_done[b], 0), "cudaStreamWaitEvent");
        // the last minibatch's GEMMs run after every dispatch has finished: they take the whole device
        // and, with combine_own_sms, every minibatch but the first leaves the combine of the one before it its multiprocessors
        const int gemm_sms = (b == nb - 1 ? (sms & ~1) : math_sms) - (b > 0 ? own_sms : 0);
        const mx8_window w{bounds + b, bounds + b + 1, gemm_sms >= (sms & ~1) ? 0 : gemm_sms, 0};
        {
            MX8_TRACE_SCOPE("gate_up", b, 0, main);
            gate_up(&w);
        }
        {
            MX8_TRACE_SCOPE("down", b, 0, main);
            ck(mx8_gemm_grouped_window(h_fp8, h_sc, a->w_down, a->w_down_sc, a->y_routed, nullptr, cap, H, I, MX8_C_BF16,
                                       a->num_tokens, a->tokens_per_expert, E, &w, main));
        }
        ck.cuda(cudaEventRecord(math_done[b], main), "cudaEventRecord");
        ck.cuda(cudaStreamWaitEvent(cx->comb, math_done[b], 0), "cudaStreamWaitEvent");
        // beside GEMMs the combine is held to combine_sms multiprocessors' worth of copy warps, spread thinly over the
        // GEMMs' multiprocessors: more of them slow the GEMM blocks they share a multiprocessor with by more than the
        // overlap gains
        const mx8_window wc{bounds + b, bounds + b + 1, b < nb - 1 ? combine_sms : 0, (own_sms && b < nb - 1) ? 1 : 0};
        {
            MX8_TRACE_SCOPE("combine", b, 2, cx->comb);
            ck(mx8_moe_combine_window(a->y_routed, a->peer_rank, a->peer_token_idx, a->num_tokens, cap, H, a->combine_ptrs, d.world,
                                      static_cast<long long>(d.tokens) * d.topk, &wc, cx->comb));
        }
    }
    ck.cuda(cudaEventRecord(done, cx->comb), "cudaEventRecord");
    ck.cuda(cudaStreamWaitEvent(main, done, 0), "cudaStreamWaitEvent");
    return ck.rc;
}

extern "C" size_t mx8_moe_bwd_workspace_bytes(const mx8_moe_dims* d) {
    if (!d || mx8::layer::check_dims(*d) != MX8_OK) return 0;
    const size_t cap = d->capacity, H = d->hidden, I = d->intermediate, T = d->tokens, Is = d->shared_intermediate;
    Carver c(nullptr);
    c.take(cap * H); c.take(cap * H / 32);          // transposed MXFP8 of the gathered output gradient
    c.take(cap * I); c.take(cap * I / 32);          // transposed MXFP8 of d_gate
    c.take(cap * I); c.take(cap * I / 32);          // transposed MXFP8 of d_up
    c.take((mx8::layer::MAX_MINIBATCHES + 1) * sizeof(int));
    if (Is > 0) {                                   // token-major copies for the shared expert's weight gradients
        c.take(T * H * 2); c.take(T * Is * 2); c.take(T * Is * 2); c.take(T * H * 2); c.take(T * Is * 2);
    }
    return c.used;
}

extern "C" int mx8_moe_bwd(const mx8_moe_bwd_args* a, void* stream) {
    using namespace mx8;
    using namespace mx8::layer;
    if (!a) return MX8_ERR_ARG;
    const mx8_moe_dims& d = a->dims;
    int rc = check_dims(d);
    if (rc != MX8_OK) return rc;
    const void* const need[] = {a->d_combine_ptrs, a->d_x_routed_ptrs, a->w_gate_T, a->w_gate_T_sc, a->w_up_T, a->w_up_T_sc, a->w_down_T,
                                a->w_down_T_sc, a->x_fp8_t, a->x_sc_t, a->gate_fp8, a->gate_sc, a->up_fp8, a->up_sc, a->hidden_fp8_t,
                                a->hidden_sc_t, a->peer_rank, a->peer_token_idx, a->num_tokens, a->tokens_per_expert, a->d_x_routed,
                                a->d_gate_fp8, a->d_gate_sc, a->d_up_fp8, a->d_up_sc, a->d_hidden_routed, a->d_y_fp8, a->d_y_sc,
                                a->d_w_gate, a->d_w_up, a->d_w_down, a->workspace};
    for (const void* p : need)
        if (!p) return MX8_ERR_ARG;
    const bool shared = d.shared_intermediate > 0;
    if (shared) {
        const void* const sneed[] = {a->d_y_shared, a->x, a->w_shared_gate_T, a->w_shared_up_T, a->w_shared_down_T, a->gate_shared,
                                     a->up_shared, a->hidden_shared, a->d_x_shared, a->d_gate_shared, a->d_up_shared, a->d_hidden_shared,
                                     a->d_w_shared_gate, a->d_w_shared_up, a->d_w_shared_down};
        for (const void* p : sneed)
            if (!p) return MX8_ERR_ARG;
    }
    if (a->workspace_bytes < mx8_moe_bwd_workspace_bytes(&d)) {
        note_cuda_error("mx8_moe_bwd", "workspace smaller than mx8_moe_bwd_workspace_bytes");
        return MX8_ERR_LIMIT;
    }
    if (!aligned16(a->workspace)) return MX8_ERR_ALIGN;
    if ((rc = check_device_sm100()) != MX8_OK) return rc;

    const int cap = d.capacity, H = d.hidden, I = d.intermediate, E = d.num_local_experts;
    Carver ws(a->workspace);
    void* d_y_fp8_t = ws.take(static_cast<size_t>(cap) * H);
    void* d_y_sc_t = ws.take(static_cast<size_t>(cap) * H / 32);
    void* d_gate_fp8_t = ws.take(static_cast<size_t>(cap) * I);
    void* d_gate_sc_t = ws.take(static_cast<size_t>(cap) * I / 32);
    void* d_up_fp8_t = ws.take(static_cast<size_t>(cap) * I);
    void* d_up_sc_t = ws.take(static_cast<size_t>(cap) * I / 32);
    int* bounds = static_cast<int*>(ws.take((MAX_MINIBATCHES + 1) * sizeof(int)));

    cudaStream_t main = static_cast<cudaStream_t>(stream);
    int first_expert[MAX_MINIBATCHES + 1];
    const int nb = plan_minibatches(d, first_expert);
    const bool pipe = nb > 1;
    Check ck;
    DeviceCtx* cx = nullptr;
    cudaStream_t s_disp = main, s_comb = main;
    int math_sms = 0, combine_sms = 0, own_sms = 0, all_sms = 0;
    cudaEvent_t* disp_done = nullptr;
    cudaEvent_t* math_done = nullptr;
    CallEvents evs(pipe ? 2 * nb + 2 : 0);
    ck.cuda(evs.err, "cudaEventCreateWithFlags");
    if (!ck.ok()) return ck.rc;
    if (pipe) {
        if ((rc = device_ctx(&cx)) != MX8_OK) return rc;
        const int sms = sm_count();
        if (sms <= 0) return MX8_ERR_CUDA;
        math_sms = (sms - d.num_comm_sms) & ~1;
        if (math_sms < 2) return MX8_ERR_ARG;
        own_sms = d.combine_own_sms > 0 ? ((d.combine_own_sms + 1) & ~1) : 0;          // as in the forward
        combine_sms = own_sms ? own_sms : (d.combine_sms > 0 ? d.combine_sms : (d.num_comm_sms / 4 > 0 ? d.num_comm_sms / 4 : 1));
        if (math_sms - own_sms < 2) return MX8_ERR_ARG;
        all_sms = sms & ~1;
        s_disp = cx->disp;
        s_comb = cx->comb;
        disp_done = evs.ev + 2;
        math_done = evs.ev + 2 + nb;
        ck(mx8_moe_minibatch_bounds_split(a->tokens_per_expert, E, nb, first_expert, bounds, main));
        ck.cuda(cudaEventRecord(evs.ev[0], main), "cudaEventRecord");
#ifdef MX8_TRACE
        for (int i = 0; i < g_trace_n; ++i) { cudaEventDestroy(g_trace[i].a); cudaEventDestroy(g_trace[i].e); }
        g_trace_n = 0;
        if (!g_trace_t0) cudaEventCreate(&g_trace_t0);
        cudaEventRecord(g_trace_t0, main);
#endif
        ck.cuda(cudaStreamWaitEvent(s_disp, evs.ev[0], 0), "cudaStreamWaitEvent");
        ck.cuda(cudaStreamWaitEvent(s_comb, evs.ev[0], 0), "cudaStreamWaitEvent");
    }
    for (int b = 0; b < nb && ck.ok(); ++b) {
        const mx8_window w{pipe ? bounds + b : nullptr, pipe ? bounds + b + 1 : nullptr, (pipe && b > 0) ? d.num_comm_sms : 0};
        // gradient rows of the routed outputs, pulled from the owners' buffers: one row per (token, k) pair,
        // hence topk = 1 for the index
        {
            MX8_TRACE_SCOPE("dispatch", b, 1, s_disp);
            ck(mx8_moe_dispatch_quantize_window(a->d_combine_ptrs, d.world, H, 1, a->peer_rank, a->peer_token_idx, a->num_tokens, cap,
                                                a->d_y_fp8, a->d_y_sc, d_y_fp8_t, d_y_sc_t, &w, s_disp));
        }
        if (pipe) ck.cuda(cudaEventRecord(disp_done[b], s_disp), "cudaEventRecord");
    }
    for (int b = 0; b < nb && ck.ok(); ++b) {
        if (pipe) ck.cuda(cudaStreamWaitEvent(main, disp_done[b], 0), "cudaStreamWaitEvent");
        // the weight-gradient GEMMs follow the last minibatch, so no minibatch has the whole device for its data gradients
        // and, with combine_own_sms, every minibatch but the first leaves the gradient combine of the one before it its multiprocessors
        const int gemm_sms = !pipe ? 0 : (b < nb - 1 ? math_sms : all_sms) - (b > 0 ? own_sms : 0);
        const mx8_window w{pipe ? bounds + b : nullptr, pipe ? bounds + b + 1 : nullptr, gemm_sms >= all_sms ? 0 : gemm_sms, 0};
        {
            MX8_TRACE_SCOPE("d_hidden", b, 0, main);
            ck(mx8_gemm_grouped_window(a->d_y_fp8, a->d_y_sc, a->w_down_T, a->w_down_T_sc, a->d_hidden_routed, nullptr, cap, I, H,
                                       MX8_C_BF16, a->num_tokens, a->tokens_per_expert, E, &w, main));
        }
        {
            MX8_TRACE_SCOPE("swiglu", b, 0, main);
            ck(mx8_swiglu_bwd_quantize_both_window(a->gate_fp8, a->gate_sc, a->up_fp8, a->up_sc, a->d_hidden_routed, cap, I,
                                                   a->num_tokens, a->d_gate_fp8, a->d_gate_sc, d_gate_fp8_t, d_gate_sc_t, a->d_up_fp8,
                                                   a->d_up_sc, d_up_fp8_t, d_up_sc_t, &w, main));
        }
        {
            MX8_TRACE_SCOPE("d_x", b, 0, main);
            ck(mx8_gemm_grouped_dual_window(a->d_gate_fp8, a->d_gate_sc, a->w_gate_T, a->w_gate_T_sc, a->d_up_fp8, a->d_up_sc,
                                            a->w_up_T, a->w_up_T_sc, a->d_x_routed, cap, H, I, I, a->num_tokens, a->tokens_per_expert,
                                            E, &w, main));
        }
        if (pipe) {
            ck.cuda(cudaEventRecord(math_done[b], main), "cudaEventRecord");
            ck.cuda(cudaStreamWaitEvent(s_comb, math_done[b], 0), "cudaStreamWaitEvent");
        }
        const mx8_window wc{pipe ? bounds + b : nullptr, pipe ? bounds + b + 1 : nullptr, (pipe && b < nb - 1) ? combine_sms : 0,
                            (pipe && own_sms && b < nb - 1) ? 1 : 0};
        {
            MX8_TRACE_SCOPE("combine", b, 2, s_comb);
            ck(mx8_moe_combine_window(a->d_x_routed, a->peer_rank, a->peer_token_idx, a->num_tokens, cap, H, a->d_x_routed_ptrs,
                                      d.world, static_cast<long long>(d.tokens) * d.topk, &wc, s_comb));
        }
    }
    // weight gradients on the transposed activations the forward produced and the transposed gradients
    {
        MX8_TRACE_SCOPE("wgrad x3", 0, 0, main);
        ck(mx8_gemm_wgrad(d_gate_fp8_t, d_gate_sc_t, a->x_fp8_t, a->x_sc_t, a->d_w_gate, I, H, cap, a->tokens_per_expert, E, main));
        ck(mx8_gemm_wgrad(d_up_fp8_t, d_up_sc_t, a->x_fp8_t, a->x_sc_t, a->d_w_up, I, H, cap, a->tokens_per_expert, E, main));
        ck(mx8_gemm_wgrad(d_y_fp8_t, d_y_sc_t, a->hidden_fp8_t, a->hidden_sc_t, a->d_w_down, H, I, cap, a->tokens_per_expert, E, main));
    }
    if (pipe) {
        // the last gradient combine ran beside the weight gradients
        ck.cuda(cudaEventRecord(evs.ev[1], s_comb), "cudaEventRecord");
        ck.cuda(cudaStreamWaitEvent(main, evs.ev[1], 0), "cudaStreamWaitEvent");
    }
    if (shared && ck.ok()) {
        const int T = d.tokens, Is = d.shared_intermediate;
        void* x_t = ws.take(static_cast<size_t>(T) * H * 2);
        void* dg_t = ws.take(static_cast<size_t>(T) * Is * 2);
        void* du_t = ws.take(static_cast<size_t>(T) * Is * 2);
        void* dy_t = ws.take(static_cast<size_t>(T) * H * 2);
        void* h_t = ws.take(static_cast<size_t>(T) * Is * 2);
        ck(mx8_gemm_bf16(a->d_y_shared, a->w_shared_down_T, a->d_hidden_shared, T, Is, H, MX8_C_BF16, main));
        ck(mx8_swiglu_bwd_bf16(a->d_hidden_shared, a->gate_shared, a->up_shared, a->d_gate_shared, a->d_up_shared,
                               static_cast<long long>(T) * Is, main));
        // data gradient: two products accumulated in one tile pass
        ck(mx8_gemm_bf16_dual(a->d_gate_shared, a->w_shared_gate_T, a->d_up_shared, a->w_shared_up_T, a->d_x_shared, T, H, Is, Is,
                              MX8_C_BF16, main));
        // weight gradients: K runs over the tokens, so both operands are transposed to K-major first
        ck(mx8_transpose_bf16(a->x, x_t, T, H, main));
        ck(mx8_transpose_bf16(a->d_gate_shared, dg_t, T, Is, main));
        ck(mx8_transpose_bf16(a->d_up_shared, du_t, T, Is, main));
        ck(mx8_transpose_bf16(a->d_y_shared, dy_t, T, H, main));
        ck(mx8_transpose_bf16(a->hidden_shared, h_t, T, Is, main));
        ck(mx8_gemm_bf16(dg_t, x_t, a->d_w_shared_gate, Is, H, T, MX8_C_BF16, main));
        ck(mx8_gemm_bf16(du_t, x_t, a->d_w_shared_up, Is, H, T, MX8_C_BF16, main));
        ck(mx8_gemm_bf16(dy_t, h_t, a->d_w_shared_down, H, Is, T, MX8_C_BF16, main));
    }
    return ck.rc;
}

#ifdef MX8_TRACE
// prints the timeline of the last minibatch forward of this process (call after synchronizing the device)
extern "C" MX8_API int mx8_debug_moe_trace_dump(void) {
    using namespace mx8::layer;
    for (int i = 0; i < g_trace_n; ++i) {
        float t_a = 0.f, t_e = 0.f;
        cudaEventElapsedTime(&t_a, g_trace_t0, g_trace[i].a);
        cudaEventElapsedTime(&t_e, g_trace_t0, g_trace[i].e);
        printf("  stream %d  %-8s mb %d  start %7.3f  end %7.3f  dur %6.3f ms\n", g_trace[i].stream, g_trace[i].name, g_trace[i].b,
               t_a, t_e, t_e - t_a);
    }
    fflush(stdout);
    return g_trace_n;
}
#endif
