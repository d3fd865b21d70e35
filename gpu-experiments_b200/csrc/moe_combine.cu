// MoE combine (expert output rows back to the ranks that own the tokens) and the weighted sum that
// finishes the layer.
//
// combine: row r of y_routed (bf16, `hidden` wide) goes to row peer_token_idx[r] of the combine
// buffer of rank peer_rank[r]; rows with peer_rank < 0 (padding) are skipped, and so is everything a
// schedule that overflowed its capacity could make the kernel touch: rows at or beyond `capacity`, a
// rank outside [0, world), a destination row outside the buffer.  The destination is
// that rank's memory, written directly with 16-byte stores over NVLink (one warp per row, 512 bytes
// per warp instruction).  The copy is exact.  Replaces combine_kernel,
// blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.cu:830-922.
//
// epilogue: out[t] = bf16( y_shared[t] + sum_j w[t][j] * combine[t*topk + j] ), fp32, products and
// sums rounded separately, j ascending, so the result does not depend on the launch shape.
// Replaces fwd_epilogue_kernel, blackwell-ultra/022-…-mxfp8-bw.cu:2789-2856.
#include <atomic>

#include "mx8_host.cuh"
#include "mx8_ptx.cuh"

namespace mx8 {
namespace moe {

struct CombineParams {
    const uint8_t* y;            // [rows][hidden] bf16
    const int* peer_rank;
    const int* peer_token_idx;
    const int* num_tokens;       // device: one past the last row
    const int* row_begin;        // device: first row (row window of a minibatch), nullptr = 0
    int hidden;
    int capacity;                // rows y_routed and the two index arrays have
    int world;
    long long dst_rows;          // rows of every destination buffer
    uint8_t* dst[16];            // every rank's combine buffer [tokens*topk][hidden] bf16
    int* status;                 // device status word (bounded waits of the bulk-copy forms)
    int piece_bytes;             // bulk-copy forms: bytes per copy (a row goes in ceil(row / piece) pieces), multiple of 16
};

__global__ void __launch_bounds__(256) combine_kernel(CombineParams p) {
    const int rows = min(*p.num_tokens, p.capacity);
    const int row0 = p.row_begin ? *p.row_begin : 0;
    const int lane = threadIdx.x & 31;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const size_t row_bytes = static_cast<size_t>(p.hidden) * 2;
    for (int r = row0 + warp; r < rows; r += warps) {
        const int pr = p.peer_rank[r];
        if (pr < 0 || pr >= p.world) continue;
        const int pt = p.peer_token_idx[r];
        if (pt < 0 || pt >= p.dst_rows) continue;
        const uint4* src = reinterpret_cast<const uint4*>(p.y + r * row_bytes);
        uint4* dst = reinterpret_cast<uint4*>(p.dst[pr] + static_cast<size_t>(pt) * row_bytes);
        const int n16 = p.hidden / 8;
        constexpr int U = 4;                             // independent 16-byte copies in flight per lane
        for (int i = lane; i < n16; i += 32 * U) {
            uint4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (i + 32 * u < n16) v[u] = src[i + 32 * u];
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (i + 32 * u < n16) dst[i + 32 * u] = v[u];
        }
    }
}

// The form with multiprocessors of its own (mx8_window.own_sms): every warp moves rows with bulk copies through two
// buffers in shared memory (global -> shared, then shared -> the owner's buffer, local or a peer's over NVLink; every
// copy has one source and one destination), a row in pieces of at most 7.5 KB.  One lane issues; while the store of one piece drains from its
// buffer the load of the next is in flight in the other.  The blocks ask for more shared memory than a multiprocessor
// has left beside a GEMM or a dispatch block, so they never share one.
constexpr int BULK_WARPS = 6;
__global__ void __launch_bounds__(32 * BULK_WARPS) combine_bulk_kernel(CombineParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 127u) & ~127u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t row_bytes = static_cast<uint32_t>(p.hidden) * 2u;
    const uint32_t piece = static_cast<uint32_t>(p.piece_bytes);
    const uint32_t buf_bytes = (piece + 127u) & ~127u;
    const int warp_in_block = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // per warp: two buffers, then (after all buffers) two barriers; the abort flag follows the barriers
    const uint32_t buf0 = base + (warp_in_block * 2) * buf_bytes;
    const uint32_t bar0 = base + BULK_WARPS * 2 * buf_bytes + warp_in_block * 16;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + BULK_WARPS * 2 * buf_bytes + BULK_WARPS * 16);
    if (threadIdx.x == 0) *abort_flag = 0;
    if (lane == 0) {
        mbar_init(bar0, 1);
        mbar_init(bar0 + 8, 1);
        fence_mbar_init();
    }
    __syncthreads();
    if (lane != 0) return;
    const AbortCtl ab{abort_flag, p.status};
    const int rows = min(*p.num_tokens, p.capacity);
    const int row0 = p.row_begin ? *p.row_begin : 0;
    const int warp = blockIdx.x * BULK_WARPS + warp_in_block;
    const int warps = gridDim.x * BULK_WARPS;
    uint32_t phase[2] = {0, 0};
    int n = 0;                                           // copies this warp has issued
    bool ok = true;
    for (int r = row0 + warp; r < rows && ok; r += warps) {
        const int pr = p.peer_rank[r];
        if (pr < 0 || pr >= p.world) continue;
        const int pt = p.peer_token_idx[r];
        if (pt < 0 || pt >= p.dst_rows) continue;
        const uint8_t* src = p.y + static_cast<size_t>(r) * row_bytes;
        uint8_t* dst = p.dst[pr] + static_cast<size_t>(pt) * row_bytes;
        for (uint32_t off = 0; off < row_bytes; off += piece, ++n) {
            const uint32_t len = min(piece, row_bytes - off);
            const int s = n & 1;
            // the store issued from this buffer two copies ago must have finished reading it
            bulk_wait_read<1>();
            mbar_arrive_expect_tx(bar0 + s * 8, len);
            bulk_load_1d(buf0 + s * buf_bytes, src + off, len, bar0 + s * 8);
            if (!mbar_wait(bar0 + s * 8, phase[s], ab, DEV_TIMEOUT_FULL)) { ok = false; break; }
            phase[s] ^= 1;
            bulk_store_1d(dst + off, buf0 + s * buf_bytes, len);
            bulk_commit();
        }
    }
    bulk_wait_all<0>();
}

struct EpilogueParams {
    const uint8_t* y_shared;     // [tokens][hidden] bf16 or nullptr (no shared expert)
    const uint8_t* combine;      // [tokens*topk][hidden] bf16
    const float* weights;        // [tokens][topk], nullptr = plain sum (backward epilogue)
    uint8_t* out;                // [tokens][hidden] bf16
    int tokens, hidden, topk;
};

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
}

__global__ void __launch_bounds__(256) epilogue_kernel(EpilogueParams p) {
    const int n16 = p.hidden / 8;
    const long long total = static_cast<long long>(p.tokens) * n16;
    for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
         idx += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int t = static_cast<int>(idx / n16), c = static_cast<int>(idx - static_cast<long long>(t) * n16);
        float acc[8];
        if (p.y_shared) {
            unpack8(reinterpret_cast<const uint4*>(p.y_shared)[idx], acc);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
        }
        for (int j = 0; j < p.topk; ++j) {
            const float w = p.weights ? p.weights[static_cast<size_t>(t) * p.topk + j] : 1.0f;
            float v[8];
            unpack8(reinterpret_cast<const uint4*>(p.combine)[(static_cast<size_t>(t) * p.topk + j) * n16 + c], v);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(acc[i], __fmul_rn(v[i], w));   // no fused multiply-add
        }
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]);
        o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]);
        o.w = pack_bf16x2(acc[6], acc[7]);
        reinterpret_cast<uint4*>(p.out)[idx] = o;
    }
}

// backward prologue: d_combine[t*topk + j] = bf16( d_output[t] * w[t][j] )
__global__ void __launch_bounds__(256) bwd_prologue_kernel(const uint8_t* d_out, const float* weights, uint8_t* d_combine, int tokens,
                                                           int hidden, int topk) {
    const int n16 = hidden / 8;
    const long long total = static_cast<long long>(tokens) * n16;
    for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
         idx += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int t = static_cast<int>(idx / n16), c = static_cast<int>(idx - static_cast<long long>(t) * n16);
        float v[8];
        unpack8(reinterpret_cast<const uint4*>(d_out)[idx], v);
        for (int j = 0; j < topk; ++j) {
            const float w = weights[static_cast<size_t>(t) * topk + j];
            uint4 o;
            o.x = pack_bf16x2(__fmul_rn(v[0], w), __fmul_rn(v[1], w));
            o.y = pack_bf16x2(__fmul_rn(v[2], w), __fmul_rn(v[3], w));
            o.z = pack_bf16x2(__fmul_rn(v[4], w), __fmul_rn(v[5], w));
            o.w = pack_bf16x2(__fmul_rn(v[6], w), __fmul_rn(v[7], w));
            reinterpret_cast<uint4*>(d_combine)[(static_cast<size_t>(t) * topk + j) * n16 + c] = o;
        }
    }
}

}  // namespace moe
}  // namespace mx8

extern "C" int mx8_moe_combine(const void* y_routed, const void* peer_rank, const void* peer_token_idx, const void* num_tokens,
                               int capacity, int hidden, void* const* combine_ptrs, int world, long long combine_rows, void* stream) {
    return mx8_moe_combine_window(y_routed, peer_rank, peer_token_idx, num_tokens, capacity, hidden, combine_ptrs, world, combine_rows,
                                  nullptr, stream);
}

extern "C" int mx8_moe_combine_window(const void* y_routed, const void* peer_rank, const void* peer_token_idx, const void* num_tokens,
                                      int capacity, int hidden, void* const* combine_ptrs, int world, long long combine_rows,
                                      const mx8_window* window, void* stream) {
    using namespace mx8;
    if (!y_routed || !peer_rank || !peer_token_idx || !num_tokens || !combine_ptrs) return MX8_ERR_ARG;
    if (world <= 0 || world > 16 || capacity <= 0 || combine_rows <= 0) return MX8_ERR_ARG;
    if (hidden <= 0 || hidden % 8) return MX8_ERR_SHAPE;
    if (!aligned16(y_routed)) return MX8_ERR_ALIGN;
    moe::CombineParams p{};
    for (int r = 0; r < world; ++r) {
        if (!combine_ptrs[r] || !aligned16(combine_ptrs[r])) return MX8_ERR_ALIGN;
        p.dst[r] = static_cast<uint8_t*>(combine_ptrs[r]);
    }
    int rc = check_device_sm100();
    if (rc != MX8_OK) return rc;
    p.y = static_cast<const uint8_t*>(y_routed);
    p.peer_rank = static_cast<const int*>(peer_rank);
    p.peer_token_idx = static_cast<const int*>(peer_token_idx);
    p.num_tokens = static_cast<const int*>(num_tokens);
    p.hidden = hidden;
    p.capacity = capacity;
    p.world = world;
    p.dst_rows = combine_rows;
    int sms = sm_count();
    if (sms <= 0) return MX8_ERR_CUDA;
    if (window) {
        if (window->row_begin) p.row_begin = static_cast<const int*>(window->row_begin);
        if (window->row_end) p.num_tokens = static_cast<const int*>(window->row_end);
        if (window->max_sms > 0 && window->max_sms < sms) sms = window->max_sms;
    }
    cudaError_t e;
    if (window && window->own_sms && window->max_sms > 0 && window->max_sms < sm_count()) {
        // Multiprocessors of its own, as clusters of two so that the blocks fill whole pairs of multiprocessors (the
        // GEMMs' clusters need both halves of a pair).  Why one would: copy warps on a GEMM's multiprocessor take issue
        // slots from its two single-thread issuers, and with tiles assigned in fixed strides the whole GEMM then waits
        // for the blocks that were slowed down.  Why not always: a multiprocessor moves only about 15 GB/s over NVLink
        // whatever it does, so a transfer that is mostly remote wants many of them.
        const size_t row_bytes = static_cast<size_t>(hidden) * 2;
        const size_t pieces = (row_bytes + 7679) / 7680;
        p.piece_bytes = static_cast<int>(((row_bytes + pieces - 1) / pieces + 15) & ~static_cast<size_t>(15));
        const size_t buf_bytes = (static_cast<size_t>(p.piece_bytes) + 127) & ~static_cast<size_t>(127);
        size_t smem = moe::BULK_WARPS * 2 * buf_bytes + moe::BULK_WARPS * 16 + 16 + 128;
        if (smem < 64 * 1024) smem = 64 * 1024;          // more than a GEMM or dispatch block leaves free
        static std::atomic<size_t> configured[64];
        int dev = 0;
        cudaGetDevice(&dev);
        if (configured[dev & 63].load(std::memory_order_acquire) < smem) {
            e = cudaFuncSetAttribute(moe::combine_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
            if (e != cudaSuccess) {
                note_cuda_error("cudaFuncSetAttribute(combine)", cudaGetErrorString(e));
                return MX8_ERR_CUDA;
            }
            configured[dev & 63].store(smem, std::memory_order_release);
        }
        p.status = device_status_ptr();
        if (!p.status) return MX8_ERR_CUDA;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>((sms + 1) & ~1));
        cfg.blockDim = dim3(32 * moe::BULK_WARPS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = static_cast<cudaStream_t>(stream);
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 2;
        at[0].val.clusterDim.y = 1;
        at[0].val.clusterDim.z = 1;
        cfg.attrs = at;
        cfg.numAttrs = 1;
        e = cudaLaunchKernelEx(&cfg, moe::combine_bulk_kernel, p);
    } else if (window && window->max_sms > 0 && window->max_sms < sm_count()) {
        // held to max_sms multiprocessors' worth of copy warps, in blocks of two warps: spread thinly over the GEMMs'
        // multiprocessors they slow every GEMM block a little instead of a few blocks a lot (tiles are assigned to GEMM
        // blocks in fixed strides, so the slowest block sets the GEMM's time)
        moe::combine_kernel<<<sms * 16, 64, 0, static_cast<cudaStream_t>(stream)>>>(p);
        e = cudaGetLastError();
    } else {
        moe::combine_kernel<<<sms * 4, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) {
        note_cuda_error("moe combine launch", cudaGetErrorString(e));
        return MX8_ERR_CUDA;
    }
    return MX8_OK;
}

extern "C" int mx8_moe_fwd_epilogue(const void* y_shared, const void* combine_buffer, const void* topk_weights, void* out,
                                    int tokens, int hidden, int topk, void* stream) {
    using namespace mx8;
    if (!combine_buffer || !topk_weights || !out) return MX8_ERR_ARG;
    if (tokens <= 0 || topk <= 0) return MX8_ERR_ARG;
    if (hidden <= 0 || hidden % 8) return MX8_ERR_SHAPE;
    if (!aligned16(y_shared) || !aligned16(combine_buffer) || !aligned16(out)) return MX8_ERR_ALIGN;
    int rc = check_device_sm100();
    if (rc != MX8_OK) return rc;
    moe::EpilogueParams p{static_cast<const uint8_t*>(y_shared), static_cast<const uint8_t*>(combine_buffer),
                          static_cast<const float*>(topk_weights), static_cast<uint8_t*>(out), tokens, hidden, topk};
    const int sms = sm_count();
    if (sms <= 0) return MX8_ERR_CUDA;
    moe::epilogue_kernel<<<sms * 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        note_cuda_error("moe epilogue launch", cudaGetErrorString(e));
        return MX8_ERR_CUDA;
    }
    return MX8_OK;
}

extern "C" int mx8_moe_bwd_prologue(const void* d_output, const void* topk_weights, void* d_combine_buffer, int tokens, int hidden,
                                    int topk, void* stream) {
    using namespace mx8;
    if (!d_output || !topk_weights || !d_combine_buffer) return MX8_ERR_ARG;
    if (tokens <= 0 || topk <= 0) return MX8_ERR_ARG;
    if (hidden <= 0 || hidden % 8) return MX8_ERR_SHAPE;
    if (!aligned16(d_output) || !aligned16(d_combine_buffer)) return MX8_ERR_ALIGN;
    int rc = check_device_sm100();
    if (rc != MX8_OK) return rc;
    const int sms = sm_count();
    if (sms <= 0) return MX8_ERR_CUDA;
    moe::bwd_prologue_kernel<<<sms * 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(d_output), static_cast<const float*>(topk_weights), static_cast<uint8_t*>(d_combine_buffer), tokens,
        hidden, topk);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        note_cuda_error("moe bwd prologue launch", cudaGetErrorString(e));
        return MX8_ERR_CUDA;
    }
    return MX8_OK;
}

extern "C" int mx8_moe_bwd_epilogue(const void* d_x_shared, const void* d_x_routed_buffer, void* d_x, int tokens, int hidden,
                                    int topk, void* stream) {
    using namespace mx8;
    if (!d_x_routed_buffer || !d_x) return MX8_ERR_ARG;
    if (tokens <= 0 || topk <= 0) return MX8_ERR_ARG;
    if (hidden <= 0 || hidden % 8) return MX8_ERR_SHAPE;
    if (!aligned16(d_x_shared) || !aligned16(d_x_routed_buffer) || !aligned16(d_x)) return MX8_ERR_ALIGN;
    int rc = check_device_sm100();
    if (rc != MX8_OK) return rc;
    moe::EpilogueParams p{static_cast<const uint8_t*>(d_x_shared), static_cast<const uint8_t*>(d_x_routed_buffer), nullptr,
                          static_cast<uint8_t*>(d_x), tokens, hidden, topk};
    const int sms = sm_count();
    if (sms <= 0) return MX8_ERR_CUDA;
    moe::epilogue_kernel<<<sms * 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        note_cuda_error("moe bwd epilogue launch", cudaGetErrorString(e));
        return MX8_ERR_CUDA;
    }
    return MX8_OK;
}
