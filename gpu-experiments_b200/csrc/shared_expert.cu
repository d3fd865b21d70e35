// Element-wise pieces of the MoE layer's shared expert (bf16 activations): SwiGLU forward and
// backward, and the transposes that turn token-major activations into the K-major operands of the
// weight-gradient GEMMs.  All three are pure streaming kernels: 16-byte accesses, grid sized to the
// machine, fp32 arithmetic with the fast exponential and reciprocal the routed path uses as well.
#include <cuda_bf16.h>

#include "mx8_host.cuh"

namespace mx8 {
namespace shared_expert {

__device__ __forceinline__ float2 unpack(uint32_t w) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
}
__device__ __forceinline__ uint32_t pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float silu(float g, float& den) {
    den = __expf(-g) + 1.0f;
    return __fdividef(g, den);
}

__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up,
                                                         uint4* __restrict__ hidden, long long n16) {
    for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n16; i += gridDim.x * 256ll) {
        const uint4 g = __ldcs(gate + i), u = __ldcs(up + i);
        const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 a = unpack(gw[j]), b = unpack(uw[j]);
            float d0, d1;
            o[j] = pack(silu(a.x, d0) * b.x, silu(a.y, d1) * b.y);
        }
        hidden[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const uint4* __restrict__ d_hidden, const uint4* __restrict__ gate,
                                                         const uint4* __restrict__ up, uint4* __restrict__ d_gate,
                                                         uint4* __restrict__ d_up, long long n16) {
    for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n16; i += gridDim.x * 256ll) {
        const uint4 h = __ldcs(d_hidden + i), g = __ldcs(gate + i), u = __ldcs(up + i);
        const uint32_t hw[4] = {h.x, h.y, h.z, h.w}, gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
        uint32_t og[4], ou[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 dh = unpack(hw[j]), a = unpack(gw[j]), b = unpack(uw[j]);
            float den0, den1;
            const float s0 = silu(a.x, den0), s1 = silu(a.y, den1);
            const float ds0 = __fdividef(1.0f - s0, den0) + s0, ds1 = __fdividef(1.0f - s1, den1) + s1;
            og[j] = pack(dh.x * ds0 * b.x, dh.y * ds1 * b.y);
            ou[j] = pack(s0 * dh.x, s1 * dh.y);
        }
        d_gate[i] = make_uint4(og[0], og[1], og[2], og[3]);
        d_up[i] = make_uint4(ou[0], ou[1], ou[2], ou[3]);
    }
}

// 64 x 64 tile per block of 256 threads: rows come in as 128-byte segments, leave as 128-byte
// segments of the transposed matrix; the shared tile is padded to keep both sides conflict-free.
__global__ void __launch_bounds__(256) transpose_kernel(const uint16_t* __restrict__ in, uint16_t* __restrict__ out, int rows,
                                                        int cols) {
    __shared__ uint16_t tile[64][66];
    const int tiles_c = cols / 64;
    const long long num_tiles = static_cast<long long>(rows / 64) * tiles_c;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;             // 32 x 8
    for (long long t = blockIdx.x; t < num_tiles; t += gridDim.x) {
        const int r0 = static_cast<int>(t / tiles_c) * 64, c0 = static_cast<int>(t % tiles_c) * 64;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int r = ty + 8 * i;
            const uint32_t w = *reinterpret_cast<const uint32_t*>(in + static_cast<size_t>(r0 + r) * cols + c0 + 2 * tx);
            tile[r][2 * tx] = static_cast<uint16_t>(w);
            tile[r][2 * tx + 1] = static_cast<uint16_t>(w >> 16);
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int c = ty + 8 * i;                                    // row of the output tile
            const uint32_t w = static_cast<uint32_t>(tile[2 * tx][c]) | (static_cast<uint32_t>(tile[2 * tx + 1][c]) << 16);
            *reinterpret_cast<uint32_t*>(out + static_cast<size_t>(c0 + c) * rows + r0 + 2 * tx) = w;
        }
        __syncthreads();
    }
}

static int launch_done(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        note_cuda_error(what, cudaGetErrorString(e));
        return MX8_ERR_CUDA;
    }
    return MX8_OK;
}

static int grid_for(long long work_items) {
    const long long want = (work_items + 255) / 256;
    const long long cap = static_cast<long long>(sm_count()) * 8;
    return static_cast<int>(want < cap ? (want > 0 ? want : 1) : cap);
}

}  // namespace shared_expert
}  // namespace mx8

extern "C" {

int mx8_swiglu_bf16(const void* gate, const void* up, void* hidden, long long n, void* stream) {
    using namespace mx8;
    if (!gate || !up || !hidden) return MX8_ERR_ARG;
    if (n <= 0 || n % 8) return MX8_ERR_SHAPE;
    if (!aligned16(gate) || !aligned16(up) || !aligned16(hidden)) return MX8_ERR_ALIGN;
    int rc = check_device_sm100();
    if (rc != MX8_OK) return rc;
    const long long n16 = n / 8;
    shared_expert::swiglu_fwd_kernel<<<shared_expert::grid_for(n16), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(gate), static_cast<const uint4*>(up), static_cast<uint4*>(hidden), n16);
    return shared_expert::launch_done("swiglu_fwd_kernel launch");
}

int mx8_swiglu_bwd_bf16(const void* d_hidden, const void* gate, const void* up, void* d_gate, void* d_up, long long n,
                        void* stream) {
    using namespace mx8;
    if (!d_hidden || !gate || !up || !d_gate || !d_up) return MX8_ERR_ARG;
    if (n <= 0 || n % 8) return MX8_ERR_SHAPE;
    if (!aligned16(d_hidden) || !aligned16(gate) || !aligned16(up) || !aligned16(d_gate) || !aligned16(d_up)) return MX8_ERR_ALIGN;
    int rc = check_device_sm100();
    if (rc != MX8_OK) return rc;
    const long long n16 = n / 8;
    shared_expert::swiglu_bwd_kernel<<<shared_expert::grid_for(n16), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(d_hidden), static_cast<const uint4*>(gate), static_cast<const uint4*>(up),
        static_cast<uint4*>(d_gate), static_cast<uint4*>(d_up), n16);
    return shared_expert::launch_done("swiglu_bwd_kernel launch");
}

int mx8_transpose_bf16(const void* in, void* out, int rows, int cols, void* stream) {
    using namespace mx8;
    if (!in || !out || in == out) return MX8_ERR_ARG;
    if (rows <= 0 || cols <= 0 || rows % 64 || cols % 64) return MX8_ERR_SHAPE;
    if (!aligned16(in) || !aligned16(out)) return MX8_ERR_ALIGN;
    int rc = check_device_sm100();
    if (rc != MX8_OK) return rc;
    const long long tiles = static_cast<long long>(rows / 64) * (cols / 64);
    const long long cap = static_cast<long long>(sm_count()) * 8;
    const int grid = static_cast<int>(tiles < cap ? tiles : cap);
    shared_expert::transpose_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(in), static_cast<uint16_t*>(out), rows, cols);
    return shared_expert::launch_done("transpose_kernel launch");
}

}  // extern "C"
