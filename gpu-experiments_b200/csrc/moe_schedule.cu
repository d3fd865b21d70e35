// Expert-parallel MoE routing schedule (integer, deterministic).
//
// Input: the routing table of every rank, topk_all[world][tokens][topk] (global expert ids).
// Output for THIS rank (which owns experts [rank*E, rank*E+E)): one row per routed (token, k) pair
// that selected a local expert, grouped by expert, every expert's segment padded to a multiple of
// 256 rows (the GEMM tile height):
//   peer_rank[row]      source rank of the row, -1 for padding and unused rows
//   peer_token_idx[row] token * topk + k on the source rank
//   tokens_per_expert[e] padded segment length, num_tokens[0] their sum
// Order inside a segment: round j takes the j-th pair (in token*topk+k order) of every source rank
// that still has one, ranks ascending — the placement rule of the reference's scheduler
// (blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.cu:34-147), which this file replaces.
// Differences: a schedule larger than `capacity` is reported through the device status word
// (the reference executes `trap`), and the counting scratch is supplied by the caller.
#include "mx8_host.cuh"
#include "mx8_ptx.cuh"

namespace mx8 {
namespace moe {

constexpr int PAD = 256;
constexpr int THREADS = 1024;
constexpr int DEV_MOE_CAPACITY = 16;   // device status: schedule does not fit `capacity`

struct SchedParams {
    const int* topk;        // [world][tokens][topk]
    int world, tokens, topk_k, experts, capacity, rank;
    int* peer_rank;         // [capacity]
    int* peer_token_idx;    // [capacity]
    int* num_tokens;        // [1]
    int* tokens_per_expert; // [experts]
    int* counts;            // scratch [experts * world] then [experts] segment bases
    int* status;
};

__global__ void sched_init_kernel(SchedParams p) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < p.capacity) p.peer_rank[i] = -1;
    if (i < p.experts * p.world + p.experts) p.counts[i] = 0;
    if (i == 0) p.num_tokens[0] = 0;
}

// pairs routed from each source rank to each local expert
__global__ void sched_count_kernel(SchedParams p) {
    extern __shared__ int hist[];   // [experts * world]
    const int bins = p.experts * p.world;
    for (int i = threadIdx.x; i < bins; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    const int stride = p.tokens * p.topk_k;
    const long long total = static_cast<long long>(p.world) * stride;
    const int first = p.rank * p.experts;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int e = p.topk[i] - first;
        if (e >= 0 && e < p.experts) atomicAdd(&hist[e * p.world + static_cast<int>(i / stride)], 1);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < bins; i += blockDim.x)
        if (hist[i]) atomicAdd(&p.counts[i], hist[i]);
}

// padded segment lengths, segment bases, total; one block
__global__ void sched_pad_kernel(SchedParams p) {
    if (threadIdx.x == 0) {
        int base = 0;
        for (int e = 0; e < p.experts; ++e) {
            int n = 0;
            for (int r = 0; r < p.world; ++r) n += p.counts[e * p.world + r];
            const int padded = (n + PAD - 1) / PAD * PAD;
            p.tokens_per_expert[e] = padded;
            p.counts[p.experts * p.world + e] = base;
            base += padded;
        }
        p.num_tokens[0] = base;
        if (base > p.capacity) atomicCAS(p.status, 0, DEV_MOE_CAPACITY);
    }
}

// block (expert e, source rank r): rank the pairs of r that chose e and place them
__global__ void sched_place_kernel(SchedParams p) {
    extern __shared__ int n_from[];           // [world] pairs per source rank for this expert
    __shared__ int warp_sums[THREADS / 32];
    __shared__ int running;
    const int e = blockIdx.x / p.world, r = blockIdx.x % p.world;
    for (int i = threadIdx.x; i < p.world; i += blockDim.x) n_from[i] = p.counts[e * p.world + i];
    if (threadIdx.x == 0) running = 0;
    __syncthreads();
    if (n_from[r] == 0) return;
    const int base = p.counts[p.experts * p.world + e];
    const int want = p.rank * p.experts + e;
    const int stride = p.tokens * p.topk_k;
    const int* src = p.topk + static_cast<size_t>(r) * stride;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i0 = 0; i0 < stride; i0 += blockDim.x) {
        const int i = i0 + threadIdx.x;
        const int hit = (i < stride && src[i] == want) ? 1 : 0;
        // exclusive rank of this pair among the block's hits
        const unsigned ballot = __ballot_sync(0xFFFFFFFFu, hit);
        const int in_warp = __popc(ballot & ((1u << lane) - 1));
        if (lane == 0) warp_sums[warp] = __popc(ballot);
        __syncthreads();
        int before = running;
        for (int w = 0; w < warp; ++w) before += warp_sums[w];
        if (hit) {
            const int j = before + in_warp;
            int dst = base;
            for (int q = 0; q < p.world; ++q) {
                const int n = n_from[q];
                dst += min(n, j) + ((q < r && n > j) ? 1 : 0);
            }
            if (dst < p.capacity) {
                p.peer_rank[dst] = r;
                p.peer_token_idx[dst] = i;
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int s = 0;
            for (int w = 0; w < THREADS / 32; ++w) s += warp_sums[w];
            running += s;
        }
        __syncthreads();
    }
}

static int run_schedule(const SchedParams& p, cudaStream_t st) {
    const int bins = p.experts * p.world + p.experts;
    const int init_n = p.capacity > bins ? p.capacity : bins;
    sched_init_kernel<<<(init_n + 255) / 256, 256, 0, st>>>(p);
    const long long total = static_cast<long long>(p.world) * p.tokens * p.topk_k;
    long long cb = (total + THREADS - 1) / THREADS;
    const int count_blocks = static_cast<int>(cb < 592 ? cb : 592);
    sched_count_kernel<<<count_blocks, THREADS, p.experts * p.world * sizeof(int), st>>>(p);
    sched_pad_kernel<<<1, 32, 0, st>>>(p);
    sched_place_kernel<<<p.experts * p.world, THREADS, p.world * sizeof(int), st>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        note_cuda_error("moe schedule launch", cudaGetErrorString(e));
        return MX8_ERR_CUDA;
    }
    return MX8_OK;
}

}  // namespace moe
}  // namespace mx8

extern "C" int mx8_moe_schedule(const void* topk_all, int world, int tokens, int topk, int num_local_experts, int capacity,
                                int rank, void* peer_rank, void* peer_token_idx, void* num_tokens, void* tokens_per_expert,
                                void* scratch, void* stream) {
    using namespace mx8;
    if (!topk_all || !peer_rank || !peer_token_idx || !num_tokens || !tokens_per_expert || !scratch) return MX8_ERR_ARG;
    if (world <= 0 || tokens <= 0 || topk <= 0 || num_local_experts <= 0 || capacity <= 0 || rank < 0 || rank >= world)
        return MX8_ERR_ARG;
    if (capacity % 256) return MX8_ERR_SHAPE;
    if (static_cast<long long>(num_local_experts) * world * sizeof(int) > 48 * 1024) return MX8_ERR_SHAPE;
    int rc = check_device_sm100();
    if (rc != MX8_OK) return rc;
    moe::SchedParams p{};
    p.topk = static_cast<const int*>(topk_all);
    p.world = world; p.tokens = tokens; p.topk_k = topk; p.experts = num_local_experts; p.capacity = capacity; p.rank = rank;
    p.peer_rank = static_cast<int*>(peer_rank);
    p.peer_token_idx = static_cast<int*>(peer_token_idx);
    p.num_tokens = static_cast<int*>(num_tokens);
    p.tokens_per_expert = static_cast<int*>(tokens_per_expert);
    p.counts = static_cast<int*>(scratch);
    p.status = device_status_ptr();
    if (!p.status) return MX8_ERR_CUDA;
    return moe::run_schedule(p, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------------------------
// Variant of the schedule that needs no scratch buffer from the caller.
//
// Some hosts of this library cannot hand over scratch memory: a serving loop whose memory plan is
// frozen after start-up, or a plugin that runs inside someone else's allocator and may not call
// cudaMalloc (which synchronizes the device) on the request path.  For them the counting scratch
// lives in this fixed array, which every device that loads the library keeps until the process
// exits (64 KiB).  The kernels clear the part they use at the start of every call; the contents
// left behind by the previous call are never read.  All calls on a device share the array, so two
// calls that overlap on the GPU (different streams, no ordering between them) race.
namespace mx8 {
namespace moe {

constexpr int STATIC_SCRATCH_INTS = 16384;     // limit: num_local_experts * (world + 1) <= 16384
static __device__ __align__(256) int g_schedule_scratch[STATIC_SCRATCH_INTS];

// Device address of the array on the current device.  In host code the array's name is only a
// handle for the runtime, not an address a kernel can use, so it is resolved once per device.
static int* static_scratch_ptr() {
    static int* cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!cached[dev]) {
        int* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_schedule_scratch);
        if (e != cudaSuccess) {
            note_cuda_error("cudaGetSymbolAddress(schedule scratch)", cudaGetErrorString(e));
            return nullptr;
        }
        cached[dev] = p;
    }
    return cached[dev];
}

}  // namespace moe
}  // namespace mx8

extern "C" int mx8_moe_schedule_static(const void* topk_all, int world, int tokens, int topk, int num_local_experts,
                                       int capacity, int rank, void* peer_rank, void* peer_token_idx, void* num_tokens,
                                       void* tokens_per_expert, void* stream) {
    using namespace mx8;
    if (world <= 0 || num_local_experts <= 0) return MX8_ERR_ARG;
    if (static_cast<long long>(num_local_experts) * (static_cast<long long>(world) + 1) > moe::STATIC_SCRATCH_INTS) {
        note_cuda_error("mx8_moe_schedule_static", "num_local_experts * (world + 1) exceeds the built-in scratch of 16384 ints");
        return MX8_ERR_LIMIT;
    }
    int rc = check_device_sm100();
    if (rc != MX8_OK) return rc;
    int* scratch = moe::static_scratch_ptr();     // first call on a device resolves the address
    if (!scratch) return MX8_ERR_CUDA;
    return mx8_moe_schedule(topk_all, world, tokens, topk, num_local_experts, capacity, rank, peer_rank, peer_token_idx,
                            num_tokens, tokens_per_expert, scratch, stream);
}
