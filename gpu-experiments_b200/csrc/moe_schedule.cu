// Expert-parallel MoE routing schedule (integer, deterministic).
//
// Input: the routing table of every rank, topk_all[world][tokens][topk] (global expert ids).
// Output for THIS rank (which owns experts [rank*E, rank*E+E)): one row per routed (token, k) pair
// that selected a local expert, grouped by expert, every expert's segment padded to a multiple of
// 256 rows (the GEMM tile height):
//   peer_rank[row]      source rank of the row, -1 for padding and unused rows
//   peer_token_idx[row] token * topk + k on the source rank
//   tokens_per_expert[e] padded segment length, num_tokens[0] their sum
// Order inside a segment: round j takes the j-th pair of every source rank that still has one, ranks
// ascending — the placement rule of the reference's scheduler
// (blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.cu:34-147), which this file replaces.
// "The j-th pair of a source rank" is the reference's order too: its placement kernel gives entry
// idx = token*topk+k of a rank's table to thread idx % 1024 of a 1024-thread block, and the threads
// take consecutive ordinals in thread order (:99-146), so the pairs of one (expert, source rank) are
// ordered by (idx % 1024, idx / 1024).  For tables of at most 1024 entries per rank that is table
// order; for larger ones it is not, and every routed tensor of the layer depends on it.
// Differences: a schedule larger than `capacity` is reported through the device status word
// (the reference executes `trap`), and the counting scratch is supplied by the caller.
// Two forms: a counting sort over chunks of the table when the scratch has room for the per-chunk
// counts (mx8_moe_schedule_scratch_bytes), else one scan of the table per (local expert, source rank).
#include <atomic>

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

// block (expert e, source rank r): thread t owns the entries t, t + 1024, ... of rank r's table; the
// pairs that chose e take ordinals thread by thread (an exclusive prefix over the threads' hit
// counts), entries of one thread in ascending order
__global__ void __launch_bounds__(THREADS) sched_place_kernel(SchedParams p) {
    extern __shared__ int n_from[];           // [world] pairs per source rank for this expert
    __shared__ int warp_sums[THREADS / 32];
    const int e = blockIdx.x / p.world, r = blockIdx.x % p.world;
    for (int i = threadIdx.x; i < p.world; i += blockDim.x) n_from[i] = p.counts[e * p.world + i];
    __syncthreads();
    if (n_from[r] == 0) return;
    const int base = p.counts[p.experts * p.world + e];
    const int want = p.rank * p.experts + e;
    const int stride = p.tokens * p.topk_k;
    const int* src = p.topk + static_cast<size_t>(r) * stride;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int mine = 0;
    for (int i = threadIdx.x; i < stride; i += THREADS) mine += (src[i] == want) ? 1 : 0;
    int incl = mine;                                                 // inclusive scan over the block
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int v = __shfl_up_sync(0xFFFFFFFFu, incl, d);
        if (lane >= d) incl += v;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    int j = incl - mine;
    for (int w = 0; w < warp; ++w) j += warp_sums[w];
    if (mine == 0) return;
    for (int i = threadIdx.x; i < stride; i += THREADS) {
        if (src[i] != want) continue;
        int dst = base;
        for (int q = 0; q < p.world; ++q) {
            const int n = n_from[q];
            dst += min(n, j) + ((q < r && n > j) ? 1 : 0);
        }
        if (dst < p.capacity) {
            p.peer_rank[dst] = r;
            p.peer_token_idx[dst] = i;
        }
        ++j;
    }
}

// ---------------------------------------------------------------------------------------------
// Counting-sort form (used when the scratch buffer is large enough).  A rank's table is read as a
// matrix of `rows` x 1024 entries (entry idx at row idx / 1024, column idx % 1024) and the order of the
// pairs is column-major over it.  A chunk is a band of consecutive columns holding about 1024 entries;
// inside a chunk, position pos = (column - first column) * rows + row.  One pass counts every chunk's
// pairs per local expert, a scan turns the counts into each chunk's first ordinal per (expert, rank),
// and a second pass places the pairs.  Every entry of the table is read twice in total, instead of
// once per local expert.
// Scratch: counts[E*W] | bases[E] | chunk_counts[W * chunks_per_rank * E].
constexpr int CHUNK = 1024;

struct ChunkGeom {
    int rows;      // entries per column = ceil(stride / 1024)
    int cols;      // columns per chunk
    int chunks;    // chunks per rank
};

__host__ __device__ inline ChunkGeom chunk_geom(int tokens, int topk_k) {
    ChunkGeom g;
    const long long stride = static_cast<long long>(tokens) * topk_k;
    g.rows = static_cast<int>((stride + THREADS - 1) / THREADS);
    g.cols = g.rows >= CHUNK ? 1 : CHUNK / g.rows;
    g.chunks = (THREADS + g.cols - 1) / g.cols;
    return g;
}

__host__ __device__ inline int chunks_per_rank(int tokens, int topk_k) { return chunk_geom(tokens, topk_k).chunks; }

// block (r, c): histogram of chunk c of rank r over the local experts; also clears the outputs
__global__ void __launch_bounds__(CHUNK) sched_chunk_count_kernel(SchedParams p) {
    extern __shared__ int hist[];             // [experts]
    for (int i = blockIdx.x * CHUNK + threadIdx.x; i < p.capacity; i += gridDim.x * CHUNK) p.peer_rank[i] = -1;
    for (int i = threadIdx.x; i < p.experts; i += CHUNK) hist[i] = 0;
    __syncthreads();
    const ChunkGeom g = chunk_geom(p.tokens, p.topk_k);
    const int r = blockIdx.x / g.chunks, c = blockIdx.x % g.chunks;
    const int stride = p.tokens * p.topk_k;
    const int col0 = c * g.cols, ncols = min(g.cols, THREADS - col0);
    const int* src = p.topk + static_cast<size_t>(r) * stride;
    // the order inside the chunk does not matter for counting: walk it row by row (contiguous reads)
    for (int q = threadIdx.x; q < ncols * g.rows; q += CHUNK) {
        const int i = (q / ncols) * THREADS + col0 + q % ncols;
        if (i < stride) {
            const int e = src[i] - p.rank * p.experts;
            if (e >= 0 && e < p.experts) atomicAdd(&hist[e], 1);
        }
    }
    __syncthreads();
    int* cc = p.counts + p.experts * p.world + p.experts + static_cast<size_t>(blockIdx.x) * p.experts;
    for (int e = threadIdx.x; e < p.experts; e += CHUNK) cc[e] = hist[e];
}

// one block: chunk counts -> exclusive prefix per (expert, rank); totals; padded segments and bases.
// Prefix over chunks: 32 (expert, rank) pairs at a time, one per lane (neighbouring lanes read
// neighbouring words), the chunks split into 32 consecutive ranges, one per warp; warps exchange
// their range totals through shared memory.
__global__ void __launch_bounds__(1024) sched_scan_kernel(SchedParams p) {
    __shared__ int warp_tot[32];
    __shared__ int range_tot[32][33];
    __shared__ int carry;
    const int cpr = chunks_per_rank(p.tokens, p.topk_k);
    int* cc = p.counts + p.experts * p.world + p.experts;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int per_warp = (cpr + 31) / 32;
    const int c_begin = min(cpr, warp * per_warp), c_end = min(cpr, c_begin + per_warp);
    const int pairs = p.experts * p.world;
    if (cpr <= 64) {
        // few chunks: one thread walks the chunks of its pair, no exchange between warps
        for (int idx = threadIdx.x; idx < pairs; idx += blockDim.x) {
            const int r = idx / p.experts, e = idx - r * p.experts;
            int running = 0;
            for (int c = 0; c < cpr; ++c) {
                int* cell = cc + (static_cast<size_t>(r) * cpr + c) * p.experts + e;
                const int v = *cell;
                *cell = running;
                running += v;
            }
            p.counts[e * p.world + r] = running;
        }
    } else
    for (int g0 = 0; g0 < pairs; g0 += 32) {
        const int idx = g0 + lane;
        const bool live = idx < pairs;
        const int r = live ? idx / p.experts : 0, e = live ? idx - r * p.experts : 0;
        int* q = cc + (static_cast<size_t>(r) * cpr + c_begin) * p.experts + e;
        int sum = 0;
        if (live)
            for (int c = c_begin; c < c_end; ++c) sum += q[static_cast<size_t>(c - c_begin) * p.experts];
        range_tot[warp][lane] = sum;
        __syncthreads();
        int running = 0, total = 0;
        for (int w = 0; w < 32; ++w) {
            const int v = range_tot[w][lane];
            if (w < warp) running += v;
            total += v;
        }
        if (live) {
            for (int c = c_begin; c < c_end; ++c) {
                int* cell = q + static_cast<size_t>(c - c_begin) * p.experts;
                const int v = *cell;
                *cell = running;
                running += v;
            }
            if (warp == 0) p.counts[e * p.world + r] = total;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int e0 = 0; e0 < p.experts; e0 += blockDim.x) {
        const int e = e0 + threadIdx.x;
        int padded = 0;
        if (e < p.experts) {
            int n = 0;
            for (int r = 0; r < p.world; ++r) n += p.counts[e * p.world + r];
            padded = (n + PAD - 1) / PAD * PAD;
            p.tokens_per_expert[e] = padded;
        }
        int incl = padded;                                           // inclusive scan inside the warp
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int v = __shfl_up_sync(0xFFFFFFFFu, incl, d);
            if (lane >= d) incl += v;
        }
        if (lane == 31) warp_tot[warp] = incl;
        __syncthreads();
        int before = carry;
        for (int w = 0; w < warp; ++w) before += warp_tot[w];
        if (e < p.experts) p.counts[p.experts * p.world + e] = before + incl - padded;
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) carry = before + incl;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        p.num_tokens[0] = carry;
        if (carry > p.capacity) atomicCAS(p.status, 0, DEV_MOE_CAPACITY);
    }
}

// block (r, c): ordinal of every pair of the chunk among the pairs of its (expert, rank), in the
// chunk's column-major order, then its row.  A chunk of more than 1024 entries (a table of more than
// a million entries per rank) is walked in windows of 1024 positions.
__global__ void __launch_bounds__(CHUNK) sched_chunk_place_kernel(SchedParams p) {
    extern __shared__ int run[];              // [experts] ordinal of the next pair of this rank per expert
    const ChunkGeom g = chunk_geom(p.tokens, p.topk_k);
    const int r = blockIdx.x / g.chunks, c = blockIdx.x % g.chunks;
    const int* cc = p.counts + p.experts * p.world + p.experts + static_cast<size_t>(blockIdx.x) * p.experts;
    for (int e = threadIdx.x; e < p.experts; e += CHUNK) run[e] = cc[e];
    const int stride = p.tokens * p.topk_k;
    const int col0 = c * g.cols, ncols = min(g.cols, THREADS - col0);
    const int entries = ncols * g.rows;
    const int* src = p.topk + static_cast<size_t>(r) * stride;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    for (int pos0 = 0; pos0 < entries; pos0 += CHUNK) {
        const int pos = pos0 + threadIdx.x;
        int e = -1, i = 0;
        if (pos < entries) {
            i = (pos % g.rows) * THREADS + col0 + pos / g.rows;
            if (i < stride) {
                e = src[i] - p.rank * p.experts;
                if (e < 0 || e >= p.experts) e = -1;
            }
        }
        const unsigned same = __match_any_sync(0xFFFFFFFFu, e);      // lanes of this warp with the same expert
        const int in_warp = __popc(same & ((1u << lane) - 1));
        int j = 0;
        for (int w = 0; w < CHUNK / 32; ++w) {                       // warps take their ordinals in position order
            if (warp == w && e >= 0) {
                j = run[e] + in_warp;
                __syncwarp(same);
                if (in_warp == 0) run[e] += __popc(same);
            }
            __syncthreads();
        }
        if (e < 0) continue;
        int dst = p.counts[p.experts * p.world + e];
        for (int q = 0; q < p.world; ++q) {
            const int n = p.counts[e * p.world + q];
            dst += min(n, j) + ((q < r && n > j) ? 1 : 0);
        }
        if (dst < p.capacity) {
            p.peer_rank[dst] = r;
            p.peer_token_idx[dst] = i;
        }
    }
}

static long long fast_scratch_ints(int world, int tokens, int topk_k, int experts) {
    return static_cast<long long>(experts) * (world + 1) + static_cast<long long>(world) * chunks_per_rank(tokens, topk_k) * experts;
}

static int run_schedule_fast(const SchedParams& p, cudaStream_t st) {
    const int blocks = p.world * chunks_per_rank(p.tokens, p.topk_k);
    sched_chunk_count_kernel<<<blocks, CHUNK, p.experts * sizeof(int), st>>>(p);
    sched_scan_kernel<<<1, 1024, 0, st>>>(p);
    sched_chunk_place_kernel<<<blocks, CHUNK, p.experts * sizeof(int), st>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        note_cuda_error("moe schedule launch", cudaGetErrorString(e));
        return MX8_ERR_CUDA;
    }
    return MX8_OK;
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
                                void* scratch, size_t scratch_bytes, void* stream) {
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
    const long long have = static_cast<long long>(scratch_bytes / sizeof(int));
    if (have < static_cast<long long>(num_local_experts) * (world + 1)) {
        note_cuda_error("mx8_moe_schedule", "scratch smaller than num_local_experts * (world + 1) ints");
        return MX8_ERR_LIMIT;
    }
    // the counting-sort form needs room for the per-chunk counts; without it the scan-per-expert form runs
    if (have >= moe::fast_scratch_ints(world, tokens, topk, num_local_experts))
        return moe::run_schedule_fast(p, static_cast<cudaStream_t>(stream));
    return moe::run_schedule(p, static_cast<cudaStream_t>(stream));
}

extern "C" size_t mx8_moe_schedule_scratch_bytes(int world, int tokens, int topk, int num_local_experts) {
    if (world <= 0 || tokens <= 0 || topk <= 0 || num_local_experts <= 0) return 0;
    return static_cast<size_t>(mx8::moe::fast_scratch_ints(world, tokens, topk, num_local_experts)) * sizeof(int);
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
    static std::atomic<int*> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    int* have = cached[dev].load(std::memory_order_acquire);
    if (!have) {
        int* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_schedule_scratch);
        if (e != cudaSuccess) {
            note_cuda_error("cudaGetSymbolAddress(schedule scratch)", cudaGetErrorString(e));
            return nullptr;
        }
        cached[dev].store(p, std::memory_order_release);
        have = p;
    }
    return have;
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
                            num_tokens, tokens_per_expert, scratch, moe::STATIC_SCRATCH_INTS * sizeof(int), stream);
}

// ---------------------------------------------------------------------------------------------
// Row bounds of `minibatches` groups of consecutive local experts: bounds[b] = rows before the first
// expert of minibatch b (experts are split as evenly as the count allows), bounds[minibatches] = all
// rows.  The windowed entry points take pointers into this array.
namespace mx8 {
namespace moe {
struct ExpertSplit {
    int first[65];       // first expert of every group, first[minibatches] = experts; first[0] < 0: even split
};

__global__ void __launch_bounds__(256) minibatch_bounds_kernel(const int* tokens_per_expert, int experts, int minibatches, int* bounds,
                                                               const ExpertSplit split) {
    // one warp per bound: sum of the segments of the experts before the group's first one
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (int b = warp; b <= minibatches; b += warps) {
        const int first = split.first[0] < 0 ? static_cast<int>(static_cast<long long>(b) * experts / minibatches) : split.first[b];
        int sum = 0;
        for (int e = lane; e < first; e += 32) sum += tokens_per_expert[e];
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, d);
        if (lane == 0) bounds[b] = sum;
    }
}
}  // namespace moe
}  // namespace mx8

extern "C" int mx8_moe_minibatch_bounds(const void* tokens_per_expert, int num_local_experts, int minibatches, void* bounds,
                                        void* stream) {
    return mx8_moe_minibatch_bounds_split(tokens_per_expert, num_local_experts, minibatches, nullptr, bounds, stream);
}

extern "C" int mx8_moe_minibatch_bounds_split(const void* tokens_per_expert, int num_local_experts, int minibatches,
                                              const int* first_expert, void* bounds, void* stream) {
    using namespace mx8;
    if (!tokens_per_expert || !bounds) return MX8_ERR_ARG;
    if (num_local_experts <= 0 || minibatches <= 0 || minibatches > num_local_experts || minibatches > 64) return MX8_ERR_ARG;
    moe::ExpertSplit split;
    split.first[0] = -1;
    if (first_expert) {
        if (first_expert[0] != 0 || first_expert[minibatches] != num_local_experts) return MX8_ERR_ARG;
        for (int b = 0; b <= minibatches; ++b) {
            if (b > 0 && first_expert[b] < first_expert[b - 1]) return MX8_ERR_ARG;
            split.first[b] = first_expert[b];
        }
    }
    int rc = check_device_sm100();
    if (rc != MX8_OK) return rc;
    moe::minibatch_bounds_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const int*>(tokens_per_expert),
                                                                                num_local_experts, minibatches, static_cast<int*>(bounds),
                                                                                split);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        note_cuda_error("minibatch bounds launch", cudaGetErrorString(e));
        return MX8_ERR_CUDA;
    }
    return MX8_OK;
}
