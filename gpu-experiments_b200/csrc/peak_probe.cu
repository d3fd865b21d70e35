// Tensor-core roof of the MXFP8 GEMM, measured: the GEMM kernel's own instruction
// (tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale, M = 256, N = 256, K = 32) issued back to back by every
// CTA pair from operands that already sit in shared memory and scales that already sit in TMEM.  No global
// memory traffic, no epilogue: what remains is what the tensor pipes sustain for this instruction shape, at
// whatever clock the power cap allows.  The benchmark divides the GEMM's rate by this figure.
// The reference has no counterpart; it quotes the data sheet's 4.5 PFLOP/s.
#include <atomic>

#include "mx8_host.cuh"
#include "mx8_ptx.cuh"

namespace mx8 {
namespace probe {

constexpr int TILE_BYTES = 128 * 128;     // one CTA's 128 x 128 E4M3 operand tile (SWIZZLE_128B image)
constexpr int STAGES = 4;                 // distinct operand tiles the MMAs rotate over
constexpr int GROUP = 8;                  // K steps (of four MMAs each) between two commits
constexpr int SMEM = 2 * STAGES * TILE_BYTES + 1024 + 64;

__global__ void __launch_bounds__(128, 1) mma_peak_kernel(int k_steps, int* status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bar = base + 2 * STAGES * TILE_BYTES;
    volatile uint32_t* tmem_ptr = reinterpret_cast<volatile uint32_t*>(base_ptr + 2 * STAGES * TILE_BYTES + 16);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + 2 * STAGES * TILE_BYTES + 32);
    const AbortCtl ab{abort_flag, status};
    const int warp = threadIdx.x >> 5;
    const uint32_t rank = cluster_ctarank();
    // operands: small E4M3 values with a varying bit pattern (0x30..0x3F: 0.5 .. 1.875), so the data paths toggle
    for (int i = threadIdx.x; i < 2 * STAGES * TILE_BYTES / 4; i += blockDim.x) {
        const uint32_t h = (static_cast<uint32_t>(i) * 2654435761u) ^ (blockIdx.x * 40503u);
        reinterpret_cast<uint32_t*>(base_ptr)[i] = 0x30303030u | (h & 0x0F0F0F0Fu) | ((h >> 3) & 0x80808080u);
    }
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(bar, 1);
        fence_mbar_init();
    }
    fence_proxy_async_smem();
    if (warp == 0) {
        tmem_alloc<2>(smem_u32(const_cast<uint32_t*>(tmem_ptr)), 512);
        tmem_relinquish<2>();
    }
    __syncwarp();
    tc_fence_before();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr;
    if (warp == 1 && rank == 0) {
        const bool leader = elect_one();
        // scale columns hold whatever TMEM held: any E8M0 byte is a valid scale, the products are never read
        const uint32_t sf = tmem_base + 480;
        uint32_t ph = 0;
        bool ok = true;
        for (int ks = 0; ks < k_steps && ok; ks += GROUP) {
            if (leader) {
#pragma unroll
                for (int g = 0; g < GROUP; ++g) {
                    const uint32_t st = static_cast<uint32_t>((ks + g) % STAGES);
                    const uint32_t a_lo = desc_sw128_lo(base + st * TILE_BYTES);
                    const uint32_t b_lo = desc_sw128_lo(base + (STAGES + st) * TILE_BYTES);
                    const uint32_t d = tmem_base;                 // one accumulator, as inside a tile of the GEMM
                    tc_mma_mxf8_lo<2, 2>(d, a_lo, b_lo, idesc_mxf8(256, 256, 0), sf, sf + 4, static_cast<uint32_t>(ks + g > 0));
                    tc_mma_mxf8_lo<2, 1>(d, a_lo + 2, b_lo + 2, idesc_mxf8(256, 256, 1), sf, sf + 4);
                    tc_mma_mxf8_lo<2, 1>(d, a_lo + 4, b_lo + 4, idesc_mxf8(256, 256, 2), sf, sf + 4);
                    tc_mma_mxf8_lo<2, 1>(d, a_lo + 6, b_lo + 6, idesc_mxf8(256, 256, 3), sf, sf + 4);
                }
                tc_commit_local<2>(bar);
            }
            // keep at most one group in flight behind the one being issued
            if (ks >= GROUP) {
                if (!__all_sync(0xFFFFFFFFu, mbar_wait(bar, ph, ab, 32))) ok = false;
                ph ^= 1;
            }
        }
        if (ok && k_steps > 0) __all_sync(0xFFFFFFFFu, mbar_wait(bar, ph, ab, 32));
        tc_fence_after();
    }
    __syncwarp();
    tc_fence_before();
    cluster_sync_all();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc<2>(tmem_base, 512);
    }
}

}  // namespace probe
}  // namespace mx8

// Queues one launch of the probe on `stream`: every CTA pair of the device issues k_steps K steps of the GEMM's
// main loop (four K = 32 MMAs of a 256 x 256 tile each).  *flops_out receives the floating-point operations of
// the launch (2 * 256 * 256 * 128 per K step and CTA pair); the caller times the launch with events.
extern "C" int mx8_probe_mma_peak(int k_steps, double* flops_out, void* stream) {
    using namespace mx8;
    if (k_steps <= 0 || k_steps % probe::GROUP) return MX8_ERR_ARG;
    int rc = check_device_sm100();
    if (rc != MX8_OK) return rc;
    int* status = device_status_ptr();
    if (!status) return MX8_ERR_CUDA;
    static std::atomic<bool> configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured[dev & 63].load(std::memory_order_acquire)) {
        cudaError_t e = cudaFuncSetAttribute(probe::mma_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, probe::SMEM);
        if (e != cudaSuccess) {
            note_cuda_error("cudaFuncSetAttribute(mma probe)", cudaGetErrorString(e));
            return MX8_ERR_CUDA;
        }
        configured[dev & 63].store(true, std::memory_order_release);
    }
    const int sms = sm_count();
    if (sms <= 1) return MX8_ERR_CUDA;
    const int grid = sms & ~1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = probe::SMEM;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, probe::mma_peak_kernel, k_steps, status);
    if (e != cudaSuccess) {
        note_cuda_error("mma probe launch", cudaGetErrorString(e));
        return MX8_ERR_CUDA;
    }
    if (flops_out) *flops_out = 2.0 * 256 * 256 * 128 * static_cast<double>(k_steps) * (grid / 2);
    return MX8_OK;
}
