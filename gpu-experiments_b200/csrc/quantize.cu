// MXFP8 quantizer for sm_100a: bf16 [E][M][N] -> E4M3 bytes + one E8M0 scale per 1x32 block,
// row-wise ("normal") and/or transposed, scales written in the tcgen05 scale tile layout.
//
// One persistent CTA per SM.  Warp 0 is the producer: it streams 128x128 bf16 tiles (32 KiB)
// into a ring of shared-memory slots with TMA.  G consumer groups of 128 threads take tiles
// round-robin.  Per tile a group
//   1. reads the tile by rows with 16-byte shared loads (two lanes per 32-element block, one
//      warp shuffle for the block amax), converts, and writes the row-wise bytes straight to
//      global memory as full 128-byte lines (16 bytes per lane);
//   2. reads the tile again by columns (8-byte loads, four columns per lane, warp w owns rows
//      32w..32w+31), releases the slot to the producer, converts in registers;
//   3. stages the transposed bytes in shared memory under the 128-byte TMA swizzle and lets one
//      thread issue four TMA tile stores plus two 512-byte bulk stores for the scale tiles.
// HBM traffic is the algorithmic minimum: 2 bytes read and (1 + 1/32) bytes written per element
// and orientation.  Replaces blackwell-ultra/019-mxfp8-quantize.cu:40-179 and the persistent
// variant blackwell-ultra/020-mxfp8-quantize-persistent.cu:139-219 of the reference.
#include "mx8_host.cuh"
#include "mx8_ptx.cuh"

namespace mx8 {
namespace quant {

constexpr int TILE = 128;
constexpr int SLOT_BYTES = TILE * TILE * 2;       // one bf16 tile
constexpr int TSTAGE_BYTES = TILE * TILE;         // transposed fp8 staging per group
constexpr int SCSTAGE_BYTES = 2 * 1024;           // [parity][row scales 512 | column scales 512]

struct Params {
    uint8_t* out;        // row-wise fp8 [E*M][N]
    uint8_t* sc;         // row-wise scale tiles
    uint8_t* sc_t;       // transposed scale tiles
    int tiles_r;         // E*M/128
    int tiles_c;         // N/128
    int tiles_rm;        // M/128 (row tiles per expert)
    int N;
    int round_add;       // 0x1F: round the scale exponent up (rceil); 0: floor
    int min_byte;        // 88 (rceil: amax/448 clamped to 1e-12) or 0 (floor)
    int* status;
};

template <int G, int S>
struct Smem {
    static constexpr int ring = 0;
    static constexpr int tstage = ring + S * SLOT_BYTES;
    static constexpr int scstage = tstage + G * TSTAGE_BYTES;
    static constexpr int bars = scstage + G * SCSTAGE_BYTES;      // full[S], empty[S]
    static constexpr int flag = bars + 2 * S * 8;
    static constexpr int total = flag + 16;
    static constexpr int dynamic = total + 1024;                  // slack to align the base to 1024
};

__device__ __forceinline__ uint32_t maxabs_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }
__device__ __forceinline__ void group_sync(int g) {
    asm volatile("bar.sync %0, %1;" ::"r"(g + 1), "r"(128) : "memory");
}
// E8M0 byte from the bit pattern of a non-negative bf16 amax; exact integer form of
// ceil(log2(amax/448)) + 127 (round_add = 0x1F) or floor(log2(amax)) - 8 + 127 (round_add = 0).
__device__ __forceinline__ int scale_byte(uint32_t amax_bits, int round_add, int min_byte) {
    return max(min_byte, static_cast<int>((amax_bits + round_add) >> 7) - 8);
}
// 2^(127 - byte) as a float: the exact reciprocal of the scale
__device__ __forceinline__ float inv_scale(int byte) { return __uint_as_float(static_cast<uint32_t>(254 - byte) << 23); }
// four bf16 (two packed words) -> four E4M3 bytes
__device__ __forceinline__ uint32_t cvt4(uint32_t v0, uint32_t v1, float inv) {
    return cvt_e4m3x2(bf16_lo(v0) * inv, bf16_hi(v0) * inv) | (cvt_e4m3x2(bf16_lo(v1) * inv, bf16_hi(v1) * inv) << 16);
}

template <int G, int S, bool ROW, bool COL>
__global__ void __launch_bounds__(32 + G * 128, 1)
quantize_kernel(const __grid_constant__ CUtensorMap tm_in, const __grid_constant__ CUtensorMap tm_t, const Params p) {
    using L = Smem<G, S>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t full0 = base + L::bars;
    const uint32_t empty0 = full0 + S * 8;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + L::flag);
    const AbortCtl ab{abort_flag, p.status};

    const int tid = threadIdx.x;
    if (tid == 0) {
        *abort_flag = 0;
        for (int s = 0; s < S; ++s) {
            mbar_init(full0 + s * 8, 1);
            mbar_init(empty0 + s * 8, 4);      // one elected lane of each of the group's four warps
        }
        fence_mbar_init();
        prefetch_tmap(&tm_in);
        if (COL) prefetch_tmap(&tm_t);
    }
    __syncthreads();

    const int num_tiles = p.tiles_r * p.tiles_c;
    const int first = blockIdx.x;
    const int step = gridDim.x;

    if (tid < 32) {
        // ---------------------------------------------------------------- producer
        if (tid == 0) {
            int n = 0;
            for (int t = first; t < num_tiles; t += step, ++n) {
                const int slot = n % S;
                const uint32_t ph = (n / S) & 1;
                if (!mbar_wait(empty0 + slot * 8, ph ^ 1, ab, DEV_TIMEOUT_EMPTY)) break;
                const int tr = t / p.tiles_c, tc = t - tr * p.tiles_c;
                mbar_arrive_expect_tx(full0 + slot * 8, SLOT_BYTES);
                tma_load_2d(base + L::ring + slot * SLOT_BYTES, &tm_in, tc * TILE, tr * TILE, full0 + slot * 8);
            }
        }
        return;
    }

    // -------------------------------------------------------------------- consumers
    const int ct = tid - 32;
    const int g = ct >> 7;             // group
    const int t128 = ct & 127;         // thread within group
    const int w = t128 >> 5;           // warp within group
    const int l = t128 & 31;
    const uint32_t tstage = base + L::tstage + g * TSTAGE_BYTES;
    const uint32_t scstage = base + L::scstage + g * SCSTAGE_BYTES;
    uint8_t* scstage_ptr = base_ptr + L::scstage + g * SCSTAGE_BYTES;

    int n = g;
    int local = 0;                     // tiles this group has processed (parity of the scale staging)
    for (int t = first + g * step; t < num_tiles; t += G * step, n += G, ++local) {
        const int slot = n % S;
        const uint32_t ph = (n / S) & 1;
        const int tr = t / p.tiles_c, tc = t - tr * p.tiles_c;
        const uint32_t slot_addr = base + L::ring + slot * SLOT_BYTES;
        const int par = local & 1;
        if (!mbar_wait(full0 + slot * 8, ph, ab, DEV_TIMEOUT_FULL)) break;

        if constexpr (ROW) {
            // lane l: row 4j + l/8 of this warp's 32 rows, 16-element segment l%8; the lane pair
            // (l, l^1) shares one 32-element block.  The two 16-byte loads are issued in an order
            // that depends on bit 2 of the lane so a quarter-warp touches all 32 banks.
            const int seg = l & 7;
            const int h0 = (l >> 2) & 1;
            const int kb = seg >> 1;
            uint8_t* out_base = p.out + (static_cast<size_t>(tr) * TILE + w * 32 + (l >> 3)) * p.N + tc * TILE + seg * 16;
#pragma unroll 4
            for (int j = 0; j < 8; ++j) {
                const int r32 = j * 4 + (l >> 3);
                const uint32_t a = slot_addr + (w * 32 + r32) * 256 + seg * 32;
                uint32_t v[8];
                ld_shared_v4(a + h0 * 16, v[0], v[1], v[2], v[3]);
                ld_shared_v4(a + (h0 ^ 1) * 16, v[4], v[5], v[6], v[7]);
                uint32_t m = maxabs_bf16x2(v[0], v[1]);
#pragma unroll
                for (int q = 2; q < 8; ++q) m = maxabs_bf16x2(m, v[q]);
                m &= 0x7FFF7FFFu;
                uint32_t amax = max(m & 0xFFFFu, m >> 16);
                amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
                const int byte = scale_byte(amax, p.round_add, p.min_byte);
                const float inv = inv_scale(byte);
                const uint32_t o0 = cvt4(v[0], v[1], inv), o1 = cvt4(v[2], v[3], inv);
                const uint32_t o2 = cvt4(v[4], v[5], inv), o3 = cvt4(v[6], v[7], inv);
                uint4 o = h0 ? make_uint4(o2, o3, o0, o1) : make_uint4(o0, o1, o2, o3);
                *reinterpret_cast<uint4*>(out_base + static_cast<size_t>(j) * 4 * p.N) = o;
                if ((l & 1) == 0) scstage_ptr[par * 1024 + r32 * 16 + w * 4 + kb] = static_cast<uint8_t>(byte);
            }
        }

        uint32_t c[32][2];
        if constexpr (COL) {
            // lane l: columns 4l..4l+3 of rows 32w..32w+31
#pragma unroll
            for (int i = 0; i < 32; ++i) ld_shared_v2(slot_addr + (w * 32 + i) * 256 + l * 8, c[i][0], c[i][1]);
        }
        __syncwarp();
        if (l == 0) mbar_arrive(empty0 + slot * 8);     // slot may be refilled

        int cb[4];
        float cinv[4];
        if constexpr (COL) {
            uint32_t m0 = maxabs_bf16x2(c[0][0], c[1][0]), m1 = maxabs_bf16x2(c[0][1], c[1][1]);
#pragma unroll
            for (int i = 2; i < 32; ++i) {
                m0 = maxabs_bf16x2(m0, c[i][0]);
                m1 = maxabs_bf16x2(m1, c[i][1]);
            }
            cb[0] = scale_byte(m0 & 0x7FFFu, p.round_add, p.min_byte);
            cb[1] = scale_byte((m0 >> 16) & 0x7FFFu, p.round_add, p.min_byte);
            cb[2] = scale_byte(m1 & 0x7FFFu, p.round_add, p.min_byte);
            cb[3] = scale_byte((m1 >> 16) & 0x7FFFu, p.round_add, p.min_byte);
#pragma unroll
            for (int k = 0; k < 4; ++k) cinv[k] = inv_scale(cb[k]);
        }

        // the stores of this group's previous tile must have finished reading the staging buffers
        if (t128 == 0) bulk_wait_read<0>();
        group_sync(g);

        if constexpr (COL) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                uint32_t wd[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    float f[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const uint32_t v = c[q * 4 + e][k >> 1];
                        f[e] = ((k & 1) ? bf16_hi(v) : bf16_lo(v)) * cinv[k];
                    }
                    wd[q] = cvt_e4m3x2(f[0], f[1]) | (cvt_e4m3x2(f[2], f[3]) << 16);
                }
                // column 4l+k -> staging buffer k, row l; 16-byte chunk index XOR (row & 7)
                const uint32_t rowa = tstage + k * 4096 + l * 128;
                st_shared_v4(rowa + (((w * 2 + 0) ^ (l & 7)) << 4), wd[0], wd[1], wd[2], wd[3]);
                st_shared_v4(rowa + (((w * 2 + 1) ^ (l & 7)) << 4), wd[4], wd[5], wd[6], wd[7]);
                const int col = 4 * l + k;
                scstage_ptr[par * 1024 + 512 + (col & 31) * 16 + (col >> 5) * 4 + w] = static_cast<uint8_t>(cb[k]);
            }
        }
        fence_proxy_async_smem();
        group_sync(g);
        if (t128 == 0) {
            const int e = tr / p.tiles_rm, trm = tr - e * p.tiles_rm;
            if constexpr (COL) {
#pragma unroll
                for (int k = 0; k < 4; ++k) tma_store_4d(&tm_t, trm * TILE, k, tc * 32, e, tstage + k * 4096);
                bulk_store_1d(p.sc_t + ((static_cast<size_t>(e) * p.tiles_c + tc) * p.tiles_rm + trm) * 512,
                              scstage + par * 1024 + 512, 512);
            }
            if constexpr (ROW)
                bulk_store_1d(p.sc + (static_cast<size_t>(tr) * p.tiles_c + tc) * 512, scstage + par * 1024, 512);
            bulk_commit();
        }
    }
    if (t128 == 0) bulk_wait_all<0>();
}

template <int G, int S, bool ROW, bool COL>
static int launch(const CUtensorMap& tm_in, const CUtensorMap& tm_t, const Params& p, int grid, cudaStream_t stream) {
    auto kern = quantize_kernel<G, S, ROW, COL>;
    constexpr int smem = Smem<G, S>::dynamic;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) {
            note_cuda_error("cudaFuncSetAttribute(quantize)", cudaGetErrorString(e));
            return MX8_ERR_CUDA;
        }
        configured[dev & 63] = true;
    }
    kern<<<grid, 32 + G * 128, smem, stream>>>(tm_in, tm_t, p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        note_cuda_error("quantize launch", cudaGetErrorString(e));
        return MX8_ERR_CUDA;
    }
    return MX8_OK;
}

}  // namespace quant
}  // namespace mx8

extern "C" int mx8_quantize(const void* x_bf16, int E, int M, int N, void* fp8, void* sc, void* fp8_t, void* sc_t,
                            int scale_mode, void* stream) {
    using namespace mx8;
    using namespace mx8::quant;
    const bool row = fp8 != nullptr || sc != nullptr;
    const bool col = fp8_t != nullptr || sc_t != nullptr;
    if (!x_bf16 || (!row && !col)) return MX8_ERR_ARG;
    if ((row && (!fp8 || !sc)) || (col && (!fp8_t || !sc_t))) return MX8_ERR_ARG;
    if (scale_mode != MX8_SCALE_RCEIL && scale_mode != MX8_SCALE_FLOOR) return MX8_ERR_ARG;
    if (E <= 0 || M <= 0 || N <= 0 || M % 128 || N % 128) return MX8_ERR_SHAPE;
    if (static_cast<long long>(E) * M > 0x7FFFFFFFll) return MX8_ERR_SHAPE;
    if (!aligned16(x_bf16) || !aligned16(fp8) || !aligned16(sc) || !aligned16(fp8_t) || !aligned16(sc_t)) return MX8_ERR_ALIGN;
    int rc = check_device_sm100();
    if (rc != MX8_OK) return rc;

    Params p{};
    p.out = static_cast<uint8_t*>(fp8);
    p.sc = static_cast<uint8_t*>(sc);
    p.sc_t = static_cast<uint8_t*>(sc_t);
    p.tiles_r = E * (M / 128);
    p.tiles_c = N / 128;
    p.tiles_rm = M / 128;
    p.N = N;
    p.round_add = scale_mode == MX8_SCALE_RCEIL ? 0x1F : 0;
    p.min_byte = scale_mode == MX8_SCALE_RCEIL ? 88 : 0;
    p.status = device_status_ptr();
    if (!p.status) return MX8_ERR_CUDA;

    CUtensorMap tm_in, tm_t;
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(E) * M};
        const uint64_t strides[1] = {static_cast<uint64_t>(N) * 2};
        const uint32_t box[2] = {128, 128};
        rc = make_tmap(&tm_in, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x_bf16, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc != MX8_OK) return rc;
    }
    if (col) {
        // transposed bytes [E][N][M] seen as (M, 4, N/4, E): column c = 4q + k lives at (k, q), so
        // one store covers the 32 columns a staging buffer holds (k fixed, q = 0..31)
        const uint64_t dims[4] = {static_cast<uint64_t>(M), 4, static_cast<uint64_t>(N) / 4, static_cast<uint64_t>(E)};
        const uint64_t strides[3] = {static_cast<uint64_t>(M), static_cast<uint64_t>(M) * 4, static_cast<uint64_t>(M) * N};
        const uint32_t box[4] = {128, 1, 32, 1};
        rc = make_tmap(&tm_t, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, fp8_t, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                       CU_TENSOR_MAP_L2_PROMOTION_NONE);
        if (rc != MX8_OK) return rc;
    } else {
        tm_t = tm_in;
    }

    const int tiles = p.tiles_r * p.tiles_c;
    int grid = sm_count();
    if (grid <= 0) return MX8_ERR_CUDA;
    if (grid > tiles) grid = tiles;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (row && col) return launch<4, 4, true, true>(tm_in, tm_t, p, grid, st);
    if (row) return launch<4, 4, true, false>(tm_in, tm_t, p, grid, st);
    return launch<4, 4, false, true>(tm_in, tm_t, p, grid, st);
}
