// MXFP8 quantizer for sm_100a: bf16 [E][M][N] -> E4M3 bytes + one E8M0 scale per 1x32 block,
// row-wise ("normal") and/or transposed, scales written in the tcgen05 scale tile layout.
//
// One persistent CTA per SM: warp 0 is the producer, W consumer warps work independently (no
// CTA-wide or group barrier anywhere).  The unit of work is a slab of 32 rows x 128 columns
// (8 KiB of bf16); a 128x128 scale tile is four consecutive slabs.  Every consumer warp owns
// one shared-memory slot and one staging buffer:
//   producer  one thread streams slabs into the warps' slots with TMA (slab n -> warp n % W);
//   consumer  1. copies its slab into registers with 32 conflict-free 8-byte shared loads
//                (lane l holds columns 4l..4l+3 of all 32 rows) and hands the slot back at
//                once, so the next load overlaps all of the arithmetic below;
//             2. row-wise: block amax by a packed (two rows per register) butterfly over the
//                eight lanes of a 32-column block, scale bytes with packed integer arithmetic,
//                bf16x2 multiply by the exact power-of-two reciprocal, cvt to E4M3, and one
//                4-byte store per lane and row: 128 contiguous bytes per warp instruction;
//             3. transposed: column amax in registers (no shuffle), convert, stage 4 KiB in
//                shared memory and let one lane issue four TMA tile stores (32 bytes along M
//                for each of 32 columns per store).
// HBM traffic is the algorithmic minimum: 2 bytes read and (1 + 1/32) bytes written per element
// and orientation.  Replaces blackwell-ultra/019-mxfp8-quantize.cu:40-179 and the persistent
// variant blackwell-ultra/020-mxfp8-quantize-persistent.cu:139-219 of the reference.
#include <atomic>
#include <type_traits>

#include "mx8_host.cuh"
#include "mx8_ptx.cuh"
#include "mx8_qmath.cuh"

// Consumer warps (W), ring slots per warp (D) and the row-wise store flavour (RTMA: staged TMA tile store
// instead of one 4-byte global store per lane and row) of the dense quantizer: build-time tunables, set
// from measurements at 16384 x 16384 with the GPU idle before each run (SM clock at its maximum):
//   both orientations  W=8 D=1 per-lane stores 181 us; W=7 or 9 are 2-6 % slower, TMA row stores 4 % slower
//   one orientation    W=7 D=2: row-wise with TMA stores 135 us (per-lane stores 143 us), transposed 132 us
// Under sustained load the SM clock drops under the power cap and the TMA row store wins for both
// orientations as well (185 vs 193 us), which is why the MoE kernels, which run inside long steps, use it.
#ifndef MX8_Q_BOTH_W
#define MX8_Q_BOTH_W 8
#endif
#ifndef MX8_Q_BOTH_D
#define MX8_Q_BOTH_D 1
#endif
#ifndef MX8_Q_BOTH_RTMA
#define MX8_Q_BOTH_RTMA 0
#endif
#ifndef MX8_Q_ONE_W
#define MX8_Q_ONE_W 7
#endif
#ifndef MX8_Q_ONE_D
#define MX8_Q_ONE_D 2
#endif
#ifndef MX8_Q_ONE_RTMA
#define MX8_Q_ONE_RTMA 1
#endif
#ifndef MX8_Q_COL_W
#define MX8_Q_COL_W 7
#endif
#ifndef MX8_Q_COL_D
#define MX8_Q_COL_D 2
#endif
#ifndef MX8_Q_MOE_RTMA
#define MX8_Q_MOE_RTMA 1
#endif
// SwiGLU backward (both gradients): consumer warps and row-store form
#ifndef MX8_Q_SWB_W
#define MX8_Q_SWB_W 8
#endif
#ifndef MX8_Q_SWB_RTMA
#define MX8_Q_SWB_RTMA MX8_Q_MOE_RTMA
#endif

namespace mx8 {
namespace quant {

constexpr int TILE = 128;
constexpr int SLAB_ROWS = 32;
constexpr int SLOT_BYTES = SLAB_ROWS * TILE * 2;   // one bf16 slab (or two E4M3 slabs)
constexpr int TSTAGE_BYTES = SLAB_ROWS * TILE;     // transposed fp8 staging per warp
constexpr int RSTAGE_BYTES = SLAB_ROWS * TILE;     // row-wise fp8 staging per warp
constexpr int SCSTAGE_BYTES = 128;                 // row-wise scale bytes of one slab: [row][kb]

struct Params {
    uint8_t* out;        // row-wise fp8 [E*M][N]
    uint8_t* sc;         // row-wise scale tiles
    uint8_t* sc_t;       // transposed scale tiles
    int tiles_r;         // E*M/128
    int tiles_c;         // N/128
    int tiles_rm;        // M/128 (row tiles per expert)
    int N;
    int group_r;         // tile rows per rasterisation group
    uint32_t round_add2; // packed per 16-bit half: 0x1F rounds the scale exponent up (rceil), 0 = floor
    uint32_t min_byte8_2;// packed per half: smallest scale byte + 8 (rceil 88: amax/448 clamped to 1e-12; floor 0)
    // source modes other than a dense bf16 matrix
    const int* rows_dev;          // device: rows present (gather / SwiGLU); tiles beyond it are skipped
    const int* row_begin_dev;     // device: first row to process (row window of a minibatch), nullptr = 0
    const int* peer_rank;         // gather: source rank per row, -1 = zero row
    const int* peer_token_idx;    // gather: token * topk + k on the source rank
    int topk;
    const uint8_t* src[16];       // gather: every rank's token matrix [tokens][N] bf16 (peer-mapped pointers)
    const uint8_t* gate_sc;       // SwiGLU: scale tiles of the two E4M3 inputs
    const uint8_t* up_sc;
    uint8_t* hidden_bf16;         // SwiGLU: optional bf16 copy of the activation (tests), else nullptr
    int bwd_which;                // SwiGLU backward: 0 = gradient of gate, 1 = gradient of up, 2 = both from one
                                  // pass over the inputs (gate's into out/sc/sc_t, up's into the *2 set)
    uint8_t* out2;                // second output set of bwd_which == 2
    uint8_t* sc2;
    uint8_t* sc_t2;
    uint8_t* hidden_bf16_2;
    int* status;
};

constexpr int SRC_DENSE = 0, SRC_GATHER = 1, SRC_SWIGLU = 2, SRC_SWIGLU_BWD = 3;
// bytes of one ring slot: the backward of SwiGLU also needs the bf16 gradient of the activation
// (and the gather source fetches 512-byte row pieces, two column tiles wide: half as many bulk copies)
__host__ __device__ constexpr int slot_bytes(int src) { return (src == SRC_SWIGLU_BWD || src == SRC_GATHER) ? 2 * SLOT_BYTES : SLOT_BYTES; }
// producer warps: the gather source looks two indices up per row before it can issue a copy, so
// several warps work on different slabs to keep enough copies in flight
__host__ __device__ constexpr int producer_warps(int src) { return src == SRC_GATHER ? 4 : 1; }

template <int W, int D, int SLOT = SLOT_BYTES, bool RTMA = true>
struct Smem {
    static constexpr int S = W * D;                               // slots in the ring
    static constexpr int ring = 0;
    static constexpr int tstage = ring + S * SLOT;
    static constexpr int rstage = tstage + W * TSTAGE_BYTES;
    static constexpr int scstage = rstage + (RTMA ? W * RSTAGE_BYTES : 0);
    static constexpr int bars = scstage + W * SCSTAGE_BYTES;      // full[S], empty[S]
    static constexpr int flag = bars + 2 * S * 8;
    static constexpr int total = flag + 16;
    static constexpr int dynamic = total + 1024;                  // slack to align the base to 1024
    static_assert(dynamic <= 232448, "shared memory budget exceeded");
};

using namespace qmath;

// Tile order: groups of `group_r` tile rows, walked column by column inside a group.  The ~148
// tiles in flight at any time then form a patch about group_r tiles tall, so each input row, each
// row-wise output row AND each transposed output row receives a contiguous run of a kilobyte or
// more within a short time window, which keeps DRAM pages open for all three streams.
__device__ __forceinline__ void tile_coords(int t, const Params& p, int tiles_r, int tiles_c, int& tr, int& tc) {
    const int per_group = p.group_r * tiles_c;
    const int grp = t / per_group;
    const int in_grp = t - grp * per_group;
    const int rows = min(p.group_r, tiles_r - grp * p.group_r);
    tc = in_grp / rows;
    tr = grp * p.group_r + (in_grp - tc * rows);
}

template <int W, int D, int SRC, bool ROW, bool COL, bool RTMA>
__global__ void __launch_bounds__((producer_warps(SRC) + W) * 32, 1)
quantize_kernel(const __grid_constant__ CUtensorMap tm_in, const __grid_constant__ CUtensorMap tm_in2,
                const __grid_constant__ CUtensorMap tm_in3, const __grid_constant__ CUtensorMap tm_t,
                const __grid_constant__ CUtensorMap tm_t2, const __grid_constant__ CUtensorMap tm_r,
                const __grid_constant__ CUtensorMap tm_r2, const Params p) {
    constexpr int SLOT = slot_bytes(SRC);
    using L = Smem<W, D, SLOT, RTMA>;
    constexpr int S = L::S;
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
            mbar_init(full0 + s * 8, SRC == SRC_GATHER ? 32 : 1);   // gather: one arrival per row
            mbar_init(empty0 + s * 8, 1);
        }
        fence_mbar_init();
        prefetch_tmap(&tm_in);
        if (COL) prefetch_tmap(&tm_t);
        if (ROW) prefetch_tmap(&tm_r);
    }
    __syncthreads();

    // this CTA's tiles: blockIdx.x, blockIdx.x + gridDim.x, ...; slab n = 4 * (tile ordinal) + quarter
    // row window: tile rows [tile0, tiles_r_end); tile coordinates are computed inside the window
    const int tile0 = p.row_begin_dev ? *p.row_begin_dev / TILE : 0;
    const int tiles_r_end = p.rows_dev ? min(p.tiles_r, (*p.rows_dev + TILE - 1) / TILE) : p.tiles_r;
    const int tiles_r = max(tiles_r_end - tile0, 0);
    // the gather source walks tiles two columns wide (the odd last column, if any, alone)
    const int tiles_ce = SRC == SRC_GATHER ? (p.tiles_c + 1) / 2 : p.tiles_c;
    const int num_tiles = tiles_r * tiles_ce;
    const int my_tiles = (num_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
    const int my_slabs = my_tiles * 4;

    constexpr int P = producer_warps(SRC);
    if (tid < 32 * P) {
        // ---------------------------------------------------------------- producer
        if constexpr (SRC == SRC_GATHER) {
            // every lane fetches one row of the slot (512 bytes = two column tiles) from the rank that owns
            // the token, straight from that rank's memory; rows without a source are filled with zeros
            const int pw = tid >> 5, pl = tid & 31;              // producer warp pw takes slabs pw, pw + P, ...
            for (int n = pw; n < my_slabs; n += P) {
                const int slot = n % S;
                const uint32_t ph = (n / S) & 1;
                const int t = static_cast<int>(blockIdx.x) + (n >> 2) * static_cast<int>(gridDim.x);
                int tr, tc;
                tile_coords(t, p, tiles_r, tiles_ce, tr, tc);
                tr += tile0;
                const int row = tr * TILE + (n & 3) * SLAB_ROWS + pl;
                const int pr = p.peer_rank[row];                 // issued before the wait: the look-up overlaps it
                const int tok = p.peer_token_idx[row];
                int ok = 1;
                if (pl == 0) ok = mbar_wait(empty0 + slot * 8, ph ^ 1, ab, DEV_TIMEOUT_EMPTY) ? 1 : 0;
                ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
                if (!ok) break;
                // this row's piece: two column tiles (512 bytes), one if the row of tiles ends here
                const uint32_t dst = base + L::ring + slot * SLOT + pl * 512;
                const uint32_t piece = (2 * tc + 1 < p.tiles_c) ? 512u : 256u;
                if (pr >= 0) {
                    const uint8_t* s = p.src[pr] + (static_cast<size_t>(tok / p.topk) * p.N + 2 * tc * TILE) * 2;
                    mbar_arrive_expect_tx(full0 + slot * 8, piece);
                    bulk_load_1d(dst, s, piece, full0 + slot * 8);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) st_shared_v4(dst + j * 16, 0, 0, 0, 0);
                    mbar_arrive(full0 + slot * 8);
                }
            }
        } else if (tid == 0) {
            for (int n = 0; n < my_slabs; ++n) {
                const int slot = n % S;
                const uint32_t ph = (n / S) & 1;
                if (!mbar_wait(empty0 + slot * 8, ph ^ 1, ab, DEV_TIMEOUT_EMPTY)) break;
                const int t = static_cast<int>(blockIdx.x) + (n >> 2) * static_cast<int>(gridDim.x);
                int tr, tc;
                tile_coords(t, p, tiles_r, tiles_ce, tr, tc);
                tr += tile0;
                const uint32_t dst = base + L::ring + slot * SLOT;
                mbar_arrive_expect_tx(full0 + slot * 8, SLOT);
                if constexpr (SRC == SRC_SWIGLU || SRC == SRC_SWIGLU_BWD) {
                    // two E4M3 slabs of 32 x 128 bytes: gate, then up
                    tma_load_2d(dst, &tm_in, tc * TILE, tr * TILE + (n & 3) * SLAB_ROWS, full0 + slot * 8);
                    tma_load_2d(dst + SLOT_BYTES / 2, &tm_in2, tc * TILE, tr * TILE + (n & 3) * SLAB_ROWS, full0 + slot * 8);
                    if constexpr (SRC == SRC_SWIGLU_BWD)   // bf16 gradient of the activation
                        tma_load_2d(dst + SLOT_BYTES, &tm_in3, tc * TILE, tr * TILE + (n & 3) * SLAB_ROWS, full0 + slot * 8);
                } else {
                    tma_load_2d(dst, &tm_in, tc * TILE, tr * TILE + (n & 3) * SLAB_ROWS, full0 + slot * 8);
                }
            }
        }
        return;
    }

    // -------------------------------------------------------------------- consumer warp
    const int w = (tid >> 5) - P;
    const int l = tid & 31;
    const uint32_t tstage = base + L::tstage + w * TSTAGE_BYTES;
    const uint32_t rstage = base + L::rstage + w * RSTAGE_BYTES;
    uint8_t* scstage_ptr = base_ptr + L::scstage + w * SCSTAGE_BYTES;
    const int hswap = (l >> 2) & 1;     // staging stores: which 16-byte half goes first (bank spreading)

    for (int n = w; n < my_slabs; n += W) {
        // slab n lives in slot n % S; S is a multiple of W, so a slot is only ever read by one warp
        const int slot = n % S;
        const uint32_t ph = (n / S) & 1;
        const uint32_t slot_addr = base + L::ring + slot * SLOT;
        const int wq = n & 3;
        const int t = static_cast<int>(blockIdx.x) + (n >> 2) * static_cast<int>(gridDim.x);
        int tr, tc;
        tile_coords(t, p, tiles_r, tiles_ce, tr, tc);
                tr += tile0;
        if (!mbar_wait(full0 + slot * 8, ph, ab, DEV_TIMEOUT_FULL)) break;

        // SwiGLU backward can emit both gradients from one visit of the slot: two passes over the same
        // shared-memory inputs, each quantizing into its own output set
        // The gather source visits a slot twice as well: its two 128-column halves are two tiles.
        const int pass_first = (SRC == SRC_SWIGLU_BWD && p.bwd_which != 2) ? p.bwd_which : 0;
        const int pass_last = SRC == SRC_SWIGLU_BWD ? (p.bwd_which == 2 ? 1 : p.bwd_which)
                            : (SRC == SRC_GATHER ? ((2 * tc + 1 < p.tiles_c) ? 1 : 0) : 0);
        const int tc_pair = tc;
#pragma unroll 1
        for (int pass = pass_first; pass <= pass_last; ++pass) {
        const bool second = SRC == SRC_SWIGLU_BWD && p.bwd_which == 2 && pass == 1;
        uint8_t* const o_out = second ? p.out2 : p.out;
        uint8_t* const o_sc = second ? p.sc2 : p.sc;
        uint8_t* const o_sc_t = second ? p.sc_t2 : p.sc_t;
        uint8_t* const o_bf16 = second ? p.hidden_bf16_2 : p.hidden_bf16;
        const CUtensorMap* const o_tm_t = second ? &tm_t2 : &tm_t;
        const CUtensorMap* const o_tm_r = second ? &tm_r2 : &tm_r;
        if constexpr (SRC == SRC_GATHER) tc = 2 * tc_pair + pass;
        uint32_t c[32][2];                 // c[i] = columns 4l..4l+3 of slab row i (bf16 pairs)
        if constexpr (SRC == SRC_SWIGLU || SRC == SRC_SWIGLU_BWD) {
            // forward: hidden = bf16( silu(dequant(gate)) * dequant(up) ), computed in fp32;
            // backward: d_gate = bf16( (silu'(g) * u) * d_hidden ) or d_up = bf16( silu(g) * d_hidden )
            const size_t sc_tile = (static_cast<size_t>(tr) * p.tiles_c + tc) * 512 + l * 16 + wq * 4;
            const uint32_t gw = *reinterpret_cast<const uint32_t*>(p.gate_sc + sc_tile);   // lane i: scale bytes of row i
            const uint32_t uw = *reinterpret_cast<const uint32_t*>(p.up_sc + sc_tile);
            const int sh = (l >> 3) * 8;                                                 // this lane's 32-column block
            // The loop body is compiled once per mode.  MODE 0: forward, or d_gate alone.  MODE 1: d_up alone, which
            // needs neither the up projection nor the derivative of silu.  MODE 2 (both gradients from one visit of
            // the slot): d_gate, and d_up = bf16(silu(g) * d_hidden) of the same elements written over the lane's own
            // d_hidden words in the slot, so that the second pass only loads them.
            auto rows = [&](auto mode) {
                constexpr int MODE = decltype(mode)::value;
                constexpr bool D_UP = MODE == 1;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    uint32_t g4, u4 = 0;
                    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(g4) : "r"(slot_addr + i * 128 + l * 4));
                    if constexpr (!D_UP) asm volatile("ld.shared.b32 %0, [%1];" : "=r"(u4) : "r"(slot_addr + SLOT_BYTES / 2 + i * 128 + l * 4));
                    const float gs = __uint_as_float(((__shfl_sync(0xFFFFFFFFu, gw, i) >> sh) & 0xFFu) << 23);
                    float us = 0.0f;
                    if constexpr (!D_UP) us = __uint_as_float(((__shfl_sync(0xFFFFFFFFu, uw, i) >> sh) & 0xFFu) << 23);
                    float gf[4], uf[4] = {0.0f, 0.0f, 0.0f, 0.0f}, h[4];
                    [[maybe_unused]] float h_up[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    e4m3x4_to_float(g4, gf);
                    if constexpr (!D_UP) e4m3x4_to_float(u4, uf);
                    [[maybe_unused]] float dh[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    if constexpr (SRC == SRC_SWIGLU_BWD) {
                        uint32_t d0, d1;
                        ld_shared_v2(slot_addr + SLOT_BYTES + i * 256 + l * 8, d0, d1);
                        dh[0] = bf16_lo(d0); dh[1] = bf16_hi(d0); dh[2] = bf16_lo(d1); dh[3] = bf16_hi(d1);
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float g = gf[e] * gs;
                        if constexpr (SRC == SRC_SWIGLU_BWD) {
                            const float sig = __fdividef(1.0f, 1.0f + __expf(-g));
                            const float silu = g * sig;
                            if constexpr (D_UP) {
                                h[e] = silu * dh[e];
                            } else {
                                const float dsilu = (1.0f - silu) * sig + silu;
                                h[e] = (dsilu * (uf[e] * us)) * dh[e];
                                if constexpr (MODE == 2) h_up[e] = silu * dh[e];
                            }
                        } else {
                            h[e] = __fdividef(g, 1.0f + __expf(-g)) * (uf[e] * us);
                        }
                    }
                    c[i][0] = pack_bf16x2(h[0], h[1]);
                    c[i][1] = pack_bf16x2(h[2], h[3]);
                    if constexpr (MODE == 2)
                        st_shared_v2(slot_addr + SLOT_BYTES + i * 256 + l * 8, pack_bf16x2(h_up[0], h_up[1]), pack_bf16x2(h_up[2], h_up[3]));
                }
            };
            if constexpr (SRC == SRC_SWIGLU_BWD) {
                if (p.bwd_which == 2) {
                    if (pass == 0) {
                        rows(std::integral_constant<int, 2>{});
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) ld_shared_v2(slot_addr + SLOT_BYTES + i * 256 + l * 8, c[i][0], c[i][1]);
                        // the slot was written through the generic proxy and is refilled through the async proxy next
                        fence_proxy_async_smem();
                    }
                } else if (pass) {
                    rows(std::integral_constant<int, 1>{});
                } else {
                    rows(std::integral_constant<int, 0>{});
                }
            } else {
                rows(std::integral_constant<int, 0>{});
            }
            if (o_bf16) {
                uint8_t* hb = o_bf16 + ((static_cast<size_t>(tr) * TILE + wq * SLAB_ROWS) * p.N + tc * TILE + l * 4) * 2;
#pragma unroll
                for (int i = 0; i < 32; ++i) *reinterpret_cast<uint2*>(hb + static_cast<size_t>(i) * p.N * 2) = make_uint2(c[i][0], c[i][1]);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                if constexpr (SRC == SRC_GATHER) ld_shared_v2(slot_addr + i * 512 + pass * 256 + l * 8, c[i][0], c[i][1]);
                else ld_shared_v2(slot_addr + i * 256 + l * 8, c[i][0], c[i][1]);
            }
        }
        __syncwarp();
        if (l == 0 && pass == pass_last) mbar_arrive(empty0 + slot * 8);       // the slot may be refilled now

        // the previous slab's tile stores must have finished reading the staging buffers
        if ((COL || RTMA) && l == 0) bulk_wait_read<0>();
        __syncwarp();

        if constexpr (ROW) {
            // RTMA: the E4M3 bytes of the slab are staged as 32 rows of 128 bytes (one conflict-free row per warp
            // instruction) and leave with one TMA tile store; otherwise every lane stores its 4 bytes of a row
            // directly (128 contiguous bytes per warp instruction).  Which is faster depends on what else the
            // memory system is doing; the launchers choose per use from measurements.
            uint8_t* out_row = o_out + (static_cast<size_t>(tr) * TILE + wq * SLAB_ROWS) * p.N + tc * TILE + l * 4;
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                // block amax of rows i and i+1 (one per 16-bit half) over the 8 lanes of a 32-column block
                const uint32_t m0 = maxabs_bf16x2(c[i][0], c[i][1]);
                const uint32_t m1 = maxabs_bf16x2(c[i + 1][0], c[i + 1][1]);
                uint32_t a2 = maxabs_bf16x2(__byte_perm(m0, m1, 0x5410), __byte_perm(m0, m1, 0x7632));
                a2 = maxabs_bf16x2(a2, __shfl_xor_sync(0xFFFFFFFFu, a2, 1));
                a2 = maxabs_bf16x2(a2, __shfl_xor_sync(0xFFFFFFFFu, a2, 2));
                a2 = maxabs_bf16x2(a2, __shfl_xor_sync(0xFFFFFFFFu, a2, 4));
                const uint32_t b2 = scale_bytes2(a2 & 0x7FFF7FFFu, p.round_add2, p.min_byte8_2);
                const uint32_t inv2 = inv_scales2(b2);
                const uint32_t inv_a = __byte_perm(inv2, inv2, 0x1010), inv_b = __byte_perm(inv2, inv2, 0x3232);
                const uint32_t qa = cvt4(mul_bf16x2(c[i][0], inv_a), mul_bf16x2(c[i][1], inv_a));
                const uint32_t qb = cvt4(mul_bf16x2(c[i + 1][0], inv_b), mul_bf16x2(c[i + 1][1], inv_b));
                if constexpr (RTMA) {
                    asm volatile("st.shared.b32 [%0], %1;" ::"r"(rstage + i * 128 + l * 4), "r"(qa) : "memory");
                    asm volatile("st.shared.b32 [%0], %1;" ::"r"(rstage + (i + 1) * 128 + l * 4), "r"(qb) : "memory");
                } else {
                    // streaming stores: the bytes are not read again by this kernel
                    __stcs(reinterpret_cast<uint32_t*>(out_row + static_cast<size_t>(i) * p.N), qa);
                    __stcs(reinterpret_cast<uint32_t*>(out_row + static_cast<size_t>(i + 1) * p.N), qb);
                }
                if ((l & 7) == 0) {
                    scstage_ptr[i * 4 + (l >> 3)] = static_cast<uint8_t>(b2);
                    scstage_ptr[(i + 1) * 4 + (l >> 3)] = static_cast<uint8_t>(b2 >> 16);
                }
            }
            if constexpr (RTMA) fence_proxy_async_smem();
            __syncwarp();
            if (RTMA && l == 0) {
                tma_store_2d(o_tm_r, tc * TILE, tr * TILE + wq * SLAB_ROWS, rstage);
                if (!COL) bulk_commit();
            }
            // row r of the tile keeps its four scale bytes at (r % 32) * 16 + (r / 32) * 4
            const uint32_t word = *reinterpret_cast<const uint32_t*>(scstage_ptr + l * 4);
            *reinterpret_cast<uint32_t*>(o_sc + (static_cast<size_t>(tr) * p.tiles_c + tc) * 512 + l * 16 + wq * 4) = word;
            __syncwarp();
        }

        if constexpr (COL) {
            uint32_t m0 = maxabs_bf16x2(c[0][0], c[1][0]), m1 = maxabs_bf16x2(c[0][1], c[1][1]);
#pragma unroll
            for (int i = 2; i < 32; ++i) {
                m0 = maxabs_bf16x2(m0, c[i][0]);
                m1 = maxabs_bf16x2(m1, c[i][1]);
            }
            const uint32_t b01 = scale_bytes2(m0 & 0x7FFF7FFFu, p.round_add2, p.min_byte8_2), b23 = scale_bytes2(m1 & 0x7FFF7FFFu, p.round_add2, p.min_byte8_2);
            const uint32_t inv01 = inv_scales2(b01), inv23 = inv_scales2(b23);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                c[i][0] = mul_bf16x2(c[i][0], inv01);
                c[i][1] = mul_bf16x2(c[i][1], inv23);
            }
            const int e = tr / p.tiles_rm, trm = tr - e * p.tiles_rm;
            uint8_t* sct = o_sc_t + ((static_cast<size_t>(e) * p.tiles_c + tc) * p.tiles_rm + trm) * 512 + wq;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                uint32_t wd[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    float f[4];
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const uint32_t v = c[q * 4 + r][k >> 1];
                        f[r] = (k & 1) ? bf16_hi(v) : bf16_lo(v);
                    }
                    wd[q] = cvt_e4m3x2(f[0], f[1]) | (cvt_e4m3x2(f[2], f[3]) << 16);
                }
                // column 4l+k -> staging buffer k, 32-byte row l (32 bytes = this slab's 32 rows)
                const uint32_t rowa = tstage + k * 1024 + l * 32;
                if (hswap) {
                    st_shared_v4(rowa + 16, wd[4], wd[5], wd[6], wd[7]);
                    st_shared_v4(rowa, wd[0], wd[1], wd[2], wd[3]);
                } else {
                    st_shared_v4(rowa, wd[0], wd[1], wd[2], wd[3]);
                    st_shared_v4(rowa + 16, wd[4], wd[5], wd[6], wd[7]);
                }
                const int col = 4 * l + k;
                const uint32_t bk = ((k >> 1) ? b23 : b01) >> ((k & 1) * 16);
                sct[(col & 31) * 16 + (col >> 5) * 4] = static_cast<uint8_t>(bk);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (l == 0) {
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    tma_store_4d(o_tm_t, trm * TILE + wq * SLAB_ROWS, k, tc * 32, e, tstage + k * 1024);
                bulk_commit();
            }
        }
        }   // pass
    }
    if ((COL || RTMA) && l == 0) bulk_wait_all<0>();
}

template <int W, int D, int SRC, bool ROW, bool COL, bool RTMA = true>
static int launch(const CUtensorMap& tm_in, const CUtensorMap& tm_in2, const CUtensorMap& tm_in3, const CUtensorMap& tm_t,
                  const CUtensorMap& tm_r, const Params& p, int grid, cudaStream_t stream, const CUtensorMap* tm_t2 = nullptr,
                  const CUtensorMap* tm_r2 = nullptr) {
    auto kern = quantize_kernel<W, D, SRC, ROW, COL, RTMA>;
    constexpr int smem = Smem<W, D, slot_bytes(SRC), RTMA>::dynamic;
    static std::atomic<bool> configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured[dev & 63].load(std::memory_order_acquire)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) {
            note_cuda_error("cudaFuncSetAttribute(quantize)", cudaGetErrorString(e));
            return MX8_ERR_CUDA;
        }
        configured[dev & 63].store(true, std::memory_order_release);
    }
    kern<<<grid, (producer_warps(SRC) + W) * 32, smem, stream>>>(tm_in, tm_in2, tm_in3, tm_t, tm_t2 ? *tm_t2 : tm_t, tm_r,
                                                                 tm_r2 ? *tm_r2 : tm_r, p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        note_cuda_error("quantize launch", cudaGetErrorString(e));
        return MX8_ERR_CUDA;
    }
    return MX8_OK;
}

}  // namespace quant
}  // namespace mx8

namespace mx8 {
namespace quant {
static int make_transposed_map(CUtensorMap* tm, void* fp8_t, int E, int M, int N);
static int make_row_map(CUtensorMap* tm, void* fp8, long long rows, int N);
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
    p.group_r = 8;
    p.round_add2 = scale_mode == MX8_SCALE_RCEIL ? RCEIL_ROUND_ADD2 : FLOOR_ROUND_ADD2;
    p.min_byte8_2 = scale_mode == MX8_SCALE_RCEIL ? RCEIL_MIN_BYTE8_2 : FLOOR_MIN_BYTE8_2;
    p.status = device_status_ptr();
    if (!p.status) return MX8_ERR_CUDA;

    CUtensorMap tm_in, tm_t;
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(E) * M};
        const uint64_t strides[1] = {static_cast<uint64_t>(N) * 2};
        const uint32_t box[2] = {128, SLAB_ROWS};
        rc = make_tmap(&tm_in, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x_bf16, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc != MX8_OK) return rc;
    }
    CUtensorMap tm_r;
    if (col) {
        if ((rc = make_transposed_map(&tm_t, fp8_t, E, M, N)) != MX8_OK) return rc;
    } else {
        tm_t = tm_in;
    }
    if (row) {
        if ((rc = make_row_map(&tm_r, fp8, static_cast<long long>(E) * M, N)) != MX8_OK) return rc;
    } else {
        tm_r = tm_in;
    }

    const int tiles = p.tiles_r * p.tiles_c;
    int grid = sm_count();
    if (grid <= 0) return MX8_ERR_CUDA;
    if (grid > tiles) grid = tiles;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // Both orientations: 8 consumer warps with one slot each measured best (deeper prefetch lowers
    // throughput once reads and both write streams compete); a single orientation does less
    // arithmetic per slab and prefers 7 warps with two slots each.
    if (row && col) return launch<MX8_Q_BOTH_W, MX8_Q_BOTH_D, SRC_DENSE, true, true, (MX8_Q_BOTH_RTMA != 0)>(tm_in, tm_in, tm_in, tm_t, tm_r, p, grid, st);
    if (row) return launch<MX8_Q_ONE_W, MX8_Q_ONE_D, SRC_DENSE, true, false, (MX8_Q_ONE_RTMA != 0)>(tm_in, tm_in, tm_in, tm_t, tm_r, p, grid, st);
    return launch<MX8_Q_COL_W, MX8_Q_COL_D, SRC_DENSE, false, true, false>(tm_in, tm_in, tm_in, tm_t, tm_r, p, grid, st);
}

namespace mx8 {
namespace quant {

// transposed bytes [E][N][M] seen as (M, 4, N/4, E): column c = 4q + k lives at (k, q), so one store
// covers the 32 columns a staging buffer holds (k fixed, q = 0..31), 32 bytes each
static int make_transposed_map(CUtensorMap* tm, void* fp8_t, int E, int M, int N) {
    const uint64_t dims[4] = {static_cast<uint64_t>(M), 4, static_cast<uint64_t>(N) / 4, static_cast<uint64_t>(E)};
    const uint64_t strides[3] = {static_cast<uint64_t>(M), static_cast<uint64_t>(M) * 4, static_cast<uint64_t>(M) * N};
    const uint32_t box[4] = {SLAB_ROWS, 1, 32, 1};
    return make_tmap(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, fp8_t, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE,
                     CU_TENSOR_MAP_L2_PROMOTION_NONE);
}

// row-wise bytes [rows][N]: a slab leaves as one store of 32 rows of 128 bytes
static int make_row_map(CUtensorMap* tm, void* fp8, long long rows, int N) {
    const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(rows)};
    const uint64_t strides[1] = {static_cast<uint64_t>(N)};
    const uint32_t box[2] = {TILE, SLAB_ROWS};
    return make_tmap(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, fp8, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE,
                     CU_TENSOR_MAP_L2_PROMOTION_NONE);
}

static void fill_common(Params& p, void* fp8, void* sc, void* sc_t, int rows, int N) {
    p.out = static_cast<uint8_t*>(fp8);
    p.sc = static_cast<uint8_t*>(sc);
    p.sc_t = static_cast<uint8_t*>(sc_t);
    p.tiles_r = rows / 128;
    p.tiles_c = N / 128;
    p.tiles_rm = rows / 128;
    p.N = N;
    p.group_r = 8;
    p.round_add2 = RCEIL_ROUND_ADD2;
    p.min_byte8_2 = RCEIL_MIN_BYTE8_2;
}

// row window of a minibatch: rows [*row_begin, *row_end) on at most max_sms multiprocessors
static void apply_window(Params& p, int& grid, const mx8_window* w) {
    if (!w) return;
    if (w->row_begin) p.row_begin_dev = static_cast<const int*>(w->row_begin);
    if (w->row_end) p.rows_dev = static_cast<const int*>(w->row_end);
    if (w->max_sms > 0 && w->max_sms < grid) grid = w->max_sms;
}

}  // namespace quant
}  // namespace mx8

extern "C" int mx8_moe_dispatch_quantize(const void* const* x_ptrs, int world, int hidden, int topk, const void* peer_rank,
                                         const void* peer_token_idx, const void* num_tokens, int capacity, void* fp8,
                                         void* sc, void* fp8_t, void* sc_t, void* stream) {
    return mx8_moe_dispatch_quantize_window(x_ptrs, world, hidden, topk, peer_rank, peer_token_idx, num_tokens, capacity, fp8, sc,
                                            fp8_t, sc_t, nullptr, stream);
}

extern "C" int mx8_moe_dispatch_quantize_window(const void* const* x_ptrs, int world, int hidden, int topk, const void* peer_rank,
                                         const void* peer_token_idx, const void* num_tokens, int capacity, void* fp8,
                                         void* sc, void* fp8_t, void* sc_t, const mx8_window* window, void* stream) {
    using namespace mx8;
    using namespace mx8::quant;
    if (!x_ptrs || !peer_rank || !peer_token_idx || !num_tokens || !fp8 || !sc || !fp8_t || !sc_t) return MX8_ERR_ARG;
    if (world <= 0 || world > 16 || topk <= 0) return MX8_ERR_ARG;
    if (capacity <= 0 || hidden <= 0 || capacity % 128 || hidden % 128) return MX8_ERR_SHAPE;
    if (!aligned16(fp8) || !aligned16(sc) || !aligned16(fp8_t) || !aligned16(sc_t)) return MX8_ERR_ALIGN;
    for (int r = 0; r < world; ++r)
        if (!x_ptrs[r] || !aligned16(x_ptrs[r])) return MX8_ERR_ALIGN;
    int rc = check_device_sm100();
    if (rc != MX8_OK) return rc;
    Params p{};
    fill_common(p, fp8, sc, sc_t, capacity, hidden);
    p.rows_dev = static_cast<const int*>(num_tokens);
    p.peer_rank = static_cast<const int*>(peer_rank);
    p.peer_token_idx = static_cast<const int*>(peer_token_idx);
    p.topk = topk;
    for (int r = 0; r < world; ++r) p.src[r] = static_cast<const uint8_t*>(x_ptrs[r]);
    p.status = device_status_ptr();
    if (!p.status) return MX8_ERR_CUDA;
    CUtensorMap tm_t, tm_r;
    if ((rc = make_transposed_map(&tm_t, fp8_t, 1, capacity, hidden)) != MX8_OK) return rc;
    if ((rc = make_row_map(&tm_r, fp8, capacity, hidden)) != MX8_OK) return rc;
    int grid = sm_count();
    if (grid <= 0) return MX8_ERR_CUDA;
    const int tiles = p.tiles_r * ((p.tiles_c + 1) / 2);       // slots are two column tiles wide
    if (grid > tiles) grid = tiles;
    apply_window(p, grid, window);
    return launch<8, 1, SRC_GATHER, true, true, (MX8_Q_MOE_RTMA != 0)>(tm_t, tm_t, tm_t, tm_t, tm_r, p, grid, static_cast<cudaStream_t>(stream));
}

extern "C" int mx8_swiglu_quantize(const void* gate_fp8, const void* gate_sc, const void* up_fp8, const void* up_sc,
                                   int rows, int cols, const void* num_rows, void* hidden_fp8, void* hidden_sc,
                                   void* hidden_fp8_t, void* hidden_sc_t, void* hidden_bf16, void* stream) {
    return mx8_swiglu_quantize_window(gate_fp8, gate_sc, up_fp8, up_sc, rows, cols, num_rows, hidden_fp8, hidden_sc, hidden_fp8_t,
                                      hidden_sc_t, hidden_bf16, nullptr, stream);
}

extern "C" int mx8_swiglu_quantize_window(const void* gate_fp8, const void* gate_sc, const void* up_fp8, const void* up_sc,
                                          int rows, int cols, const void* num_rows, void* hidden_fp8, void* hidden_sc,
                                          void* hidden_fp8_t, void* hidden_sc_t, void* hidden_bf16, const mx8_window* window,
                                          void* stream) {
    using namespace mx8;
    using namespace mx8::quant;
    if (!gate_fp8 || !gate_sc || !up_fp8 || !up_sc || !hidden_fp8 || !hidden_sc || !hidden_fp8_t || !hidden_sc_t) return MX8_ERR_ARG;
    if (rows <= 0 || cols <= 0 || rows % 128 || cols % 128) return MX8_ERR_SHAPE;
    if (!aligned16(gate_fp8) || !aligned16(gate_sc) || !aligned16(up_fp8) || !aligned16(up_sc) || !aligned16(hidden_fp8) ||
        !aligned16(hidden_sc) || !aligned16(hidden_fp8_t) || !aligned16(hidden_sc_t) || !aligned16(hidden_bf16))
        return MX8_ERR_ALIGN;
    int rc = check_device_sm100();
    if (rc != MX8_OK) return rc;
    Params p{};
    fill_common(p, hidden_fp8, hidden_sc, hidden_sc_t, rows, cols);
    p.rows_dev = static_cast<const int*>(num_rows);
    p.gate_sc = static_cast<const uint8_t*>(gate_sc);
    p.up_sc = static_cast<const uint8_t*>(up_sc);
    p.hidden_bf16 = static_cast<uint8_t*>(hidden_bf16);
    p.status = device_status_ptr();
    if (!p.status) return MX8_ERR_CUDA;
    CUtensorMap tm_g, tm_u, tm_t;
    const uint64_t dims[2] = {static_cast<uint64_t>(cols), static_cast<uint64_t>(rows)};
    const uint64_t strides[1] = {static_cast<uint64_t>(cols)};
    const uint32_t box[2] = {128, SLAB_ROWS};
    if ((rc = make_tmap(&tm_g, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, gate_fp8, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE)) != MX8_OK) return rc;
    if ((rc = make_tmap(&tm_u, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, up_fp8, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE)) != MX8_OK) return rc;
    if ((rc = make_transposed_map(&tm_t, hidden_fp8_t, 1, rows, cols)) != MX8_OK) return rc;
    CUtensorMap tm_r;
    if ((rc = make_row_map(&tm_r, hidden_fp8, rows, cols)) != MX8_OK) return rc;
    int grid = sm_count();
    if (grid <= 0) return MX8_ERR_CUDA;
    const int tiles = p.tiles_r * p.tiles_c;
    if (grid > tiles) grid = tiles;
    apply_window(p, grid, window);
    return launch<8, 1, SRC_SWIGLU, true, true, (MX8_Q_MOE_RTMA != 0)>(tm_g, tm_u, tm_u, tm_t, tm_r, p, grid, static_cast<cudaStream_t>(stream));
}

extern "C" int mx8_swiglu_bwd_quantize(const void* gate_fp8, const void* gate_sc, const void* up_fp8, const void* up_sc,
                                       const void* d_hidden, int rows, int cols, const void* num_rows, int which, void* out_fp8,
                                       void* out_sc, void* out_fp8_t, void* out_sc_t, void* out_bf16, void* stream) {
    using namespace mx8;
    using namespace mx8::quant;
    if (!gate_fp8 || !gate_sc || !up_fp8 || !up_sc || !d_hidden || !out_fp8 || !out_sc || !out_fp8_t || !out_sc_t) return MX8_ERR_ARG;
    if (which != 0 && which != 1) return MX8_ERR_ARG;
    if (rows <= 0 || cols <= 0 || rows % 128 || cols % 128) return MX8_ERR_SHAPE;
    if (!aligned16(gate_fp8) || !aligned16(gate_sc) || !aligned16(up_fp8) || !aligned16(up_sc) || !aligned16(d_hidden) ||
        !aligned16(out_fp8) || !aligned16(out_sc) || !aligned16(out_fp8_t) || !aligned16(out_sc_t) || !aligned16(out_bf16))
        return MX8_ERR_ALIGN;
    int rc = check_device_sm100();
    if (rc != MX8_OK) return rc;
    Params p{};
    fill_common(p, out_fp8, out_sc, out_sc_t, rows, cols);
    p.rows_dev = static_cast<const int*>(num_rows);
    p.gate_sc = static_cast<const uint8_t*>(gate_sc);
    p.up_sc = static_cast<const uint8_t*>(up_sc);
    p.hidden_bf16 = static_cast<uint8_t*>(out_bf16);
    p.bwd_which = which;
    p.status = device_status_ptr();
    if (!p.status) return MX8_ERR_CUDA;
    CUtensorMap tm_g, tm_u, tm_d, tm_t;
    const uint64_t dims[2] = {static_cast<uint64_t>(cols), static_cast<uint64_t>(rows)};
    const uint64_t strides[1] = {static_cast<uint64_t>(cols)};
    const uint64_t strides2[1] = {static_cast<uint64_t>(cols) * 2};
    const uint32_t box[2] = {128, SLAB_ROWS};
    if ((rc = make_tmap(&tm_g, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, gate_fp8, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE)) != MX8_OK) return rc;
    if ((rc = make_tmap(&tm_u, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, up_fp8, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE)) != MX8_OK) return rc;
    if ((rc = make_tmap(&tm_d, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, d_hidden, dims, strides2, box, CU_TENSOR_MAP_SWIZZLE_NONE)) != MX8_OK) return rc;
    if ((rc = make_transposed_map(&tm_t, out_fp8_t, 1, rows, cols)) != MX8_OK) return rc;
    CUtensorMap tm_r;
    if ((rc = make_row_map(&tm_r, out_fp8, rows, cols)) != MX8_OK) return rc;
    int grid = sm_count();
    if (grid <= 0) return MX8_ERR_CUDA;
    const int tiles = p.tiles_r * p.tiles_c;
    if (grid > tiles) grid = tiles;
    return launch<8, 1, SRC_SWIGLU_BWD, true, true, (MX8_Q_MOE_RTMA != 0)>(tm_g, tm_u, tm_d, tm_t, tm_r, p, grid, static_cast<cudaStream_t>(stream));
}

// Both gradients from one pass over gate, up and d_hidden (each input is read once instead of twice).
extern "C" int mx8_swiglu_bwd_quantize_both(const void* gate_fp8, const void* gate_sc, const void* up_fp8, const void* up_sc,
                                            const void* d_hidden, int rows, int cols, const void* num_rows,
                                            void* d_gate_fp8, void* d_gate_sc, void* d_gate_fp8_t, void* d_gate_sc_t,
                                            void* d_up_fp8, void* d_up_sc, void* d_up_fp8_t, void* d_up_sc_t, void* stream) {
    return mx8_swiglu_bwd_quantize_both_window(gate_fp8, gate_sc, up_fp8, up_sc, d_hidden, rows, cols, num_rows, d_gate_fp8, d_gate_sc,
                                               d_gate_fp8_t, d_gate_sc_t, d_up_fp8, d_up_sc, d_up_fp8_t, d_up_sc_t, nullptr, stream);
}

extern "C" int mx8_swiglu_bwd_quantize_both_window(const void* gate_fp8, const void* gate_sc, const void* up_fp8, const void* up_sc,
                                                   const void* d_hidden, int rows, int cols, const void* num_rows,
                                                   void* d_gate_fp8, void* d_gate_sc, void* d_gate_fp8_t, void* d_gate_sc_t,
                                                   void* d_up_fp8, void* d_up_sc, void* d_up_fp8_t, void* d_up_sc_t,
                                                   const mx8_window* window, void* stream) {
    using namespace mx8;
    using namespace mx8::quant;
    const void* const all[] = {gate_fp8, gate_sc, up_fp8, up_sc, d_hidden, d_gate_fp8, d_gate_sc, d_gate_fp8_t, d_gate_sc_t,
                               d_up_fp8, d_up_sc, d_up_fp8_t, d_up_sc_t};
    for (const void* q : all) {
        if (!q) return MX8_ERR_ARG;
        if (!aligned16(q)) return MX8_ERR_ALIGN;
    }
    if (rows <= 0 || cols <= 0 || rows % 128 || cols % 128) return MX8_ERR_SHAPE;
    int rc = check_device_sm100();
    if (rc != MX8_OK) return rc;
    Params p{};
    fill_common(p, d_gate_fp8, d_gate_sc, d_gate_sc_t, rows, cols);
    p.out2 = static_cast<uint8_t*>(d_up_fp8);
    p.sc2 = static_cast<uint8_t*>(d_up_sc);
    p.sc_t2 = static_cast<uint8_t*>(d_up_sc_t);
    p.rows_dev = static_cast<const int*>(num_rows);
    p.gate_sc = static_cast<const uint8_t*>(gate_sc);
    p.up_sc = static_cast<const uint8_t*>(up_sc);
    p.bwd_which = 2;
    p.status = device_status_ptr();
    if (!p.status) return MX8_ERR_CUDA;
    CUtensorMap tm_g, tm_u, tm_d, tm_t, tm_t2;
    const uint64_t dims[2] = {static_cast<uint64_t>(cols), static_cast<uint64_t>(rows)};
    const uint64_t strides[1] = {static_cast<uint64_t>(cols)};
    const uint64_t strides2[1] = {static_cast<uint64_t>(cols) * 2};
    const uint32_t box[2] = {128, SLAB_ROWS};
    if ((rc = make_tmap(&tm_g, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, gate_fp8, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE)) != MX8_OK) return rc;
    if ((rc = make_tmap(&tm_u, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, up_fp8, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE)) != MX8_OK) return rc;
    if ((rc = make_tmap(&tm_d, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, d_hidden, dims, strides2, box, CU_TENSOR_MAP_SWIZZLE_NONE)) != MX8_OK) return rc;
    if ((rc = make_transposed_map(&tm_t, d_gate_fp8_t, 1, rows, cols)) != MX8_OK) return rc;
    if ((rc = make_transposed_map(&tm_t2, d_up_fp8_t, 1, rows, cols)) != MX8_OK) return rc;
    CUtensorMap tm_r, tm_r2;
    if ((rc = make_row_map(&tm_r, d_gate_fp8, rows, cols)) != MX8_OK) return rc;
    if ((rc = make_row_map(&tm_r2, d_up_fp8, rows, cols)) != MX8_OK) return rc;
    int grid = sm_count();
    if (grid <= 0) return MX8_ERR_CUDA;
    const int tiles = p.tiles_r * p.tiles_c;
    if (grid > tiles) grid = tiles;
    apply_window(p, grid, window);
    return launch<MX8_Q_SWB_W, 1, SRC_SWIGLU_BWD, true, true, (MX8_Q_SWB_RTMA != 0)>(tm_g, tm_u, tm_d, tm_t, tm_r, p, grid, static_cast<cudaStream_t>(stream), &tm_t2, &tm_r2);
}
