// Block-scaled MXFP8 GEMM for sm_100a:  C[M][N] = dequant(A[M][K]) . dequant(B[N][K])^T.
//
// Persistent kernel, one CTA per SM, six warps.  Producer and MMA warps run their loops with
// warp-uniform control flow and let one elected lane issue, so that addresses, descriptors and
// coordinates live in uniform registers (where TMA and tcgen05 instructions read them) instead of
// being converted for every instruction:
//   warp 0  producer   streams A/B tiles (SWIZZLE_128B) and scale tiles with TMA into a ring of
//                      shared-memory stages; each CTA fetches only its own tiles
//   warp 1  MMA        (leader CTA when CG == 2) copies the scale tiles of the NEXT K step into one of
//                      two TMEM scale slots with tcgen05.cp, then issues four K=32
//                      tcgen05.mma.kind::mxf8f6f4.block_scale for the current 128-wide K step;
//                      tcgen05.commit releases the stage and, after the last K step, publishes the
//                      accumulator
//   warps 2-5 epilogue tcgen05.ld the fp32 accumulator (warp q owns TMEM lanes 32q..32q+31),
//                      round to bf16 (or keep fp32), stage through swizzled shared memory and
//                      write C with TMA stores
// CG == 2: a cluster of two CTAs computes one 256x256 tile with cta_group::2 instructions; each
// CTA holds 128 rows of A, 128 rows of B, its own A scales and both B scale tiles.
// CG == 1: one CTA computes a 128x256 tile.
//
// TMEM budget (512 columns): two accumulators of 256 columns cannot sit beside the scale
// columns, so they overlap: accumulator 0 = columns [0,256), accumulator 1 = [224,480), scales
// in [480,512).  The epilogue drains the shared 32 columns first and signals the MMA warp, which
// may then start the next tile while the remaining 224 columns are still being drained.
//
// M/N tails need no special case: out-of-range TMA loads are zero-filled, out-of-range TMA stores
// are clipped.  Replaces blackwell/047-mxfp8-mma-2cta-MNK128-polished.cu:12-541 of the reference.
#include <atomic>

#include "mx8_host.cuh"
#include "mx8_ptx.cuh"
#include "mx8_qmath.cuh"

// Timing studies switch parts of the kernel off through Params::dbg.  The shipped library is built without
// MX8_ABLATION: the switches are compile-time false and the setter is not exported.
#ifdef MX8_ABLATION
#define MX8_DBG(p, bits) (((p).dbg & (bits)) != 0)
#else
#define MX8_DBG(p, bits) false
#endif

namespace mx8 {
namespace gemm {

constexpr int BK = 128;                 // K elements (bytes) per stage
constexpr int BN = 256;                 // tile columns
constexpr int ACC1_COL = 224;           // first column of accumulator 1
constexpr int SF_COL = 480;             // first scale column; slot s at SF_COL + 16 s: A +0, B +4 and +8
// 4: one warp per TMEM lane quadrant drains all 256 columns.  8 (two warps per quadrant, 128 columns each)
// also works but costs a pipeline stage of shared memory and measured 3-7 % slower on every shape tried.
constexpr int EPI_WARPS = 4;
constexpr int EPI_UNITS = 8 / (EPI_WARPS / 4);   // 32-column units per epilogue warp
constexpr int MAX_GROUPS = 256;          // experts per launch of the grouped form
constexpr int THREADS = 32 * (2 + EPI_WARPS);   // producer, MMA issuer, epilogue warps

constexpr int CONV_WARPS = 8;            // A16 form: two threads per A row convert bf16 -> E4M3 + scales in shared memory
constexpr int A16_BYTES = 128 * BK * 2;  // A16 form: one bf16 A tile (two 128-byte-wide TMA boxes)
constexpr int A16_SLOTS = 2;             // A16 form: depth of the bf16 staging ring (the E4M3 stage ring is deeper)

// A16: the A operand arrives as bf16 and is quantized inside the main loop (four pipeline stages and a
// two-slot bf16 staging ring instead of six stages)
template <int CG, bool A16 = false>
struct Cfg {
    static constexpr int STAGES = A16 ? 4 : (EPI_WARPS == 4 ? (CG == 2 ? 6 : 4) : (CG == 2 ? 5 : 3));
    static constexpr int A_BYTES = 128 * BK;                 // this CTA's 128 rows of A
    static constexpr int B_ROWS = BN / CG;                   // this CTA's rows of B
    static constexpr int B_BYTES = B_ROWS * BK;
    static constexpr int SFA_BYTES = 512;
    static constexpr int SFB_BYTES = 1024;                   // both 128-column scale tiles
    static constexpr int STAGE_TX = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;   // bytes one CTA loads per stage
    static constexpr int EPI_BYTES = 32 * 128;               // per warp: 32 rows x 128 bytes (64 bf16 or 32 f32 columns)
    // offsets from the 1024-aligned base
    static constexpr int a_off = 0;
    static constexpr int b_off = a_off + STAGES * A_BYTES;
    static constexpr int sfa_off = b_off + STAGES * B_BYTES;
    static constexpr int sfb_off = sfa_off + STAGES * SFA_BYTES;
    static constexpr int a16_off = (sfb_off + STAGES * SFB_BYTES + 1023) & ~1023;     // bf16 staging ring (A16 only)
    static constexpr int epi_off = a16_off + (A16 ? A16_SLOTS * A16_BYTES : 0);
    static constexpr int bar_off = epi_off + EPI_WARPS * EPI_BYTES;
    // barriers: full[STAGES], empty[STAGES], acc_full[2], drained; A16: a_full[A16_SLOTS], a_empty[A16_SLOTS], conv_done[STAGES]
    static constexpr int n_bars = 2 * STAGES + 3 + (A16 ? 2 * A16_SLOTS + STAGES : 0);
    static constexpr int threads = THREADS + (A16 ? 32 * (CONV_WARPS + 1) : 0);   // A16: converters + the bf16 tile producer
    static constexpr int tmem_ptr_off = bar_off + n_bars * 8;
    static constexpr int flag_off = tmem_ptr_off + 8;
    static constexpr int seg_off = flag_off + 8;               // end row of every group's segment (grouped GEMM)
    static constexpr int total = seg_off + MAX_GROUPS * 4;
    static constexpr int dynamic = total + 1024;
    static_assert(dynamic <= 232448, "shared memory budget exceeded");
};

struct Params {
    int tiles_m, tiles_n, k_steps;      // tile grid (tile = 128*CG x 256) and K / 128
    int group_m;                        // rasterisation: tiles_m rows per supergroup
    int c_mode;                         // 0 bf16, 1 f32, 2 MXFP8 (E4M3 bytes + scale tiles, blocks along N),
                                        // 3 bf16 rows scattered to the ranks that own the tokens (MoE combine),
                                        // 4 gate / up as MXFP8 plus hidden = SwiGLU(gate, up) as MXFP8, row-wise and transposed
    const int* sc_peer_rank;            // c_mode 3: destination rank per row (-1: skip) and row in its buffer
    const int* sc_peer_token_idx;
    uint8_t* sc_dst[16];
    uint8_t* c_sc;                      // scale tiles of C for c_mode 2
    int n_cols;                         // N
    int rows_cap;                       // M (rows the C tensors have)
    const int* rows_dev;                // device: rows actually present (nullptr: all tiles_m tiles)
    const int* row_begin_dev;           // device: first row of the window to compute (multiple of the tile height), nullptr = 0
    const int* group_rows;              // device: rows of every group (multiples of the tile height), nullptr = dense
    int num_groups;
    int group_b_rows;                   // rows of B per group (N)
    int k_steps2;                       // second operand pair accumulated into the same tile (0 = none)
    int pair_tiles_n;                   // > 0: two products A B1^T and A B2^T in one launch; column tiles [0, pair_tiles_n) belong
                                        // to the first (B1 -> C), [pair_tiles_n, 2 pair_tiles_n) to the second (B2 -> C2)
    uint8_t* c_sc2;                     // scale tiles of C2 for c_mode 2
    // c_mode 4 (gate and up projections with SwiGLU in the epilogue): a tile is 128 output columns wide, CTA 0 of the
    // pair holds the gate weights' rows, CTA 1 the up weights' rows, so accumulator columns [0,128) are gate and
    // [128,256) are up of the same 128 output columns
    uint8_t *sw_gate, *sw_gate_sc, *sw_up, *sw_up_sc, *sw_h, *sw_h_sc, *sw_ht, *sw_ht_sc;
    int wgrad;                          // 1: one output matrix per group, K runs over the group's rows of A^T / B^T
    int group_c_rows;                   // wgrad: rows of C per group (M)
    int dbg;                            // ablation switches (only in a build with -DMX8_ABLATION; timing only, results are wrong):
                                        // 1 no MMA, 2 no TMA loads, 4 no C stores, 8 no scale traffic, 16 no scale copies,
                                        // 32 no scale loads, 128 no wait for the epilogue
    int* status;
};

// persistent tile order: supergroups of `group_m` tile rows, column-major inside a supergroup so
// that CTAs running at the same time share A row panels and B column panels in L2
__device__ __forceinline__ void tile_coords(int t, const Params& p, int tiles_m, int& tm, int& tn) {
    const int per_group = p.group_m * p.tiles_n;
    const int grp = t / per_group;
    const int in_grp = t - grp * per_group;
    const int rows = min(p.group_m, tiles_m - grp * p.group_m);
    tm = grp * p.group_m + in_grp % rows;
    tn = in_grp / rows;
}

// Everything a role needs to know about tile t.  Three shapes of problem share the kernel:
//   dense    tile (tm, tn) of C = A B^T;
//   grouped  the same, but the B rows of a tile come from the group that owns its A rows;
//   wgrad    C_g = A^T_g B^T_g^T for every group g: A^T is [M][rows], B^T is [N][rows] and the K loop of
//            a tile covers only the rows (columns of A^T) of its group.
struct TileInfo {
    int tm, tn;        // tile coordinates inside one C matrix
    int b_base;        // first row of B for this tile (before the CTA's own offset)
    int c_row;         // first row of C for this tile (before the CTA's own offset)
    int k0, kcount;    // first K step and number of K steps
    int second;        // 1: this tile belongs to the second product of a pair launch (tn already counts inside it)
};

template <int CG>
__device__ __forceinline__ TileInfo tile_info(int t, const Params& p, int tiles_m, const int* seg_end, int tm0 = 0) {
    TileInfo ti;
    ti.second = 0;
    if (p.wgrad) {
        const int per_group = tiles_m * p.tiles_n;
        const int e = t / per_group;
        tile_coords(t - e * per_group, p, tiles_m, ti.tm, ti.tn);
        const int begin = e ? seg_end[e - 1] : 0;
        ti.k0 = begin / BK;
        ti.kcount = (seg_end[e] - begin) / BK;
        ti.b_base = ti.tn * BN;
        ti.c_row = e * p.group_c_rows + ti.tm * 128 * CG;
        return ti;
    }
    tile_coords(t, p, tiles_m, ti.tm, ti.tn);
    ti.tm += tm0;                                     // row window: tile rows are counted from its first row
    if (p.pair_tiles_n > 0 && ti.tn >= p.pair_tiles_n) {
        ti.second = 1;
        ti.tn -= p.pair_tiles_n;
    }
    ti.b_base = ti.tn * (p.c_mode == 4 ? BN / 2 : BN);
    if (p.num_groups > 0) {
        const int row0 = ti.tm * 128 * CG;
        int lo = 0, hi = p.num_groups - 1;            // first group whose segment ends beyond row0
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (seg_end[mid] > row0) hi = mid; else lo = mid + 1;
        }
        ti.b_base += lo * p.group_b_rows;
    }
    ti.c_row = ti.tm * 128 * CG;
    ti.k0 = 0;
    ti.kcount = p.k_steps + p.k_steps2;
    return ti;
}

// Epilogue of c_mode 4 for one warp (TMEM lane quadrant q, lane = row): accumulator columns [0,128) hold the gate
// projection and [128,256) the up projection of output columns [ocol0, ocol0 + 128).  Per group of 32 columns:
// both are rounded to bf16 and quantized as one block each (the bytes and scales the separate launches write),
// hidden = bf16( silu(dequant(gate)) * dequant(up) ) is computed from the quantized values with the arithmetic of
// the stand-alone SwiGLU kernel, quantized row-wise, and, after a transposition of the 32 x 32 block through shared
// memory, quantized along the rows as well.  Replaces expert_grouped_gemm's quantizing epilogue plus swiglu_fwd<false>
// (blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.cu:1644-1700, 924-1129).
// `drain` is called once, after the first two accumulator units (which include the unit the two accumulators share)
// have been read.
template <typename DrainFn>
__device__ __forceinline__ void swiglu_epilogue(const Params& p, uint32_t t_acc, int acc, int row0, int ocol0, int q, int lane,
                                                uint32_t stg, uint8_t* stg_ptr, DrainFn drain) {
    using namespace qmath;
    const int I = p.n_cols;
    const bool row_ok = row0 + lane < p.rows_cap;
    const size_t row_off = static_cast<size_t>(row0 + lane) * I + ocol0;
    uint32_t sc_g = 0, sc_u = 0, sc_h = 0;
#pragma unroll 1
    for (int s = 0; s < 4; ++s) {
        const int j = acc ? s : 3 - s;                        // accumulator 0 shares its last unit, accumulator 1 its first
        uint32_t rg[32], ru[32];
        tc_ld_32x32(t_acc + j * 32, rg);
        tc_ld_32x32(t_acc + (4 + j) * 32, ru);
        tc_wait_ld(rg);
        tc_wait_ld(ru);
        if (s == 0) drain();
        // ---- gate and up: bf16 rounding, one MXFP8 block each
        uint32_t hg[16], hu[16], qg[8], qu[8];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            hg[i] = pack_bf16x2(__uint_as_float(rg[2 * i]), __uint_as_float(rg[2 * i + 1]));
            hu[i] = pack_bf16x2(__uint_as_float(ru[2 * i]), __uint_as_float(ru[2 * i + 1]));
        }
        auto block_scale = [&](const uint32_t (&h)[16], uint32_t& byte, uint32_t& inv) {
            uint32_t m = maxabs_bf16x2(h[0], h[1]);
#pragma unroll
            for (int i = 2; i < 16; ++i) m = maxabs_bf16x2(m, h[i]);
            m &= 0x7FFF7FFFu;
            byte = scale_bytes2(max(m & 0xFFFFu, m >> 16), RCEIL_ROUND_ADD2, RCEIL_MIN_BYTE8_2) & 0xFFu;
            inv = inv_scales2(byte | (byte << 16));
        };
        uint32_t bg, bu, ig, iu;
        block_scale(hg, bg, ig);
        block_scale(hu, bu, iu);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            qg[i] = cvt4(mul_bf16x2(hg[2 * i], ig), mul_bf16x2(hg[2 * i + 1], ig));
            qu[i] = cvt4(mul_bf16x2(hu[2 * i], iu), mul_bf16x2(hu[2 * i + 1], iu));
        }
        if (row_ok) {
            uint4* dg = reinterpret_cast<uint4*>(p.sw_gate + row_off + j * 32);
            uint4* du = reinterpret_cast<uint4*>(p.sw_up + row_off + j * 32);
            dg[0] = make_uint4(qg[0], qg[1], qg[2], qg[3]);
            dg[1] = make_uint4(qg[4], qg[5], qg[6], qg[7]);
            du[0] = make_uint4(qu[0], qu[1], qu[2], qu[3]);
            du[1] = make_uint4(qu[4], qu[5], qu[6], qu[7]);
        }
        sc_g |= bg << (8 * j);
        sc_u |= bu << (8 * j);
        // ---- hidden from the quantized values, in fp32
        const float gs = __uint_as_float(bg << 23), us = __uint_as_float(bu << 23);
        uint32_t hh[16];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float gf[4], uf[4], h[4];
            e4m3x4_to_float(qg[i], gf);
            e4m3x4_to_float(qu[i], uf);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float g = gf[e] * gs;
                h[e] = __fdividef(g, 1.0f + __expf(-g)) * (uf[e] * us);
            }
            hh[2 * i] = pack_bf16x2(h[0], h[1]);
            hh[2 * i + 1] = pack_bf16x2(h[2], h[3]);
        }
        // ---- row-wise block of hidden
        uint32_t bh, ih;
        block_scale(hh, bh, ih);
        if (row_ok) {
            uint4* dh = reinterpret_cast<uint4*>(p.sw_h + row_off + j * 32);
            dh[0] = make_uint4(cvt4(mul_bf16x2(hh[0], ih), mul_bf16x2(hh[1], ih)), cvt4(mul_bf16x2(hh[2], ih), mul_bf16x2(hh[3], ih)),
                               cvt4(mul_bf16x2(hh[4], ih), mul_bf16x2(hh[5], ih)), cvt4(mul_bf16x2(hh[6], ih), mul_bf16x2(hh[7], ih)));
            dh[1] = make_uint4(cvt4(mul_bf16x2(hh[8], ih), mul_bf16x2(hh[9], ih)), cvt4(mul_bf16x2(hh[10], ih), mul_bf16x2(hh[11], ih)),
                               cvt4(mul_bf16x2(hh[12], ih), mul_bf16x2(hh[13], ih)), cvt4(mul_bf16x2(hh[14], ih), mul_bf16x2(hh[15], ih)));
        }
        sc_h |= bh << (8 * j);
        // ---- the 32 x 32 block transposed through shared memory (rows of 17 words: stores and loads are conflict-free):
        // afterwards lane c holds column c of the 32 rows this warp owns, one 32-row block of the transposed matrix
        __syncwarp();
#pragma unroll
        for (int w = 0; w < 16; ++w) asm volatile("st.shared.b32 [%0], %1;" ::"r"(stg + lane * 68 + w * 4), "r"(hh[w]) : "memory");
        __syncwarp();
        uint32_t ht[16];
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            const uint32_t lo = *reinterpret_cast<const uint16_t*>(stg_ptr + (2 * r) * 68 + lane * 2);
            const uint32_t hi = *reinterpret_cast<const uint16_t*>(stg_ptr + (2 * r + 1) * 68 + lane * 2);
            ht[r] = lo | (hi << 16);
        }
        uint32_t bt, it;
        block_scale(ht, bt, it);
        const int col = ocol0 + j * 32 + lane;
        if (row0 < p.rows_cap && col < I) {
            uint4* dt = reinterpret_cast<uint4*>(p.sw_ht + static_cast<size_t>(col) * p.rows_cap + row0);
            dt[0] = make_uint4(cvt4(mul_bf16x2(ht[0], it), mul_bf16x2(ht[1], it)), cvt4(mul_bf16x2(ht[2], it), mul_bf16x2(ht[3], it)),
                               cvt4(mul_bf16x2(ht[4], it), mul_bf16x2(ht[5], it)), cvt4(mul_bf16x2(ht[6], it), mul_bf16x2(ht[7], it)));
            dt[1] = make_uint4(cvt4(mul_bf16x2(ht[8], it), mul_bf16x2(ht[9], it)), cvt4(mul_bf16x2(ht[10], it), mul_bf16x2(ht[11], it)),
                               cvt4(mul_bf16x2(ht[12], it), mul_bf16x2(ht[13], it)), cvt4(mul_bf16x2(ht[14], it), mul_bf16x2(ht[15], it)));
            // scale byte of (column col, rows row0 .. row0 + 31) in the tile layout of the transposed matrix
            p.sw_ht_sc[(static_cast<size_t>(ocol0 / 128) * (p.rows_cap / 128) + row0 / 128) * 512 + lane * 16 + j * 4 + q] = static_cast<uint8_t>(bt);
        }
    }
    if (row_ok) {
        const size_t word = (static_cast<size_t>(row0 / 128) * (I / 128) + ocol0 / 128) * 512 + lane * 16 + q * 4;
        *reinterpret_cast<uint32_t*>(p.sw_gate_sc + word) = sc_g;
        *reinterpret_cast<uint32_t*>(p.sw_up_sc + word) = sc_u;
        *reinterpret_cast<uint32_t*>(p.sw_h_sc + word) = sc_h;
    }
}

// F16: A and B are bf16 (kind::f16, no scale tiles); the byte images in shared memory, the stage
// ring and the epilogue are the same, a K step being 128 bytes = 64 bf16 elements of a row.
template <int CG, bool F16, bool A16 = false, bool SW = false>
__global__ void __launch_bounds__((Cfg<CG, A16>::threads), 1)
gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
            const __grid_constant__ CUtensorMap tm_sfa, const __grid_constant__ CUtensorMap tm_sfb,
            const __grid_constant__ CUtensorMap tm_a2, const __grid_constant__ CUtensorMap tm_b2,
            const __grid_constant__ CUtensorMap tm_sfa2, const __grid_constant__ CUtensorMap tm_sfb2,
            const __grid_constant__ CUtensorMap tm_c, const __grid_constant__ CUtensorMap tm_c2, const Params p) {
    using C = Cfg<CG, A16>;
    constexpr int S = C::STAGES;
    static_assert(!A16 || (CG == 2 && !F16), "the bf16-activation form exists for the 2-CTA MXFP8 kernel only");
    static_assert(!SW || (CG == 2 && !F16 && !A16 && EPI_WARPS == 4), "the SwiGLU epilogue exists for the 2-CTA MXFP8 kernel only");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t full0 = base + C::bar_off;
    const uint32_t empty0 = full0 + S * 8;
    const uint32_t accfull0 = empty0 + S * 8;
    const uint32_t drained = accfull0 + 2 * 8;
    const uint32_t afull0 = drained + 8;            // A16 only: bf16 tile landed / staging free / fp8 tile + scales written
    const uint32_t aempty0 = afull0 + A16_SLOTS * 8;
    const uint32_t convdone0 = aempty0 + A16_SLOTS * 8;
    volatile uint32_t* tmem_ptr = reinterpret_cast<volatile uint32_t*>(base_ptr + C::tmem_ptr_off);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + C::flag_off);
    const AbortCtl ab{abort_flag, p.status};

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = CG == 2 ? cluster_ctarank() : 0;
    const int cluster = CG == 2 ? static_cast<int>(cluster_id_x()) : static_cast<int>(blockIdx.x);
    const int num_clusters = CG == 2 ? static_cast<int>(num_clusters_x()) : static_cast<int>(gridDim.x);

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < S; ++s) {
            mbar_init(full0 + s * 8, 1);       // the leader producer's arrive.expect_tx
            mbar_init(empty0 + s * 8, 1);      // one tcgen05.commit
        }
        mbar_init(accfull0, 1);
        mbar_init(accfull0 + 8, 1);
        mbar_init(drained, EPI_WARPS * CG);
        if constexpr (A16) {
            for (int s = 0; s < A16_SLOTS; ++s) {
                mbar_init(afull0 + s * 8, 1);               // this CTA's bf16 tile producer
                mbar_init(aempty0 + s * 8, CONV_WARPS);     // this CTA's converter warps
            }
            for (int s = 0; s < S; ++s) mbar_init(convdone0 + s * 8, CONV_WARPS * CG);   // both CTAs' converters (leader's copy is waited on)
        }
        fence_mbar_init();
        prefetch_tmap(&tm_a);
        prefetch_tmap(&tm_b);
        prefetch_tmap(&tm_sfa);
        prefetch_tmap(&tm_sfb);
        prefetch_tmap(&tm_c);
    }
    if (warp == 1) {
        tmem_alloc<CG>(smem_u32(const_cast<uint32_t*>(tmem_ptr)), 512);
        tmem_relinquish<CG>();
    }
    __syncwarp();
    tc_fence_before();
    if constexpr (CG == 2) cluster_sync_all(); else __syncthreads();
    tc_fence_after();
    // broadcast from lane 0 so the compiler can keep the value (and everything derived from it) in
    // uniform registers, which is where tcgen05 and TMA instructions take their operands from
    const uint32_t tmem_base = __shfl_sync(0xFFFFFFFFu, *tmem_ptr, 0);
    // grouped form: row tiles come from a device-side count and every tile's B rows from its group
    int* seg_end = reinterpret_cast<int*>(base_ptr + C::seg_off);
    int tiles_m = p.tiles_m;
    if (p.rows_dev) {
        const int rows = *p.rows_dev;
        tiles_m = min(tiles_m, (rows + 128 * CG - 1) / (128 * CG));
    }
    int tm0 = 0;
    if (p.row_begin_dev) {
        tm0 = *p.row_begin_dev / (128 * CG);
        tiles_m = max(tiles_m - tm0, 0);
    }
    tiles_m = __shfl_sync(0xFFFFFFFFu, tiles_m, 0);     // loaded value: make it provably warp-uniform
    tm0 = __shfl_sync(0xFFFFFFFFu, tm0, 0);
    if (p.num_groups > 0) {
        if (threadIdx.x == 0) {
            int acc = 0;
            for (int e = 0; e < p.num_groups; ++e) {
                acc += p.group_rows[e];
                seg_end[e] = acc;
            }
        }
        __syncthreads();
    }
    const int num_tiles = tiles_m * p.tiles_n * (p.wgrad ? p.num_groups : 1);

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        // The whole warp walks the loop (uniform control flow, operands in uniform registers); one
        // elected lane issues the copies.
        {
            const bool leader = elect_one();
            uint32_t stage = 0, ph = 0;
            const uint32_t full_leader0 = CG == 2 ? map_to_cta(full0, 0) : full0;
            bool ok = true;
            for (int t = cluster; t < num_tiles && ok; t += num_clusters) {
                const TileInfo ti = tile_info<CG>(t, p, tiles_m, seg_end, tm0);
                const int a_row = (__shfl_sync(0xFFFFFFFFu, ti.tm, 0) * CG + static_cast<int>(rank)) * 128;
                const int b_base = __shfl_sync(0xFFFFFFFFu, ti.b_base, 0);
                const int kcount_t = __shfl_sync(0xFFFFFFFFu, ti.kcount, 0), k0_t = __shfl_sync(0xFFFFFFFFu, ti.k0, 0);
                // c_mode 4: both CTAs fetch the same rows, CTA 0 of the gate weights and CTA 1 of the up weights
                constexpr bool swiglu = SW;
                const int b_row = swiglu ? b_base : b_base + static_cast<int>(rank) * C::B_ROWS;
                const bool pair_second = __shfl_sync(0xFFFFFFFFu, ti.second, 0) != 0 || (swiglu && rank == 1);
                for (int ks = 0; ks < kcount_t; ++ks) {
                    if (!__all_sync(0xFFFFFFFFu, mbar_wait(empty0 + stage * 8, ph ^ 1, ab, DEV_TIMEOUT_EMPTY))) { ok = false; break; }
                    const uint32_t a_dst = base + C::a_off + stage * C::A_BYTES;
                    const uint32_t b_dst = base + C::b_off + stage * C::B_BYTES;
                    const uint32_t sfa_dst = base + C::sfa_off + stage * C::SFA_BYTES;
                    const uint32_t sfb_dst = base + C::sfb_off + stage * C::SFB_BYTES;
                    // K step within the operand pair it belongs to
                    const bool second = ks >= p.k_steps && p.k_steps2 > 0;
                    const int kk = k0_t + (second ? ks - p.k_steps : ks);
                    const CUtensorMap* ma = second ? &tm_a2 : &tm_a;
                    const CUtensorMap* mb = (second || pair_second) ? &tm_b2 : &tm_b;
                    const CUtensorMap* msa = second ? &tm_sfa2 : &tm_sfa;
                    const CUtensorMap* msb = (second || pair_second) ? &tm_sfb2 : &tm_sfb;
                    if (!leader) {
                        // only the elected lane issues
                    } else if constexpr (A16) {
                        // B and its scales as usual (signalling the leader's barrier); A as bf16 into this CTA's own
                        // staging slot, two 128-byte-wide boxes, signalling this CTA's a_full
                        const uint32_t bar = full_leader0 + stage * 8;
                        if (rank == 0) mbar_arrive_expect_tx(full0 + stage * 8, 2 * (C::B_BYTES + C::SFB_BYTES));
                        tma_load_2d_pair(b_dst, mb, kk * BK, b_row, bar);
                        tma_load_3d_pair(sfb_dst, msb, 0, kk, b_base / 128, bar);
                    } else if constexpr (CG == 2) {
                        const uint32_t bar = full_leader0 + stage * 8;
                        if (MX8_DBG(p, 2)) {
                            if (rank == 0) mbar_arrive(full0 + stage * 8);
                        } else if (F16 || MX8_DBG(p, 8 | 32)) {
                            if (rank == 0) mbar_arrive_expect_tx(full0 + stage * 8, 2 * (C::A_BYTES + C::B_BYTES));
                            tma_load_2d_pair(a_dst, ma, kk * BK, a_row, bar);
                            tma_load_2d_pair(b_dst, mb, kk * BK, b_row, bar);
                        } else {
                            if (rank == 0) mbar_arrive_expect_tx(full0 + stage * 8, 2 * C::STAGE_TX);
                            tma_load_2d_pair(a_dst, ma, kk * BK, a_row, bar);
                            tma_load_2d_pair(b_dst, mb, kk * BK, b_row, bar);
                            tma_load_3d_pair(sfa_dst, msa, 0, kk, a_row / 128, bar);
                            if (swiglu) {
                                // one scale tile of each weight matrix (their maps have a box of one tile)
                                tma_load_3d_pair(sfb_dst, &tm_sfb, 0, kk, b_base / 128, bar);
                                tma_load_3d_pair(sfb_dst + 512, &tm_sfb2, 0, kk, b_base / 128, bar);
                            } else {
                                tma_load_3d_pair(sfb_dst, msb, 0, kk, b_base / 128, bar);
                            }
                        }
                    } else {
                        const uint32_t bar = full0 + stage * 8;
                        mbar_arrive_expect_tx(bar, F16 ? C::A_BYTES + C::B_BYTES : C::STAGE_TX);
                        tma_load_2d(a_dst, ma, kk * BK, a_row, bar);
                        tma_load_2d(b_dst, mb, kk * BK, b_row, bar);
                        if constexpr (!F16) {
                            tma_load_3d(sfa_dst, msa, 0, kk, a_row / 128, bar);
                            tma_load_3d(sfb_dst, msb, 0, kk, b_base / 128, bar);
                        }
                    }
                    if (++stage == S) { stage = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader CTA only)
        if (rank == 0) {
            const bool leader = elect_one();
            // Everything this loop needs per K step is kept as a running 32-bit value so that the
            // single issuing thread spends its time on tcgen05 instructions, not on address math.
            // The scale copies run one K step ahead of the MMAs (two scale slots in TMEM), so an MMA
            // never waits for the copy issued right before it.
            const uint32_t a_lo0 = desc_sw128_lo(base + C::a_off), b_lo0 = desc_sw128_lo(base + C::b_off);
            const uint32_t sfa_lo0 = desc_scales_lo(base + C::sfa_off), sfb_lo0 = desc_scales_lo(base + C::sfb_off);
            uint32_t a_lo = a_lo0, b_lo = b_lo0;                 // stage the MMAs read
            uint32_t sfa_lo = sfa_lo0, sfb_lo = sfb_lo0;         // stage the next scale copy reads
            uint32_t empty_bar = empty0, stage = 0;              // MMA side
            uint32_t full_bar = full0, cstage = 0, cph = 0;      // copy side (one step ahead)
            uint32_t sf_mma = tmem_base + SF_COL, sf_cp = tmem_base + SF_COL;
            constexpr uint32_t ID0 = idesc_mxf8(128 * CG, BN, 0), ID1 = idesc_mxf8(128 * CG, BN, 1);
            constexpr uint32_t ID2 = idesc_mxf8(128 * CG, BN, 2), ID3 = idesc_mxf8(128 * CG, BN, 3);
            const bool do_cp = !F16 && !MX8_DBG(p, 8 | 16), do_mma = !MX8_DBG(p, 1);
            const int my_tiles = cluster < num_tiles ? (num_tiles - cluster + num_clusters - 1) / num_clusters : 0;
            long long remaining = 0;                             // K steps whose scales are not copied yet
            for (int t = cluster; t < num_tiles; t += num_clusters) remaining += tile_info<CG>(t, p, tiles_m, seg_end, tm0).kcount;
            bool ok = true;
            // wait for a stage and copy its scale tiles into the next TMEM scale slot
            auto copy_scales = [&]() -> bool {
                if (!__all_sync(0xFFFFFFFFu, mbar_wait(full_bar, cph, ab, DEV_TIMEOUT_FULL))) return false;
                if constexpr (A16) {
                    // both CTAs' converters have written this stage's E4M3 tile and A scales
                    if (!__all_sync(0xFFFFFFFFu, mbar_wait<true>(convdone0 + cstage * 8, cph, ab, DEV_TIMEOUT_FULL))) return false;
                }
                tc_fence_after();
                if (do_cp && leader) {
                    tc_cp_scales_lo<CG>(sf_cp, sfa_lo);
                    tc_cp_scales_lo<CG>(sf_cp + 4, sfb_lo);
                    tc_cp_scales_lo<CG>(sf_cp + 8, sfb_lo + (512 >> 4));
                }
                sf_cp ^= 16;                                     // SF_COL is a multiple of 32: toggles the slot
                --remaining;
                if (++cstage == S) {
                    cstage = 0; cph ^= 1; sfa_lo = sfa_lo0; sfb_lo = sfb_lo0; full_bar = full0;
                } else {
                    sfa_lo += C::SFA_BYTES >> 4; sfb_lo += C::SFB_BYTES >> 4; full_bar += 8;
                }
                return true;
            };
            if (remaining > 0) ok = copy_scales();
            for (int it = 0; it < my_tiles && ok; ++it) {
                const uint32_t d_tmem = tmem_base + ((it & 1) ? ACC1_COL : 0);
                if (it > 0) {
                    // the epilogue has emptied the previous-but-one accumulator and the 32 columns
                    // the previous accumulator shares with this one
                    if (!MX8_DBG(p, 128) && !__all_sync(0xFFFFFFFFu, mbar_wait<true>(drained, (it - 1) & 1, ab, DEV_TIMEOUT_TMEM_FREE))) { ok = false; break; }
                    tc_fence_after();
                }
                const int kcount = __shfl_sync(0xFFFFFFFFu, tile_info<CG>(cluster + it * num_clusters, p, tiles_m, seg_end, tm0).kcount, 0);
                for (int ks = 0; ks < kcount; ++ks) {
                    if (remaining > 0 && !copy_scales()) { ok = false; break; }
                    if constexpr (F16) {
                        if (do_mma && leader) {
                            constexpr uint32_t IDF = idesc_bf16(128 * CG, BN);
                            tc_mma_bf16_lo<CG, 2>(d_tmem, a_lo, b_lo, IDF, static_cast<uint32_t>(ks));
                            tc_mma_bf16_lo<CG, 1>(d_tmem, a_lo + 2, b_lo + 2, IDF);
                            tc_mma_bf16_lo<CG, 1>(d_tmem, a_lo + 4, b_lo + 4, IDF);
                            tc_mma_bf16_lo<CG, 1>(d_tmem, a_lo + 6, b_lo + 6, IDF);
                        }
                    } else if (do_mma && leader) {
                        // each K=32 slice lies 32 bytes further inside the swizzle atom: +2 in the address field
                        tc_mma_mxf8_lo<CG, 2>(d_tmem, a_lo, b_lo, ID0, sf_mma, sf_mma + 4, static_cast<uint32_t>(ks));
                        tc_mma_mxf8_lo<CG, 1>(d_tmem, a_lo + 2, b_lo + 2, ID1, sf_mma, sf_mma + 4);
                        tc_mma_mxf8_lo<CG, 1>(d_tmem, a_lo + 4, b_lo + 4, ID2, sf_mma, sf_mma + 4);
                        tc_mma_mxf8_lo<CG, 1>(d_tmem, a_lo + 6, b_lo + 6, ID3, sf_mma, sf_mma + 4);
                    }
                    if (leader) tc_commit<CG>(empty_bar);        // stage reusable once these MMAs retire
                    sf_mma ^= 16;
                    if (++stage == S) {
                        stage = 0; a_lo = a_lo0; b_lo = b_lo0; empty_bar = empty0;
                    } else {
                        a_lo += C::A_BYTES >> 4; b_lo += C::B_BYTES >> 4; empty_bar += 8;
                    }
                }
                if (ok && leader) tc_commit<CG>(accfull0 + (it & 1) * 8);  // accumulator complete
            }
        }
    } else if (A16 && warp == 2 + EPI_WARPS + CONV_WARPS) {
        // ------------------------------------------------------------------ bf16 tile producer (A16 form)
        // Its own warp, so that the bf16 tiles run ahead by the depth of the staging ring no matter how far the
        // MMAs are behind: a staging slot is free as soon as the converters have read it.
        if constexpr (A16) {
            const bool leader = elect_one();
            uint32_t slot = 0, ph = 0;
            bool ok = true;
            for (int t = cluster; t < num_tiles && ok; t += num_clusters) {
                const TileInfo ti = tile_info<CG>(t, p, tiles_m, seg_end, tm0);
                const int a_row = (__shfl_sync(0xFFFFFFFFu, ti.tm, 0) * CG + static_cast<int>(rank)) * 128;
                const int kcount_t = __shfl_sync(0xFFFFFFFFu, ti.kcount, 0), k0_t = __shfl_sync(0xFFFFFFFFu, ti.k0, 0);
                for (int ks = 0; ks < kcount_t; ++ks) {
                    if (!__all_sync(0xFFFFFFFFu, mbar_wait(aempty0 + slot * 8, ph ^ 1, ab, DEV_TIMEOUT_EMPTY))) { ok = false; break; }
                    if (leader) {
                        const uint32_t a16 = base + C::a16_off + slot * A16_BYTES, abar = afull0 + slot * 8;
                        mbar_arrive_expect_tx(abar, A16_BYTES);
                        tma_load_2d(a16, &tm_a, (k0_t + ks) * 2 * BK, a_row, abar);
                        tma_load_2d(a16 + A16_BYTES / 2, &tm_a, (k0_t + ks) * 2 * BK + BK, a_row, abar);
                    }
                    if (++slot == A16_SLOTS) { slot = 0; ph ^= 1; }
                }
            }
        }
    } else if (A16 && warp >= 2 + EPI_WARPS) {
        // ------------------------------------------------------------------ converter (A16 form)
        // Two threads share row r of this CTA's A tile, one per 64-column half: 128 bf16 of a K step arrive in the
        // staging slot (two SWIZZLE_128B boxes of 64 columns); per 32-column block a thread takes the amax, the
        // scale byte (the reference's rule) and writes 32 E4M3 bytes into the stage's A tile in the layout a TMA
        // load with SWIZZLE_128B would have produced, then its two scale bytes into the stage's scale tile.
        if constexpr (A16) {
            using namespace qmath;
            const int ct = static_cast<int>(threadIdx.x) - 32 * (2 + EPI_WARPS);
            const int r = ct & 127, half = ct >> 7;
            const uint32_t sw = static_cast<uint32_t>(r & 7);
            const uint32_t convdone_leader0 = map_to_cta(convdone0, 0);
            uint32_t stage = 0, ph = 0;        // E4M3 stage ring
            uint32_t slot = 0, sph = 0;        // bf16 staging ring
            bool ok = true;
            for (int t = cluster; t < num_tiles && ok; t += num_clusters) {
                const int kcount_t = tile_info<CG>(t, p, tiles_m, seg_end, tm0).kcount;
                for (int ks = 0; ks < kcount_t; ++ks) {
                    if (!mbar_wait(afull0 + slot * 8, sph, ab, DEV_TIMEOUT_FULL)) { ok = false; break; }
                    if (!mbar_wait(empty0 + stage * 8, ph ^ 1, ab, DEV_TIMEOUT_EMPTY)) { ok = false; break; }   // MMAs of the previous use retired
                    const uint32_t src = base + C::a16_off + slot * A16_BYTES + half * (A16_BYTES / 2) + r * 128;
                    const uint32_t a8 = base + C::a_off + stage * C::A_BYTES + r * 128;
                    uint32_t scword = 0;
#pragma unroll
                    for (int b2 = 0; b2 < 2; ++b2) {
                        const int kb = 2 * half + b2;
                        const uint32_t c0 = b2 * 4;
                        uint32_t v[16];
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            ld_shared_v4(src + (((c0 + c) ^ sw) << 4), v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
                        uint32_t m = maxabs_bf16x2(v[0], v[1]);
#pragma unroll
                        for (int j = 2; j < 16; ++j) m = maxabs_bf16x2(m, v[j]);
                        m &= 0x7FFF7FFFu;
                        const uint32_t amax = max(m & 0xFFFFu, m >> 16);
                        const uint32_t byte = scale_bytes2(amax, RCEIL_ROUND_ADD2, RCEIL_MIN_BYTE8_2) & 0xFFu;
                        const uint32_t inv = inv_scales2(byte | (byte << 16));
                        uint32_t w[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) w[j] = cvt4(mul_bf16x2(v[2 * j], inv), mul_bf16x2(v[2 * j + 1], inv));
                        st_shared_v4(a8 + (((2 * kb) ^ sw) << 4), w[0], w[1], w[2], w[3]);
                        st_shared_v4(a8 + (((2 * kb + 1) ^ sw) << 4), w[4], w[5], w[6], w[7]);
                        scword |= byte << (8 * b2);
                    }
                    asm volatile("st.shared.b16 [%0], %1;" ::"r"(base + C::sfa_off + stage * C::SFA_BYTES + (r & 31) * 16 + (r >> 5) * 4 + 2 * half),
                                 "h"(static_cast<uint16_t>(scword)) : "memory");
                    fence_proxy_async_smem();                 // generic-proxy writes -> visible to tcgen05 / tcgen05.cp
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(aempty0 + slot * 8);                          // staging slot may be refilled
                        mbar_arrive_remote(convdone_leader0 + stage * 8);          // tile + scales ready for the MMA warp
                    }
                    if (++stage == S) { stage = 0; ph ^= 1; }
                    if (++slot == A16_SLOTS) { slot = 0; sph ^= 1; }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue
        const int q = warp & 3;                                  // TMEM lane quadrant this warp may read
        const int half = (warp - 2) >> 2;                        // which 128 columns of the 256-column tile
        const uint32_t stg = base + C::epi_off + (warp - 2) * C::EPI_BYTES;
        const uint32_t drained_leader = CG == 2 ? map_to_cta(drained, 0) : drained;
        int it = 0;
        bool ok = true;
        for (int t = cluster; t < num_tiles && ok; t += num_clusters, ++it) {
            const TileInfo ti = tile_info<CG>(t, p, tiles_m, seg_end, tm0);
            const int tn = ti.tn;
            const bool zero_tile = ti.kcount == 0;                // wgrad of a group without rows: nothing was accumulated
            const int acc = it & 1;
            if (!mbar_wait(accfull0 + acc * 8, (it >> 1) & 1, ab, DEV_TIMEOUT_TMEM_FULL)) { ok = false; break; }
            tc_fence_after();
            const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + (acc ? ACC1_COL : 0);
            const int row0 = ti.c_row + static_cast<int>(rank) * 128 + q * 32;
            const int col0 = tn * BN;
            const CUtensorMap* const mc = ti.second ? &tm_c2 : &tm_c;
            uint8_t* const c_sc = ti.second ? p.c_sc2 : p.c_sc;
            uint32_t scword = 0;                                 // four scale bytes of one row (c_mode 2)
            uint8_t* sc_row = nullptr;                           // c_mode 3: where this lane's row goes
            if constexpr (SW) {
                swiglu_epilogue(p, t_acc, acc, row0, tn * (BN / 2), q, lane, stg, base_ptr + C::epi_off + (warp - 2) * C::EPI_BYTES, [&]() {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_remote(drained_leader);
                });
                continue;
            }
#pragma unroll 1
            for (int s = 0; s < EPI_UNITS; ++s) {
                // 32-column unit of this warp's half; the unit the two accumulators share (the last of
                // accumulator 0, the first of accumulator 1) is the first one its warp drains
                const int u = half * EPI_UNITS + (acc ? s : EPI_UNITS - 1 - s);
                uint32_t r[32];
                tc_ld_32x32(t_acc + u * 32, r);
                tc_wait_ld(r);
                if (zero_tile) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = 0;
                }
                if (s == 0) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_remote(drained_leader);
                }
                const uint32_t rowa = stg + lane * 128;
                if (p.c_mode == 1) {
                    if (lane == 0) bulk_wait_read<0>();
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        st_shared_v4(rowa + ((j ^ (lane & 7)) << 4), r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0 && !MX8_DBG(p, 4)) {
                        tma_store_2d(mc, col0 + u * 32, row0, stg);
                        bulk_commit();
                    }
                } else if (p.c_mode == 2) {
                    // MXFP8 output: round the accumulator to bf16, then quantize this thread's 32
                    // consecutive columns as one block (amax in registers, no shuffle)
                    using namespace qmath;
                    uint32_t h[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) h[j] = pack_bf16x2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                    uint32_t m = maxabs_bf16x2(h[0], h[1]);
#pragma unroll
                    for (int j = 2; j < 16; ++j) m = maxabs_bf16x2(m, h[j]);
                    m &= 0x7FFF7FFFu;
                    const uint32_t amax = max(m & 0xFFFFu, m >> 16);
                    const uint32_t byte = scale_bytes2(amax, RCEIL_ROUND_ADD2, RCEIL_MIN_BYTE8_2) & 0xFFu;
                    const uint32_t inv = inv_scales2(byte | (byte << 16));
                    if ((u & 3) == (acc ? 0 : 3)) {      // first unit of a 128-column group
                        if (lane == 0) bulk_wait_read<0>();
                        __syncwarp();
                        scword = 0;
                    }
                    const uint32_t w0 = cvt4(mul_bf16x2(h[0], inv), mul_bf16x2(h[1], inv)), w1 = cvt4(mul_bf16x2(h[2], inv), mul_bf16x2(h[3], inv));
                    const uint32_t w2 = cvt4(mul_bf16x2(h[4], inv), mul_bf16x2(h[5], inv)), w3 = cvt4(mul_bf16x2(h[6], inv), mul_bf16x2(h[7], inv));
                    const uint32_t w4 = cvt4(mul_bf16x2(h[8], inv), mul_bf16x2(h[9], inv)), w5 = cvt4(mul_bf16x2(h[10], inv), mul_bf16x2(h[11], inv));
                    const uint32_t w6 = cvt4(mul_bf16x2(h[12], inv), mul_bf16x2(h[13], inv)), w7 = cvt4(mul_bf16x2(h[14], inv), mul_bf16x2(h[15], inv));
                    const int cpos = (u & 3) * 2;                        // 16-byte chunk inside the 128-byte row
                    st_shared_v4(rowa + (((cpos + 0) ^ (lane & 7)) << 4), w0, w1, w2, w3);
                    st_shared_v4(rowa + (((cpos + 1) ^ (lane & 7)) << 4), w4, w5, w6, w7);
                    scword |= byte << ((u & 3) * 8);
                    if ((u & 3) == (acc ? 3 : 0)) {      // last unit of the group
                        fence_proxy_async_smem();
                        __syncwarp();
                        const int ctile = (col0 + (u & ~3) * 32) / 128;  // scale tile column
                        if (lane == 0 && !MX8_DBG(p, 4)) {
                            tma_store_2d(mc, col0 + (u & ~3) * 32, row0, stg);
                            bulk_commit();
                        }
                        if (row0 + lane < p.rows_cap && ctile * 128 < p.n_cols)
                            *reinterpret_cast<uint32_t*>(c_sc + (static_cast<size_t>(row0 / 128) * (p.n_cols / 128) + ctile) * 512 +
                                                         lane * 16 + q * 4) = scword;
                    }
                } else {
                    if ((s & 1) == 0) {
                        if (p.c_mode == 3) {
                            // combine fused into the epilogue: look up where this lane's row goes
                            if (s == 0) {
                                const int row = row0 + lane;
                                const int pr = p.sc_peer_rank[row];
                                sc_row = pr >= 0 ? p.sc_dst[pr] + static_cast<size_t>(p.sc_peer_token_idx[row]) * p.n_cols * 2 : nullptr;
                            }
                        } else if (lane == 0) {
                            bulk_wait_read<0>();
                        }
                        __syncwarp();
                    }
                    const int hh = u & 1;                        // which half of the 64-column chunk
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t w0 = pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
                        const uint32_t w1 = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
                        const uint32_t w2 = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
                        const uint32_t w3 = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
                        st_shared_v4(rowa + (((hh * 4 + j) ^ (lane & 7)) << 4), w0, w1, w2, w3);
                    }
                    if ((s & 1) && p.c_mode == 3) {
                        // staged 32 rows x 128 bytes -> the owners' buffers, four whole 128-byte row
                        // pieces per warp instruction (8 lanes per row)
                        __syncwarp();
                        const int cbyte = (col0 + (u & ~1) * 32) * 2 + (lane & 7) * 16;
                        const bool col_ok = col0 + (u & ~1) * 32 < p.n_cols;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int rr = 4 * i + (lane >> 3);
                            uint32_t v0, v1, v2, v3;
                            ld_shared_v4(stg + rr * 128 + (((lane & 7) ^ (rr & 7)) << 4), v0, v1, v2, v3);
                            const unsigned long long dp = __shfl_sync(0xFFFFFFFFu, reinterpret_cast<unsigned long long>(sc_row), rr);
                            if (dp && col_ok) *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(dp) + cbyte) = make_uint4(v0, v1, v2, v3);
                        }
                        __syncwarp();
                    } else if (s & 1) {
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0 && !MX8_DBG(p, 4)) {
                            tma_store_2d(mc, col0 + (u & ~1) * 32, row0, stg);
                            bulk_commit();
                        }
                    }
                }
            }
        }
        if (lane == 0) bulk_wait_all<0>();
    }

    // ---------------------------------------------------------------------- teardown
    if (*abort_flag) {
        // a wait gave up: let copies that may still be in flight land before shared memory goes away
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 1000000ull) __nanosleep(1000);
    }
    __syncwarp();
    tc_fence_before();
    if constexpr (CG == 2) cluster_sync_all(); else __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc<CG>(tmem_base, 512);
    }
}

#ifdef MX8_ABLATION
// process-wide ablation switches for timing studies (mx8_debug_set_gemm_ablation, exported by such a build only)
static int g_ablation_flags = 0;
#endif

struct Maps {
    CUtensorMap a, b, sfa, sfb, a2, b2, sfa2, sfb2, c, c2;
};

// tensor maps of one operand pair: A [a_rows][K], B [b_rows][K] and their scale tiles
// (K = bytes per row: the element count for E4M3, twice that for bf16 operands, which have no scales)
template <int CG>
static int build_operand_maps(CUtensorMap* ma, CUtensorMap* mb, CUtensorMap* msa, CUtensorMap* msb, const void* A,
                              const void* A_sc, const void* B, const void* B_sc, int a_rows, int b_rows, int K) {
    int rc;
    const uint64_t kb = static_cast<uint64_t>(K) / 128;
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(a_rows)};
        const uint64_t strides[1] = {static_cast<uint64_t>(K)};
        const uint32_t box[2] = {BK, 128};
        if ((rc = make_tmap(ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, A, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) != MX8_OK) return rc;
    }
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(b_rows)};
        const uint64_t strides[1] = {static_cast<uint64_t>(K)};
        const uint32_t box[2] = {BK, static_cast<uint32_t>(Cfg<CG>::B_ROWS)};
        if ((rc = make_tmap(mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, B, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) != MX8_OK) return rc;
    }
    if (!A_sc) {          // bf16 operands: the kernel never touches the scale maps
        *msa = *ma;
        *msb = *mb;
        return MX8_OK;
    }
    {
        // scale tiles [rows/128][K/128][512 bytes] seen as 32-bit words so one box row is a whole tile
        const uint64_t dims[3] = {128, kb, static_cast<uint64_t>(a_rows) / 128};
        const uint64_t strides[2] = {512, 512 * kb};
        const uint32_t box[3] = {128, 1, 1};
        if ((rc = make_tmap(msa, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, A_sc, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE)) != MX8_OK) return rc;
    }
    {
        const uint64_t dims[3] = {128, kb, static_cast<uint64_t>(b_rows) / 128};
        const uint64_t strides[2] = {512, 512 * kb};
        const uint32_t box[3] = {128, 1, 2};
        if ((rc = make_tmap(msb, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, B_sc, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE)) != MX8_OK) return rc;
    }
    return MX8_OK;
}

static int build_c_map(CUtensorMap* mc, void* Cp, int c_rows, int N, int c_dtype) {
    // C rows are 128 bytes wide in the staging buffer: 64 bf16, 32 float or 128 E4M3 columns
    const int esz = c_dtype == MX8_C_F32 ? 4 : (c_dtype == MX8_C_MXFP8 ? 1 : 2);
    const CUtensorMapDataType dt = c_dtype == MX8_C_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : (c_dtype == MX8_C_MXFP8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
    const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(c_rows)};
    const uint64_t strides[1] = {static_cast<uint64_t>(N) * esz};
    const uint32_t box[2] = {static_cast<uint32_t>(128 / esz), 32};
    return make_tmap(mc, dt, 2, Cp, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

template <int CG, bool F16, bool A16 = false, bool SW = false>
static int max_grid() {
    // CTAs that can be resident at once (cluster placement included), cached per device
    static std::atomic<int> cached[64];
    int dev = 0;
    cudaGetDevice(&dev);
    dev &= 63;
    if (const int have = cached[dev].load(std::memory_order_acquire)) return have;
    auto kern = gemm_kernel<CG, F16, A16, SW>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<CG, A16>::dynamic);
    if (e != cudaSuccess) {
        note_cuda_error("cudaFuncSetAttribute(gemm)", cudaGetErrorString(e));
        return 0;
    }
    int n = sm_count();
    if (CG == 2) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(n & ~1));
        cfg.blockDim = dim3(Cfg<CG, A16>::threads);
        cfg.dynamicSmemBytes = Cfg<CG, A16>::dynamic;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 2;
        at[0].val.clusterDim.y = 1;
        at[0].val.clusterDim.z = 1;
        cfg.attrs = at;
        cfg.numAttrs = 1;
        int clusters = 0;
        e = cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg);
        if (e != cudaSuccess || clusters <= 0) {
            note_cuda_error("cudaOccupancyMaxActiveClusters", cudaGetErrorString(e));
            cudaGetLastError();
            clusters = n / 2;
        }
        n = clusters * 2;
    }
    cached[dev].store(n, std::memory_order_release);
    return n;
}

struct Grouping {
    void* c_sc = nullptr;            // scale tiles of C (MX8_C_MXFP8)
    const int* rows_dev = nullptr;   // device count of rows present
    const int* row_begin_dev = nullptr; // device: first row of the window
    const int* group_rows = nullptr; // device rows per group
    int num_groups = 0;
    const int* peer_rank = nullptr;  // scatter epilogue
    const int* peer_token_idx = nullptr;
    void* const* dst = nullptr;
    int world = 0;
    // second operand pair accumulated into the same output: C = A B^T + A2 B2^T
    const void *A2 = nullptr, *A2_sc = nullptr, *B2 = nullptr, *B2_sc = nullptr;
    int K2 = 0;
    // weight-gradient form: A is A^T [M][K], B is B^T [N][K] with K = all rows; one C [M][N] per group
    bool wgrad = false;
    // pair launch: a second product of the same A with B_pair (same shape as B) into C_pair (same type as C)
    const void *B_pair = nullptr, *B_pair_sc = nullptr;
    void *C_pair = nullptr, *C_pair_sc = nullptr;
    // SwiGLU form (B = gate weights, B_pair = up weights): gate, gate_sc, up, up_sc, hidden, hidden_sc, hidden_t, hidden_t_sc
    void* sw[8] = {};
};

template <int CG, bool F16 = false, bool A16 = false, bool SW = false>
static int run(const void* A, const void* A_sc, const void* B, const void* B_sc, void* Cp, int M, int N, int K,
               int c_dtype, int max_ctas, const Grouping& gr, cudaStream_t stream) {
    Maps m;
    const int groups = gr.num_groups > 0 ? gr.num_groups : 1;
    const int b_rows = gr.wgrad ? N : groups * N;              // wgrad: B^T is one [N][K] matrix
    const int c_rows = gr.wgrad ? groups * M : M;
    int rc;
    if constexpr (A16) {
        // A is bf16 [M][K]: its rows are 2K bytes and arrive in 128-byte-wide boxes; there are no A scale tiles
        rc = build_operand_maps<CG>(&m.a, &m.b, &m.sfa, &m.sfb, B, B_sc, B, B_sc, b_rows, b_rows, K);
        if (rc != MX8_OK) return rc;
        const uint64_t dims[2] = {2 * static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
        const uint64_t strides[1] = {2 * static_cast<uint64_t>(K)};
        const uint32_t box[2] = {BK, 128};
        rc = make_tmap(&m.a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, A, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    } else {
        rc = build_operand_maps<CG>(&m.a, &m.b, &m.sfa, &m.sfb, A, A_sc, B, B_sc, M, b_rows, K);
    }
    if (rc != MX8_OK) return rc;
    if (gr.K2 > 0) rc = build_operand_maps<CG>(&m.a2, &m.b2, &m.sfa2, &m.sfb2, gr.A2, gr.A2_sc, gr.B2, gr.B2_sc, M, b_rows, gr.K2);
    else if (gr.B_pair) rc = build_operand_maps<CG>(&m.a2, &m.b2, &m.sfa2, &m.sfb2, A, A_sc, gr.B_pair, gr.B_pair_sc, M, b_rows, K);
    else { m.a2 = m.a; m.b2 = m.b; m.sfa2 = m.sfa; m.sfb2 = m.sfb; }
    if (rc != MX8_OK) return rc;
    if ((rc = build_c_map(&m.c, Cp, c_rows, N, c_dtype)) != MX8_OK) return rc;
    if (gr.C_pair) rc = build_c_map(&m.c2, gr.C_pair, c_rows, N, c_dtype);
    else m.c2 = m.c;
    if (rc != MX8_OK) return rc;
    if constexpr (SW) {
        // a tile takes one scale tile of the gate weights and one of the up weights: maps with a box of one tile
        const uint64_t kb = static_cast<uint64_t>(K) / 128;
        const uint64_t dims[3] = {128, kb, static_cast<uint64_t>(b_rows) / 128};
        const uint64_t strides[2] = {512, 512 * kb};
        const uint32_t box[3] = {128, 1, 1};
        if ((rc = make_tmap(&m.sfb, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, B_sc, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE)) != MX8_OK) return rc;
        if ((rc = make_tmap(&m.sfb2, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, gr.B_pair_sc, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE)) != MX8_OK) return rc;
    }
    Params p{};
    p.c_sc = static_cast<uint8_t*>(gr.c_sc);
    p.n_cols = N;
    p.rows_cap = c_rows;
    p.k_steps2 = gr.K2 / BK;
    p.wgrad = gr.wgrad ? 1 : 0;
    p.group_c_rows = M;
    p.rows_dev = gr.rows_dev;
    p.row_begin_dev = gr.row_begin_dev;
    p.group_rows = gr.group_rows;
    p.num_groups = gr.num_groups;
    p.group_b_rows = N;
    p.sc_peer_rank = gr.peer_rank;
    p.sc_peer_token_idx = gr.peer_token_idx;
    for (int i = 0; i < gr.world && i < 16; ++i) p.sc_dst[i] = static_cast<uint8_t*>(gr.dst[i]);
    p.tiles_m = (M + 128 * CG - 1) / (128 * CG);
    p.tiles_n = (N + BN - 1) / BN;
    if constexpr (SW) {
        p.tiles_n = N / (BN / 2);                                  // a tile is 128 output columns of gate and of up
        uint8_t** dst[8] = {&p.sw_gate, &p.sw_gate_sc, &p.sw_up, &p.sw_up_sc, &p.sw_h, &p.sw_h_sc, &p.sw_ht, &p.sw_ht_sc};
        for (int i = 0; i < 8; ++i) *dst[i] = static_cast<uint8_t*>(gr.sw[i]);
    } else if (gr.B_pair) {
        p.pair_tiles_n = p.tiles_n;
        p.tiles_n *= 2;
        p.c_sc2 = static_cast<uint8_t*>(gr.C_pair_sc);
    }
    p.k_steps = gr.wgrad ? 0 : K / BK;
    p.group_m = 16;
    p.c_mode = SW ? 4 : (gr.dst ? 3 : c_dtype);
#ifdef MX8_ABLATION
    p.dbg = gr.wgrad ? (g_ablation_flags & ~128) : g_ablation_flags;   // the weight-gradient form cannot drop the epilogue wait
#endif
    p.status = device_status_ptr();
    if (!p.status) return MX8_ERR_CUDA;
    int grid = max_grid<CG, F16, A16, SW>();
    if (grid <= 0) return MX8_ERR_CUDA;
    if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
    const int tiles = p.tiles_m * p.tiles_n * (gr.wgrad ? groups : 1);
    if (grid > tiles * CG) grid = tiles * CG;
    grid = (grid / CG) * CG;
    if (grid <= 0) grid = CG;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(Cfg<CG, A16>::threads);
    cfg.dynamicSmemBytes = Cfg<CG, A16>::dynamic;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = CG;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_kernel<CG, F16, A16, SW>, m.a, m.b, m.sfa, m.sfb, m.a2, m.b2, m.sfa2, m.sfb2, m.c, m.c2, p);
    if (e != cudaSuccess) {
        note_cuda_error("gemm launch", cudaGetErrorString(e));
        return MX8_ERR_CUDA;
    }
    return MX8_OK;
}

}  // namespace gemm
}  // namespace mx8

extern "C" int mx8_gemm_ex(const void* A, const void* A_sc, const void* B, const void* B_sc, void* C, int M, int N, int K,
                           int c_dtype, int cta_group, int max_ctas, void* stream) {
    using namespace mx8;
    if (!A || !A_sc || !B || !B_sc || !C) return MX8_ERR_ARG;
    if (c_dtype != MX8_C_BF16 && c_dtype != MX8_C_F32) return MX8_ERR_ARG;
    if (cta_group < 0 || cta_group > 2 || max_ctas < 0) return MX8_ERR_ARG;
    if (M <= 0 || N <= 0 || K <= 0 || M % 128 || N % 128 || K % 128) return MX8_ERR_SHAPE;
    if (!aligned16(A) || !aligned16(A_sc) || !aligned16(B) || !aligned16(B_sc) || !aligned16(C)) return MX8_ERR_ALIGN;
    int rc = check_device_sm100();
    if (rc != MX8_OK) return rc;
    if (cta_group == 0) cta_group = (M <= 128) ? 1 : 2;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const gemm::Grouping none;
    if (cta_group == 2) return gemm::run<2>(A, A_sc, B, B_sc, C, M, N, K, c_dtype, max_ctas, none, st);
    return gemm::run<1>(A, A_sc, B, B_sc, C, M, N, K, c_dtype, max_ctas, none, st);
}

extern "C" int mx8_gemm_grouped(const void* A, const void* A_sc, const void* B, const void* B_sc, void* C, void* C_sc,
                                int M, int N, int K, int c_dtype, const void* num_rows, const void* group_rows,
                                int num_groups, void* stream) {
    return mx8_gemm_grouped_window(A, A_sc, B, B_sc, C, C_sc, M, N, K, c_dtype, num_rows, group_rows, num_groups, nullptr, stream);
}

extern "C" int mx8_gemm_grouped_window(const void* A, const void* A_sc, const void* B, const void* B_sc, void* C, void* C_sc,
                                       int M, int N, int K, int c_dtype, const void* num_rows, const void* group_rows,
                                       int num_groups, const mx8_window* window, void* stream) {
    using namespace mx8;
    if (!A || !A_sc || !B || !B_sc || !C) return MX8_ERR_ARG;
    if (c_dtype != MX8_C_BF16 && c_dtype != MX8_C_F32 && c_dtype != MX8_C_MXFP8) return MX8_ERR_ARG;
    if ((c_dtype == MX8_C_MXFP8) != (C_sc != nullptr)) return MX8_ERR_ARG;
    if (num_groups < 0 || (num_groups > 0 && !group_rows)) return MX8_ERR_ARG;
    if (num_groups > gemm::MAX_GROUPS) {
        note_cuda_error("mx8_gemm_grouped", "more than 256 groups in one call");
        return MX8_ERR_LIMIT;
    }
    if (M <= 0 || N <= 0 || K <= 0 || M % 128 || N % 128 || K % 128) return MX8_ERR_SHAPE;
    if (num_groups > 0 && (M % 256 || N % 256)) return MX8_ERR_SHAPE;     // groups are whole 256-row / 256-column tiles
    if (!aligned16(A) || !aligned16(A_sc) || !aligned16(B) || !aligned16(B_sc) || !aligned16(C) || !aligned16(C_sc)) return MX8_ERR_ALIGN;
    int rc = check_device_sm100();
    if (rc != MX8_OK) return rc;
    gemm::Grouping gr;
    gr.c_sc = C_sc;
    gr.rows_dev = static_cast<const int*>(num_rows);
    gr.group_rows = static_cast<const int*>(group_rows);
    gr.num_groups = num_groups;
    int max_ctas = 0;
    if (window) {
        if (window->row_begin) gr.row_begin_dev = static_cast<const int*>(window->row_begin);
        if (window->row_end) gr.rows_dev = static_cast<const int*>(window->row_end);
        max_ctas = window->max_sms > 0 ? window->max_sms : 0;
    }
    return gemm::run<2>(A, A_sc, B, B_sc, C, M, N, K, c_dtype, max_ctas, gr, static_cast<cudaStream_t>(stream));
}

// Two grouped products of the same A in one launch (the MoE layer's gate and up projections): column tiles of
// both share the persistent schedule, so there is one tail and the A panels are fetched once for both.
extern "C" int mx8_gemm_grouped_pair_window(const void* A, const void* A_sc, const void* B1, const void* B1_sc, const void* B2,
                                            const void* B2_sc, void* C1, void* C1_sc, void* C2, void* C2_sc, int M, int N, int K,
                                            int c_dtype, const void* num_rows, const void* group_rows, int num_groups,
                                            const mx8_window* window, void* stream) {
    using namespace mx8;
    if (!A || !A_sc || !B1 || !B1_sc || !B2 || !B2_sc || !C1 || !C2) return MX8_ERR_ARG;
    if (c_dtype != MX8_C_BF16 && c_dtype != MX8_C_F32 && c_dtype != MX8_C_MXFP8) return MX8_ERR_ARG;
    if ((c_dtype == MX8_C_MXFP8) != (C1_sc != nullptr) || (C1_sc == nullptr) != (C2_sc == nullptr)) return MX8_ERR_ARG;
    if (num_groups < 0 || (num_groups > 0 && !group_rows)) return MX8_ERR_ARG;
    if (num_groups > gemm::MAX_GROUPS) {
        note_cuda_error("mx8_gemm_grouped_pair", "more than 256 groups in one call");
        return MX8_ERR_LIMIT;
    }
    if (M <= 0 || N <= 0 || K <= 0 || M % 128 || N % 256 || K % 128) return MX8_ERR_SHAPE;     // whole column tiles per product
    if (num_groups > 0 && M % 256) return MX8_ERR_SHAPE;
    if (!aligned16(A) || !aligned16(A_sc) || !aligned16(B1) || !aligned16(B1_sc) || !aligned16(B2) || !aligned16(B2_sc) ||
        !aligned16(C1) || !aligned16(C1_sc) || !aligned16(C2) || !aligned16(C2_sc)) return MX8_ERR_ALIGN;
    int rc = check_device_sm100();
    if (rc != MX8_OK) return rc;
    gemm::Grouping gr;
    gr.c_sc = C1_sc;
    gr.rows_dev = static_cast<const int*>(num_rows);
    gr.group_rows = static_cast<const int*>(group_rows);
    gr.num_groups = num_groups;
    gr.B_pair = B2; gr.B_pair_sc = B2_sc; gr.C_pair = C2; gr.C_pair_sc = C2_sc;
    int max_ctas = 0;
    if (window) {
        if (window->row_begin) gr.row_begin_dev = static_cast<const int*>(window->row_begin);
        if (window->row_end) gr.rows_dev = static_cast<const int*>(window->row_end);
        max_ctas = window->max_sms > 0 ? window->max_sms : 0;
    }
    return gemm::run<2>(A, A_sc, B1, B1_sc, C1, M, N, K, c_dtype, max_ctas, gr, static_cast<cudaStream_t>(stream));
}

// Gate and up projections with SwiGLU and all four quantizations in the epilogue (see swiglu_epilogue).
extern "C" int mx8_gemm_grouped_swiglu_window(const void* A, const void* A_sc, const void* B_gate, const void* B_gate_sc,
                                              const void* B_up, const void* B_up_sc, void* gate_fp8, void* gate_sc, void* up_fp8,
                                              void* up_sc, void* hidden_fp8, void* hidden_sc, void* hidden_fp8_t, void* hidden_sc_t,
                                              int M, int N, int K, const void* num_rows, const void* group_rows, int num_groups,
                                              const mx8_window* window, void* stream) {
    using namespace mx8;
    const void* const all[] = {A, A_sc, B_gate, B_gate_sc, B_up, B_up_sc, gate_fp8, gate_sc, up_fp8, up_sc, hidden_fp8, hidden_sc,
                               hidden_fp8_t, hidden_sc_t};
    for (const void* q : all) {
        if (!q) return MX8_ERR_ARG;
        if (!aligned16(q)) return MX8_ERR_ALIGN;
    }
    if (num_groups < 0 || (num_groups > 0 && !group_rows)) return MX8_ERR_ARG;
    if (num_groups > gemm::MAX_GROUPS) {
        note_cuda_error("mx8_gemm_grouped_swiglu", "more than 256 groups in one call");
        return MX8_ERR_LIMIT;
    }
    if (M <= 0 || N <= 0 || K <= 0 || M % 256 || N % 128 || K % 128) return MX8_ERR_SHAPE;
    int rc = check_device_sm100();
    if (rc != MX8_OK) return rc;
    gemm::Grouping gr;
    gr.rows_dev = static_cast<const int*>(num_rows);
    gr.group_rows = static_cast<const int*>(group_rows);
    gr.num_groups = num_groups;
    gr.B_pair = B_up;
    gr.B_pair_sc = B_up_sc;
    void* const outs[8] = {gate_fp8, gate_sc, up_fp8, up_sc, hidden_fp8, hidden_sc, hidden_fp8_t, hidden_sc_t};
    for (int i = 0; i < 8; ++i) gr.sw[i] = outs[i];
    int max_ctas = 0;
    if (window) {
        if (window->row_begin) gr.row_begin_dev = static_cast<const int*>(window->row_begin);
        if (window->row_end) gr.rows_dev = static_cast<const int*>(window->row_end);
        max_ctas = window->max_sms > 0 ? window->max_sms : 0;
    }
    // the C tensor map is unused by this epilogue; A stands in so that the map encodes
    return gemm::run<2, false, false, true>(A, A_sc, B_gate, B_gate_sc, const_cast<void*>(A), M, N, K, MX8_C_MXFP8, max_ctas, gr,
                                            static_cast<cudaStream_t>(stream));
}

extern "C" int mx8_gemm(const void* A, const void* A_sc, const void* B, const void* B_sc, void* C, int M, int N, int K,
                        int c_dtype, void* stream) {
    return mx8_gemm_ex(A, A_sc, B, B_sc, C, M, N, K, c_dtype, 0, 0, stream);
}

extern "C" int mx8_gemm_grouped_scatter(const void* A, const void* A_sc, const void* B, const void* B_sc, int M, int N, int K,
                                        const void* num_rows, const void* group_rows, int num_groups, const void* peer_rank,
                                        const void* peer_token_idx, void* const* dst_ptrs, int world, void* stream) {
    using namespace mx8;
    if (!A || !A_sc || !B || !B_sc || !num_rows || !peer_rank || !peer_token_idx || !dst_ptrs) return MX8_ERR_ARG;
    if (world <= 0 || world > 16 || num_groups < 0 || (num_groups > 0 && !group_rows)) return MX8_ERR_ARG;
    if (num_groups > gemm::MAX_GROUPS) {
        note_cuda_error("mx8_gemm_grouped_scatter", "more than 256 groups in one call");
        return MX8_ERR_LIMIT;
    }
    if (M <= 0 || N <= 0 || K <= 0 || M % 256 || N % 128 || K % 128 || (num_groups > 0 && N % 256)) return MX8_ERR_SHAPE;
    if (!aligned16(A) || !aligned16(A_sc) || !aligned16(B) || !aligned16(B_sc)) return MX8_ERR_ALIGN;
    for (int r = 0; r < world; ++r)
        if (!dst_ptrs[r] || !aligned16(dst_ptrs[r])) return MX8_ERR_ALIGN;
    int rc = check_device_sm100();
    if (rc != MX8_OK) return rc;
    gemm::Grouping gr;
    gr.rows_dev = static_cast<const int*>(num_rows);
    gr.group_rows = static_cast<const int*>(group_rows);
    gr.num_groups = num_groups;
    gr.peer_rank = static_cast<const int*>(peer_rank);
    gr.peer_token_idx = static_cast<const int*>(peer_token_idx);
    gr.dst = dst_ptrs;
    gr.world = world;
    // the C tensor map is unused by this epilogue; A stands in so that the map encodes
    return gemm::run<2>(A, A_sc, B, B_sc, const_cast<void*>(A), M, N, K, MX8_C_MXFP8, 0, gr, static_cast<cudaStream_t>(stream));
}

// bf16 operands (shared expert of the MoE layer): the same kernel with kind::f16 MMAs and no scale
// tiles.  Rows are handed to the common launcher as bytes (2 per element).
extern "C" int mx8_gemm_bf16_dual(const void* A1, const void* B1, const void* A2, const void* B2, void* C, int M, int N,
                                  int K1, int K2, int c_dtype, void* stream) {
    using namespace mx8;
    if (!A1 || !B1 || !C || (K2 > 0 && (!A2 || !B2))) return MX8_ERR_ARG;
    if (c_dtype != MX8_C_BF16 && c_dtype != MX8_C_F32) return MX8_ERR_ARG;
    if (M <= 0 || N <= 0 || K1 <= 0 || K2 < 0 || M % 128 || N % 128 || K1 % 64 || K2 % 64) return MX8_ERR_SHAPE;
    if (!aligned16(A1) || !aligned16(B1) || !aligned16(C) || !aligned16(A2) || !aligned16(B2)) return MX8_ERR_ALIGN;
    int rc = check_device_sm100();
    if (rc != MX8_OK) return rc;
    gemm::Grouping gr;
    if (K2 > 0) {
        gr.A2 = A2;
        gr.B2 = B2;
        gr.K2 = 2 * K2;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (M <= 128) return gemm::run<1, true>(A1, nullptr, B1, nullptr, C, M, N, 2 * K1, c_dtype, 0, gr, st);
    return gemm::run<2, true>(A1, nullptr, B1, nullptr, C, M, N, 2 * K1, c_dtype, 0, gr, st);
}

extern "C" int mx8_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int c_dtype, void* stream) {
    return mx8_gemm_bf16_dual(A, B, nullptr, nullptr, C, M, N, K, 0, c_dtype, stream);
}

// A bf16, quantized row-wise inside the main loop (see the converter role in the kernel)
extern "C" int mx8_gemm_a_bf16_fused(const void* A_bf16, const void* B, const void* B_sc, void* C, int M, int N, int K, int c_dtype,
                                     void* stream) {
    using namespace mx8;
    if (!A_bf16 || !B || !B_sc || !C) return MX8_ERR_ARG;
    if (c_dtype != MX8_C_BF16 && c_dtype != MX8_C_F32) return MX8_ERR_ARG;
    if (M <= 0 || N <= 0 || K <= 0 || M % 128 || N % 128 || K % 128) return MX8_ERR_SHAPE;
    if (!aligned16(A_bf16) || !aligned16(B) || !aligned16(B_sc) || !aligned16(C)) return MX8_ERR_ALIGN;
    int rc = check_device_sm100();
    if (rc != MX8_OK) return rc;
    const gemm::Grouping none;
    return gemm::run<2, false, true>(A_bf16, nullptr, B, B_sc, C, M, N, K, c_dtype, 0, none, static_cast<cudaStream_t>(stream));
}

#ifdef MX8_ABLATION
extern "C" MX8_API int mx8_debug_set_gemm_ablation(int flags) {
    const int old = mx8::gemm::g_ablation_flags;
    mx8::gemm::g_ablation_flags = flags;
    return old;
}
#endif

extern "C" int mx8_gemm_grouped_dual(const void* A1, const void* A1_sc, const void* B1, const void* B1_sc, const void* A2,
                                     const void* A2_sc, const void* B2, const void* B2_sc, void* C, int M, int N, int K1, int K2,
                                     const void* num_rows, const void* group_rows, int num_groups, void* stream) {
    return mx8_gemm_grouped_dual_window(A1, A1_sc, B1, B1_sc, A2, A2_sc, B2, B2_sc, C, M, N, K1, K2, num_rows, group_rows, num_groups,
                                        nullptr, stream);
}

extern "C" int mx8_gemm_grouped_dual_window(const void* A1, const void* A1_sc, const void* B1, const void* B1_sc, const void* A2,
                                            const void* A2_sc, const void* B2, const void* B2_sc, void* C, int M, int N, int K1,
                                            int K2, const void* num_rows, const void* group_rows, int num_groups,
                                            const mx8_window* window, void* stream) {
    using namespace mx8;
    if (!A1 || !A1_sc || !B1 || !B1_sc || !A2 || !A2_sc || !B2 || !B2_sc || !C) return MX8_ERR_ARG;
    if (num_groups < 0 || (num_groups > 0 && !group_rows)) return MX8_ERR_ARG;
    if (num_groups > gemm::MAX_GROUPS) {
        note_cuda_error("mx8_gemm_grouped_dual", "more than 256 groups in one call");
        return MX8_ERR_LIMIT;
    }
    if (M <= 0 || N <= 0 || K1 <= 0 || K2 <= 0 || M % 128 || N % 128 || K1 % 128 || K2 % 128) return MX8_ERR_SHAPE;
    if (num_groups > 0 && (M % 256 || N % 256)) return MX8_ERR_SHAPE;
    if (!aligned16(A1) || !aligned16(A1_sc) || !aligned16(B1) || !aligned16(B1_sc) || !aligned16(A2) || !aligned16(A2_sc) ||
        !aligned16(B2) || !aligned16(B2_sc) || !aligned16(C)) return MX8_ERR_ALIGN;
    int rc = check_device_sm100();
    if (rc != MX8_OK) return rc;
    gemm::Grouping gr;
    gr.rows_dev = static_cast<const int*>(num_rows);
    gr.group_rows = static_cast<const int*>(group_rows);
    gr.num_groups = num_groups;
    gr.A2 = A2; gr.A2_sc = A2_sc; gr.B2 = B2; gr.B2_sc = B2_sc; gr.K2 = K2;
    int max_ctas = 0;
    if (window) {
        if (window->row_begin) gr.row_begin_dev = static_cast<const int*>(window->row_begin);
        if (window->row_end) gr.rows_dev = static_cast<const int*>(window->row_end);
        max_ctas = window->max_sms > 0 ? window->max_sms : 0;
    }
    return gemm::run<2>(A1, A1_sc, B1, B1_sc, C, M, N, K1, MX8_C_BF16, max_ctas, gr, static_cast<cudaStream_t>(stream));
}

extern "C" int mx8_gemm_wgrad(const void* A_t, const void* A_t_sc, const void* B_t, const void* B_t_sc, void* C, int M, int N,
                              int rows, const void* group_rows, int num_groups, void* stream) {
    using namespace mx8;
    if (!A_t || !A_t_sc || !B_t || !B_t_sc || !C || !group_rows) return MX8_ERR_ARG;
    if (num_groups <= 0) return MX8_ERR_ARG;
    if (num_groups > gemm::MAX_GROUPS) {
        note_cuda_error("mx8_gemm_wgrad", "more than 256 groups in one call");
        return MX8_ERR_LIMIT;
    }
    if (M <= 0 || N <= 0 || rows <= 0 || M % 256 || N % 128 || rows % 128) return MX8_ERR_SHAPE;
    if (!aligned16(A_t) || !aligned16(A_t_sc) || !aligned16(B_t) || !aligned16(B_t_sc) || !aligned16(C)) return MX8_ERR_ALIGN;
    int rc = check_device_sm100();
    if (rc != MX8_OK) return rc;
    gemm::Grouping gr;
    gr.group_rows = static_cast<const int*>(group_rows);
    gr.num_groups = num_groups;
    gr.wgrad = true;
    return gemm::run<2>(A_t, A_t_sc, B_t, B_t_sc, C, M, N, rows, MX8_C_BF16, 0, gr, static_cast<cudaStream_t>(stream));
}
