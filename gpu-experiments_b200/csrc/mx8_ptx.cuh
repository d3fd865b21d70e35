// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (cp.async.bulk[.tensor]), tcgen05 and
// the fences between them.  Every wait is bounded: after a time limit it records a status
// code and returns false so the calling role can unwind instead of spinning forever.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace mx8 {

// Device-side status codes recorded when a bounded wait gives up (0 = healthy).
enum : int {
    DEV_OK = 0,
    DEV_TIMEOUT_FULL = 1,      // consumer waited for a TMA-filled stage
    DEV_TIMEOUT_EMPTY = 2,     // producer waited for a stage to be released
    DEV_TIMEOUT_TMEM_FULL = 3, // epilogue waited for an accumulator
    DEV_TIMEOUT_TMEM_FREE = 4, // MMA issuer waited for the epilogue to drain
    DEV_TIMEOUT_SELFTEST = 8,  // the wait of mx8_selftest_bounded_wait, which nothing ever satisfies
};

#ifndef MX8_WAIT_LIMIT_NS
#define MX8_WAIT_LIMIT_NS 2000000000ull   // 2 s per wait
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t num_clusters_x() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
    return r;
}
// shared::cta address of this CTA -> shared::cluster address of the same offset in CTA `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// arrive on a barrier that may live in another CTA of the cluster (address from map_to_cta)
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Acquire at CTA scope: enough for barriers completed by TMA byte counts, by tcgen05.commit or by
// threads of this CTA.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Acquire at cluster scope: for barriers that threads of the peer CTA arrive on with release.cluster.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Shared by all roles of a CTA: set once a wait gave up, polled by every other wait.
struct AbortCtl {
    volatile int* smem_flag;   // per-CTA word in shared memory
    int* global_status;        // device word the host reads after the launch
};

// Bounded wait.  Returns false after limit_ns (MX8_WAIT_LIMIT_NS unless the caller says otherwise; recording `code`) or as soon as
// another role of this CTA has given up.  CLUSTER selects the acquire scope (see above).
template <bool CLUSTER = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const AbortCtl& ab, int code,
                                          uint64_t limit_ns = MX8_WAIT_LIMIT_NS) {
    auto probe = [&]() { return CLUSTER ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity); };
    if (probe()) return true;
    uint64_t t0 = 0;
    for (uint32_t spins = 1;; ++spins) {
        if (probe()) return true;
        if ((spins & 0x3FF) == 0) {
            if (*ab.smem_flag) return false;
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_ns) {
                *ab.smem_flag = 1;
                atomicCAS(ab.global_status, 0, code);
                return false;
            }
        }
    }
}

// ------------------------------------------------------------------ fences
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ------------------------------------------------------------------ TMA loads (each CTA fetches its own tiles)
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, int x, int y, int z, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(z), "r"(bar)
        : "memory");
}
// CTA-pair form: data lands in the issuing CTA's shared memory, completion bytes are
// signalled on a barrier that may belong to the peer CTA (shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, int x, int y, uint32_t bar_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(bar_cluster)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* m, int x, int y, int z, uint32_t bar_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(z), "r"(bar_cluster)
        : "memory");
}

// contiguous bytes, global (local or a peer GPU's mapped memory) -> this CTA's shared memory;
// both addresses 16-byte aligned, size a multiple of 16
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* gsrc, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(bar)
                 : "memory");
}

// ------------------------------------------------------------------ TMA stores
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, int x, int y, uint32_t src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(src)
                 : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, int x, int y, int z, int w, uint32_t src) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%1, %2, %3, %4}], [%5];"
                 ::"l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(z), "r"(w), "r"(src)
                 : "memory");
}
// contiguous bytes, shared -> global; both addresses 16-byte aligned, size a multiple of 16
__device__ __forceinline__ void bulk_store_1d(void* gdst, uint32_t src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 ::"l"(reinterpret_cast<uint64_t>(gdst)), "r"(src), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_all() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ------------------------------------------------------------------ tcgen05: TMEM management
template <int CG>
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    if constexpr (CG == 2)
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
    else
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
template <int CG>
__device__ __forceinline__ void tmem_relinquish() {
    if constexpr (CG == 2) asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    else asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
template <int CG>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    if constexpr (CG == 2) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// ------------------------------------------------------------------ tcgen05: descriptors
// Shared-memory matrix descriptor, K-major operand stored as rows of 128 bytes under the
// 128-byte swizzle (what a SWIZZLE_128B tensor map writes): 8-row atoms of 1024 bytes, so the
// stride between atoms is 1024; the leading offset is unused for this layout.  Advancing along
// K by 32 bytes adds 2 to the (address >> 4) field.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    return static_cast<uint64_t>((addr & 0x3FFFFu) >> 4)
         | (static_cast<uint64_t>(1) << 16)
         | (static_cast<uint64_t>(1024 >> 4) << 32)
         | (static_cast<uint64_t>(1) << 46)
         | (static_cast<uint64_t>(2) << 61);
}
// Descriptor of one 512-byte scale tile (32 rows of 16 bytes, no swizzle) for tcgen05.cp.
__device__ __forceinline__ uint64_t smem_desc_scales(uint32_t addr) {
    return static_cast<uint64_t>((addr & 0x3FFFFu) >> 4)
         | (static_cast<uint64_t>(128 >> 4) << 16)
         | (static_cast<uint64_t>(128 >> 4) << 32)
         | (static_cast<uint64_t>(1) << 46);
}
// Instruction descriptor for kind::mxf8f6f4 block-scaled MMA, A and B E4M3 K-major, UE8M0 scales.
__host__ __device__ constexpr uint32_t idesc_mxf8(int M, int N, int sf_id) {
    return (static_cast<uint32_t>(sf_id) << 4)      // B scale byte within the TMEM word
         | (static_cast<uint32_t>(N >> 3) << 17)
         | (1u << 23)                                // scale type UE8M0
         | (static_cast<uint32_t>(M >> 4) << 24)
         | (static_cast<uint32_t>(sf_id) << 29);    // A scale byte within the TMEM word
}

// Instruction descriptor for kind::f16 with bf16 A and B (K-major) and an fp32 accumulator.
__host__ __device__ constexpr uint32_t idesc_bf16(int M, int N) {
    return (1u << 4)                                 // D format f32
         | (1u << 7) | (1u << 10)                    // A and B format bf16
         | (static_cast<uint32_t>(N >> 3) << 17)
         | (static_cast<uint32_t>(M >> 4) << 24);
}

// The same descriptors split into 32-bit halves: the high word is a constant, the low word carries
// the address field, so advancing to another stage or K offset is one 32-bit add.
constexpr uint32_t DESC_SW128_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
constexpr uint32_t DESC_SCALES_HI = (128u >> 4) | (1u << 14);
__device__ __forceinline__ uint32_t desc_sw128_lo(uint32_t addr) { return (addr >> 4) | (1u << 16); }
__device__ __forceinline__ uint32_t desc_scales_lo(uint32_t addr) { return (addr >> 4) | ((128u >> 4) << 16); }

// ------------------------------------------------------------------ tcgen05: copy, MMA, commit, load
template <int CG>
__device__ __forceinline__ void tc_cp_scales_lo(uint32_t taddr, uint32_t desc_lo) {
    if constexpr (CG == 2)
        asm volatile("{\n\t.reg .b64 d;\n\tmov.b64 d, {%1, %2};\n\ttcgen05.cp.cta_group::2.32x128b.warpx4 [%0], d;\n\t}"
                     ::"r"(taddr), "r"(desc_lo), "n"(DESC_SCALES_HI) : "memory");
    else
        asm volatile("{\n\t.reg .b64 d;\n\tmov.b64 d, {%1, %2};\n\ttcgen05.cp.cta_group::1.32x128b.warpx4 [%0], d;\n\t}"
                     ::"r"(taddr), "r"(desc_lo), "n"(DESC_SCALES_HI) : "memory");
}
// ACC: 0 = overwrite the accumulator, 1 = accumulate, 2 = decide at run time from `acc`
template <int CG, int ACC>
__device__ __forceinline__ void tc_mma_mxf8_lo(uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                               uint32_t sfa, uint32_t sfb, uint32_t acc = 1) {
    if constexpr (CG == 2)
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
            "mov.b64 da, {%1, %7};\n\tmov.b64 db, {%2, %7};\n\tsetp.ne.u32 p, %6, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], da, db, %3, [%4], [%5], p;\n\t}"
            ::"r"(d), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(sfa), "r"(sfb), "r"(ACC == 2 ? acc : static_cast<uint32_t>(ACC)), "n"(DESC_SW128_HI)
            : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
            "mov.b64 da, {%1, %7};\n\tmov.b64 db, {%2, %7};\n\tsetp.ne.u32 p, %6, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], da, db, %3, [%4], [%5], p;\n\t}"
            ::"r"(d), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(sfa), "r"(sfb), "r"(ACC == 2 ? acc : static_cast<uint32_t>(ACC)), "n"(DESC_SW128_HI)
            : "memory");
}
// bf16 x bf16 -> f32 (kind::f16), K = 16 per instruction; ACC as above
template <int CG, int ACC>
__device__ __forceinline__ void tc_mma_bf16_lo(uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t acc = 1) {
    if constexpr (CG == 2)
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
            "mov.b64 da, {%1, %5};\n\tmov.b64 db, {%2, %5};\n\tsetp.ne.u32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %3, p;\n\t}"
            ::"r"(d), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(ACC == 2 ? acc : static_cast<uint32_t>(ACC)), "n"(DESC_SW128_HI)
            : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
            "mov.b64 da, {%1, %5};\n\tmov.b64 db, {%2, %5};\n\tsetp.ne.u32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t}"
            ::"r"(d), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(ACC == 2 ? acc : static_cast<uint32_t>(ACC)), "n"(DESC_SW128_HI)
            : "memory");
}
template <int CG>
__device__ __forceinline__ void tc_cp_scales(uint32_t taddr, uint64_t sdesc) {
    if constexpr (CG == 2) asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
    else asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
template <int CG>
__device__ __forceinline__ void tc_mma_mxf8(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
    if constexpr (CG == 2)
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %6, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
            ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
            : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %6, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
            ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
            : "memory");
}
// Arrive on `bar` (same shared-memory offset in every CTA of the pair) once all tcgen05
// operations issued so far by this thread have completed.  This is an mbarrier arrive
// broadcast to the CTA pair, not a data copy.
template <int CG>
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    if constexpr (CG == 2)
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                     ::"r"(bar), "h"(static_cast<uint16_t>(3))
                     : "memory");
    else
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// Same, arriving only on the issuing CTA's barrier.
template <int CG>
__device__ __forceinline__ void tc_commit_local(uint32_t bar) {
    if constexpr (CG == 2)
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
    else
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread `lane` of the warp receives row (lane base + lane).
__device__ __forceinline__ void tc_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Same wait, with the loaded registers as in/out operands so the compiler cannot move their
// first use above it.
__device__ __forceinline__ void tc_wait_ld(uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.wait::ld.sync.aligned;"
        : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
          "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
          "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
          "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
        :
        : "memory");
}

// ------------------------------------------------------------------ small numeric helpers
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}
// two floats -> two E4M3 bytes (RNE, saturating to +-448); `lo` lands in bits 0-7
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
    uint16_t d;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(d) : "f"(hi), "f"(lo));
    return d;
}
// four packed E4M3 bytes -> four floats (exact)
__device__ __forceinline__ void e4m3x4_to_float(uint32_t b4, float (&f)[4]) {
    uint32_t lo, hi;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(lo) : "h"(static_cast<uint16_t>(b4 & 0xFFFFu)));
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(hi) : "h"(static_cast<uint16_t>(b4 >> 16)));
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&hi));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void ld_shared_v4(uint32_t addr, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) {
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr));
}
__device__ __forceinline__ void st_shared_v2(uint32_t addr, uint32_t a, uint32_t b) {
    asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void ld_shared_v2(uint32_t addr, uint32_t& a, uint32_t& b) {
    asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(a), "=r"(b) : "r"(addr));
}

}  // namespace mx8
