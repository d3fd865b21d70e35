// Arithmetic shared by every kernel that produces MXFP8: packed bf16 amax, the integer E8M0 scale
// rule, exact power-of-two scaling and the E4M3 conversion.
#pragma once
#include "mx8_ptx.cuh"

namespace mx8 {
namespace qmath {

// packed constants of the two scale rules (one value per 16-bit half)
constexpr uint32_t RCEIL_ROUND_ADD2 = 0x001F001Fu, RCEIL_MIN_BYTE8_2 = 0x00600060u;   // byte >= 88
constexpr uint32_t FLOOR_ROUND_ADD2 = 0u, FLOOR_MIN_BYTE8_2 = 0x00080008u;            // byte >= 0

__device__ __forceinline__ uint32_t maxabs_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t max_u16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("max.u16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }

// Two non-negative bf16 amax bit patterns (one per 16-bit half) -> two E8M0 bytes (one per half):
// byte = max(min_byte, ((amax + round_add) >> 7) - 8), the exact integer form of
// ceil(log2(amax / 448)) + 127 (round_add 0x1F) or floor(log2(amax)) - 8 + 127 (round_add 0).
__device__ __forceinline__ uint32_t scale_bytes2(uint32_t amax2, uint32_t round_add2, uint32_t min_byte8_2) {
    uint32_t t = ((amax2 + round_add2) >> 7) & 0x00FF00FFu;
    return max_u16x2(t, min_byte8_2) - 0x00080008u;
}
// two scale bytes -> two bf16 reciprocals 2^(127 - byte): exponent field 254 - byte, mantissa 0
__device__ __forceinline__ uint32_t inv_scales2(uint32_t bytes2) { return (0x00FE00FEu - bytes2) << 7; }
// four bf16 (two packed words, already scaled) -> four E4M3 bytes
__device__ __forceinline__ uint32_t cvt4(uint32_t v0, uint32_t v1) {
    return cvt_e4m3x2(bf16_lo(v0), bf16_hi(v0)) | (cvt_e4m3x2(bf16_lo(v1), bf16_hi(v1)) << 16);
}

}  // namespace qmath
}  // namespace mx8
