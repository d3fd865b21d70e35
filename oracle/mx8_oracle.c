/* CPU restatement of the MXFP8 hot path in plain C.  TEST INFRASTRUCTURE ONLY: it is the checker
 * for the CUDA kernels (tests, smoke check, benchmark's CPU leg), never part of the shipped path.
 *
 * Parity status: pinned.  tests/test_oracle_c.py checks every function here against the golden
 * vectors that tests/golden/make_golden.py produced by running the reference's own torch code.
 *
 * Reference lines followed (paths inside the reference project):
 *   quantize (ceil scale rule) .. blackwell-ultra/019-mxfp8-quantize.py:31-46
 *   scale tile layout ........... blackwell-ultra/019-mxfp8-quantize.py:49-53 and the kernel's
 *                                 store address, blackwell-ultra/019-mxfp8-quantize.cu:131
 *   dequantize .................. blackwell/047-mxfp8-mma-2cta-MNK128-polished.py:36-51
 *   GEMM check .................. blackwell/047-mxfp8-mma-2cta-MNK128-polished.py:138-143
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define MX8O_API __attribute__((visibility("default")))

static float bf16_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static uint16_t f32_to_bf16_rne(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* E8M0 byte from the bit pattern of |amax| (bf16).  mode 0: ceil(log2(amax/448)) + 127 with
 * amax/448 clamped to 1e-12 (byte >= 88); mode 1: floor(log2(amax)) - 8 + 127 clamped to 0. */
MX8O_API uint8_t mx8o_scale_byte(uint16_t amax_bits, int mode) {
    int a = amax_bits & 0x7FFF;
    int b = mode == 0 ? ((a + 0x1F) >> 7) - 8 : (a >> 7) - 8;
    int lo = mode == 0 ? 88 : 0;
    return (uint8_t)(b < lo ? lo : b);
}

/* float -> E4M3 (fn), round to nearest even, saturating to +-448 */
MX8O_API uint8_t mx8o_e4m3_encode(float v) {
    uint8_t sign = signbit(v) ? 0x80 : 0;
    double a = fabs((double)v);
    if (a > 448.0) a = 448.0;
    int code;
    if (a < 0.015625) {                    /* below 2^-6: multiples of 2^-9 */
        code = (int)nearbyint(a * 512.0);  /* default rounding mode is to-nearest-even */
    } else {
        int e;
        double m = frexp(a, &e);           /* a = m * 2^e, m in [0.5, 1) */
        int q = (int)nearbyint(m * 16.0);  /* significand * 8 in [8, 16] */
        e -= 1;
        if (q == 16) { q = 8; e += 1; }
        code = ((e + 7) << 3) | (q - 8);
    }
    if (code > 0x7E) code = 0x7E;
    return (uint8_t)(code | sign);
}

MX8O_API float mx8o_e4m3_decode(uint8_t b) {
    int e = (b >> 3) & 0xF, m = b & 7;
    float v;
    if (e == 0xF && m == 7) return NAN;
    if (e == 0) v = ldexpf((float)m, -9);
    else v = ldexpf(1.0f + (float)m / 8.0f, e - 7);
    return (b & 0x80) ? -v : v;
}

/* x: bf16 bits [M][N]; q: bytes [M][N]; sc: bytes [M][N/32] (plain row-major, not tiled) */
MX8O_API void mx8o_quantize(const uint16_t* x, int M, int N, int mode, uint8_t* q, uint8_t* sc) {
    for (int r = 0; r < M; ++r)
        for (int kb = 0; kb < N / 32; ++kb) {
            const uint16_t* blk = x + (size_t)r * N + kb * 32;
            uint16_t amax = 0;
            for (int i = 0; i < 32; ++i) {
                uint16_t a = blk[i] & 0x7FFF;
                if (a > amax) amax = a;
            }
            uint8_t b = mx8o_scale_byte(amax, mode);
            sc[(size_t)r * (N / 32) + kb] = b;
            float inv = ldexpf(1.0f, 127 - (int)b);
            for (int i = 0; i < 32; ++i) q[(size_t)r * N + kb * 32 + i] = mx8o_e4m3_encode(bf16_to_f32(blk[i]) * inv);
        }
}

/* plain [R][C/32] scale bytes -> tiles [R/128][C/128][512] */
MX8O_API void mx8o_scale_swizzle(const uint8_t* sc, int R, int KB, uint8_t* out) {
    for (int r = 0; r < R; ++r)
        for (int kb = 0; kb < KB; ++kb) {
            size_t tile = (size_t)(r / 128) * (KB / 4) + kb / 4;
            int rr = r % 128;
            out[tile * 512 + (rr % 32) * 16 + (rr / 32) * 4 + kb % 4] = sc[(size_t)r * KB + kb];
        }
}

MX8O_API void mx8o_scale_unswizzle(const uint8_t* tiles, int R, int KB, uint8_t* sc) {
    for (int r = 0; r < R; ++r)
        for (int kb = 0; kb < KB; ++kb) {
            size_t tile = (size_t)(r / 128) * (KB / 4) + kb / 4;
            int rr = r % 128;
            sc[(size_t)r * KB + kb] = tiles[tile * 512 + (rr % 32) * 16 + (rr / 32) * 4 + kb % 4];
        }
}

/* the four outputs of the reference's mxfp8_quantize for one matrix (scales tiled) */
MX8O_API int mx8o_quantize_both(const uint16_t* x, int M, int N, int mode, uint8_t* q, uint8_t* sc_tiles, uint8_t* qt,
                                uint8_t* sct_tiles) {
    uint8_t* plain = (uint8_t*)malloc((size_t)M * N / 32);
    uint16_t* xt = (uint16_t*)malloc((size_t)M * N * 2);
    if (!plain || !xt) { free(plain); free(xt); return 1; }
    mx8o_quantize(x, M, N, mode, q, plain);
    mx8o_scale_swizzle(plain, M, N / 32, sc_tiles);
    for (int r = 0; r < M; ++r)
        for (int c = 0; c < N; ++c) xt[(size_t)c * M + r] = x[(size_t)r * N + c];
    mx8o_quantize(xt, N, M, mode, qt, plain);
    mx8o_scale_swizzle(plain, N, M / 32, sct_tiles);
    free(plain);
    free(xt);
    return 0;
}

/* C = dequant(A) . dequant(B)^T with fp32 accumulation in K order, rounded to bf16 (c_bf16) and/or
 * kept as float (c_f32); either output may be NULL.  Scales in the tiled layout. */
MX8O_API int mx8o_gemm(const uint8_t* a, const uint8_t* a_sc, const uint8_t* b, const uint8_t* b_sc, int M, int N, int K,
                       uint16_t* c_bf16, float* c_f32) {
    float* ad = (float*)malloc((size_t)M * K * 4);
    float* bd = (float*)malloc((size_t)N * K * 4);
    if (!ad || !bd) { free(ad); free(bd); return 1; }
    const int KB = K / 32;
    for (int pass = 0; pass < 2; ++pass) {
        const uint8_t* q = pass ? b : a;
        const uint8_t* s = pass ? b_sc : a_sc;
        float* d = pass ? bd : ad;
        int R = pass ? N : M;
        for (int r = 0; r < R; ++r)
            for (int k = 0; k < K; ++k) {
                int kb = k / 32, rr = r % 128;
                uint8_t byte = s[((size_t)(r / 128) * (KB / 4) + kb / 4) * 512 + (rr % 32) * 16 + (rr / 32) * 4 + kb % 4];
                d[(size_t)r * K + k] = mx8o_e4m3_decode(q[(size_t)r * K + k]) * ldexpf(1.0f, (int)byte - 127);
            }
    }
    for (int i = 0; i < M; ++i)
        for (int j = 0; j < N; ++j) {
            float acc = 0.0f;
            const float* ar = ad + (size_t)i * K;
            const float* br = bd + (size_t)j * K;
            for (int k = 0; k < K; ++k) acc += ar[k] * br[k];
            if (c_f32) c_f32[(size_t)i * N + j] = acc;
            if (c_bf16) c_bf16[(size_t)i * N + j] = f32_to_bf16_rne(acc);
        }
    free(ad);
    free(bd);
    return 0;
}
