/* mx8 — C ABI of the B200 (sm_100a) MXFP8 hot path: bf16 -> E4M3 + E8M0 quantize and the
 * block-scaled GEMM that consumes it.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer owned by the caller (HOST arrays of device pointers and the *_host forms are
 *     marked as such); the library allocates no device memory and keeps no reference after the call returns.  Two
 *     families create CUDA streams once per device and keep them: the *_host forms (copy streams) and mx8_moe_fwd /
 *     mx8_moe_bwd in minibatch mode (two side streams);
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream); launches are
 *     asynchronous, exactly like the reference's entry points;
 *   - the return value is a status code (MX8_OK == 0); nothing calls exit() and nothing traps.
 *     The reference prints and exits on errors (blackwell/gpu-experiments.cuh:29-47);
 *   - M, N, K are multiples of 128, the granularity of the tcgen05 scale-factor layout, as in
 *     the reference (blackwell-ultra/019-mxfp8-quantize.py:59);
 *   - "scale tile layout": the E8M0 bytes of a 128-row x 128-column (4 blocks of 32) tile are
 *     512 consecutive bytes, the byte of (row r, block kb) at (r % 32) * 16 + (r / 32) * 4 + kb;
 *     tiles are ordered [rows / 128][cols / 128] (blackwell-ultra/019-mxfp8-quantize.cu:131).
 *
 * There is no CPU fallback: on a machine without an sm_100 device every compute entry point
 * returns MX8_ERR_UNSUPPORTED or MX8_ERR_CUDA.
 */
#ifndef MX8_H_
#define MX8_H_

#if defined(__GNUC__)
#define MX8_API __attribute__((visibility("default")))
#else
#define MX8_API
#endif

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    MX8_OK = 0,
    MX8_ERR_ARG = 1,            /* null pointer, bad enum value, nothing requested          */
    MX8_ERR_SHAPE = 2,          /* a dimension is not a positive multiple of 128            */
    MX8_ERR_ALIGN = 3,          /* a pointer is not 16-byte aligned                         */
    MX8_ERR_CUDA = 4,           /* a CUDA runtime / driver call failed (mx8_last_cuda_error) */
    MX8_ERR_UNSUPPORTED = 5,    /* device is not compute capability 10.x                    */
    MX8_ERR_DEVICE_TIMEOUT = 6, /* a kernel's bounded wait expired (mx8_device_status)      */
    MX8_ERR_LIMIT = 7           /* problem exceeds a built-in size limit (mx8_last_cuda_error has the text) */
};

/* scale rounding */
enum {
    MX8_SCALE_RCEIL = 0, /* E = ceil(log2(amax / 448)); the reference's rule                  */
    MX8_SCALE_FLOOR = 1  /* E = floor(log2(amax)) - 8; OCP rule, E4M3 saturation live         */
};

/* GEMM output element type */
enum {
    MX8_C_BF16 = 0, /* blackwell/047-mxfp8-mma-2cta-MNK128-polished.cu:461 (C is bf16)       */
    MX8_C_F32 = 1,  /* blackwell/009-mxfp8-mm.cu:46, 010..017 (C is float)                   */
    MX8_C_MXFP8 = 2 /* E4M3 bytes + scale tiles (mx8_gemm_grouped only): the quantizing epilogue of
                       blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.cu:1644-1700 */
};

/* Quantize x[E][M][N] (bf16, row-major; E = 1 for a matrix) to MXFP8.
 *   fp8   [E][M][N] bytes and sc   [E*M/128][N/128][512]: blocks of 32 along N ("normal");
 *   fp8_t [E][N][M] bytes and sc_t [E*N/128][M/128][512]: the transpose, blocks of 32 along M.
 * Pass fp8 == sc == NULL or fp8_t == sc_t == NULL to skip that orientation.
 * Replaces mxfp8_quantize_entrypoint, blackwell-ultra/019-mxfp8-quantize.cu:185-219 (caller-
 * allocated outputs) and the [E,M,N] form at
 * blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.cu:404-448; also the legacy
 * kernel / kernel_transpose pair of blackwell/018-mxfp8-quantize.cu:288-300 and the combined
 * blackwell/038-mxfp8-quantize-combined.cu:397-399. */
MX8_API int mx8_quantize(const void* x_bf16, int E, int M, int N,
                 void* fp8, void* sc, void* fp8_t, void* sc_t,
                 int scale_mode, void* stream);

/* C[M][N] = dequant(A[M][K]) . dequant(B[N][K])^T, fp32 accumulation on tcgen05 tensor cores.
 *   A, B: E4M3 bytes, K contiguous; A_sc [M/128][K/128][512], B_sc [N/128][K/128][512] in the
 *   scale tile layout; C row-major, bf16 or float per c_dtype.
 * Replaces `kernel(A_fp8, A_sc, B_fp8, B_sc, C)`,
 * blackwell/047-mxfp8-mma-2cta-MNK128-polished.cu:525-541 (and 009/010/016/017/045/046). */
MX8_API int mx8_gemm(const void* A, const void* A_sc, const void* B, const void* B_sc, void* C,
             int M, int N, int K, int c_dtype, void* stream);

/* Same contract as mx8_gemm with the kernel variant chosen by the caller:
 *   cta_group 2 = one 256x256 tile per CTA pair (cluster of 2), 1 = one 128x256 tile per CTA,
 *   0 = library default; max_ctas caps the persistent grid (0 = all SMs). Used by the tests and
 *   the benchmark's ablations. */
MX8_API int mx8_gemm_ex(const void* A, const void* A_sc, const void* B, const void* B_sc, void* C,
                int M, int N, int K, int c_dtype, int cta_group, int max_ctas, void* stream);

/* Grouped / quantizing form of the GEMM.
 *   A [M][K] holds the rows of all groups back to back; group g owns group_rows[g] rows (device
 *   int32, multiples of 256) and multiplies them with its own B_g [N][K]: B is [num_groups][N][K],
 *   B_sc [num_groups*N/128][K/128][512].  num_groups == 0: one B for all rows (plain GEMM).
 *   num_rows (device int32, may be NULL): rows actually present; row tiles beyond it are skipped,
 *   so M can be a capacity.  c_dtype MX8_C_MXFP8: the accumulator is rounded to bf16 and quantized
 *   with blocks of 32 along N into C (bytes [M][N]) and C_sc ([M/128][N/128][512]); otherwise C_sc
 *   must be NULL.
 * Replaces expert_grouped_gemm<false> and its two epilogues,
 * blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.cu:1399-1736. */
MX8_API int mx8_gemm_grouped(const void* A, const void* A_sc, const void* B, const void* B_sc, void* C, void* C_sc,
                             int M, int N, int K, int c_dtype, const void* num_rows, const void* group_rows,
                             int num_groups, void* stream);

/* MoE dispatch fused with quantize: row r of the routed activation matrix is token
 * peer_token_idx[r] / topk of rank peer_rank[r] (all-zero when peer_rank[r] < 0); the rows are pulled
 * from x_ptrs[rank] (HOST array of `world` device pointers to every rank's [tokens][hidden] bf16
 * matrix; peer-mapped memory for other GPUs) and quantized both ways in one pass:
 *   fp8 [capacity][hidden], sc; fp8_t [hidden][capacity], sc_t.  Only the first *num_tokens rows
 * (device int32, a multiple of 256) are produced.  world <= 16.
 * Replaces dispatch_quantize_kernel, blackwell-ultra/022-…-mxfp8-bw.cu:717-828. */
MX8_API int mx8_moe_dispatch_quantize(const void* const* x_ptrs, int world, int hidden, int topk, const void* peer_rank,
                                      const void* peer_token_idx, const void* num_tokens, int capacity, void* fp8,
                                      void* sc, void* fp8_t, void* sc_t, void* stream);

/* hidden = bf16( silu(dequant(gate)) * dequant(up) ) from two MXFP8 matrices [rows][cols], re-quantized
 * both ways (hidden_fp8/sc blocks along cols, hidden_fp8_t/sc_t the transpose).  num_rows (device
 * int32 or NULL) bounds the rows processed.  hidden_bf16 (may be NULL) receives the bf16 activation.
 * Replaces swiglu_fwd<false>, blackwell-ultra/022-…-mxfp8-bw.cu:924-1129. */
MX8_API int mx8_swiglu_quantize(const void* gate_fp8, const void* gate_sc, const void* up_fp8, const void* up_sc,
                                int rows, int cols, const void* num_rows, void* hidden_fp8, void* hidden_sc,
                                void* hidden_fp8_t, void* hidden_sc_t, void* hidden_bf16, void* stream);

/* MoE combine: row r (< min(*num_tokens, capacity), peer_rank[r] >= 0) of y_routed [capacity][hidden] bf16 is
 * written to row peer_token_idx[r] of combine_ptrs[peer_rank[r]] (HOST array of `world` device pointers to
 * every rank's [combine_rows][hidden] bf16 buffer, combine_rows = tokens*topk, peer-mapped for other GPUs).
 * A schedule that overflowed its capacity (device status word set by mx8_moe_schedule) cannot make this call
 * read or write out of bounds: rows beyond capacity, ranks outside [0, world) and destination rows outside
 * [0, combine_rows) are skipped; the reference traps in that case (same file :86).  The caller orders this call
 * against the readers of those buffers (a cross-rank barrier), as the reference's harness does.
 * Replaces combine_kernel, blackwell-ultra/022-…-mxfp8-bw.cu:830-922. */
MX8_API int mx8_moe_combine(const void* y_routed, const void* peer_rank, const void* peer_token_idx, const void* num_tokens,
                            int capacity, int hidden, void* const* combine_ptrs, int world, long long combine_rows, void* stream);

/* out[t] = bf16( y_shared[t] + sum_j topk_weights[t][j] * combine_buffer[t*topk + j] ); y_shared may be
 * NULL (no shared expert).  topk_weights float32 [tokens][topk]; the other tensors bf16.
 * Replaces fwd_epilogue, blackwell-ultra/022-…-mxfp8-bw.cu:2789-2856. */
MX8_API int mx8_moe_fwd_epilogue(const void* y_shared, const void* combine_buffer, const void* topk_weights, void* out,
                                 int tokens, int hidden, int topk, void* stream);

/* Grouped GEMM whose epilogue performs the MoE combine: row r (< *num_rows, peer_rank[r] >= 0) of
 * dequant(A).dequant(B_g)^T is written as bf16 to row peer_token_idx[r] of dst_ptrs[peer_rank[r]]
 * (HOST array of `world` device pointers to [.][N] bf16 buffers, peer-mapped for other GPUs); no
 * [M][N] result is materialised.  Same result as mx8_gemm_grouped followed by mx8_moe_combine.
 * Fuses expert_grouped_gemm<false> (bf16 epilogue) with combine_kernel,
 * blackwell-ultra/022-…-mxfp8-bw.cu:1701-1720 and :830-922. */
MX8_API int mx8_gemm_grouped_scatter(const void* A, const void* A_sc, const void* B, const void* B_sc, int M, int N, int K,
                                     const void* num_rows, const void* group_rows, int num_groups, const void* peer_rank,
                                     const void* peer_token_idx, void* const* dst_ptrs, int world, void* stream);

/* Grouped GEMM with two operand pairs accumulated into one bf16 result:
 *   C = dequant(A1).dequant(B1_g)^T + dequant(A2).dequant(B2_g)^T,  A1 [M][K1], A2 [M][K2],
 *   B1 [num_groups][N][K1], B2 [num_groups][N][K2]; grouping and num_rows as in mx8_gemm_grouped.
 * This is the data-gradient GEMM of the MoE backward, d_x = [d_gate | d_up] . [Wg^T | Wu^T]^T without the
 * concatenations; the optional second GEMM of expert_grouped_gemm,
 * blackwell-ultra/022-…-mxfp8-bw.cu:1399-1736. */
MX8_API int mx8_gemm_grouped_dual(const void* A1, const void* A1_sc, const void* B1, const void* B1_sc, const void* A2,
                                  const void* A2_sc, const void* B2, const void* B2_sc, void* C, int M, int N, int K1, int K2,
                                  const void* num_rows, const void* group_rows, int num_groups, void* stream);

/* Weight-gradient GEMM: for every group g, C_g [M][N] (bf16) = dequant(A^T[:, rows_g]) . dequant(B^T[:, rows_g])^T
 * where A^T is [M][rows] and B^T is [N][rows] (the transposed outputs of the quantizer, scale blocks
 * along the row index), rows_g the consecutive group_rows[g] columns of group g (device int32,
 * multiples of 128).  A group without rows yields zeros.  C is [num_groups][M][N].
 * Replaces expert_grouped_gemm<false, true> (IS_WGRAD), blackwell-ultra/022-…-mxfp8-bw.cu:1399-1736. */
MX8_API int mx8_gemm_wgrad(const void* A_t, const void* A_t_sc, const void* B_t, const void* B_t_sc, void* C, int M, int N,
                           int rows, const void* group_rows, int num_groups, void* stream);

/* Backward of SwiGLU on MXFP8 inputs, re-quantized both ways: with g = dequant(gate), u = dequant(up),
 * s = sigmoid(g): which == 0 -> d_gate = bf16( ((1 - g s) s + g s) * u * d_hidden ), which == 1 ->
 * d_up = bf16( g s * d_hidden ); d_hidden bf16 [rows][cols].  Outputs as in mx8_swiglu_quantize;
 * out_bf16 (may be NULL) receives the bf16 gradient.
 * Replaces the SwiGLU backward task of the reference's backward kernel,
 * blackwell-ultra/022-…-mxfp8-bw.cu:1131-1397; arithmetic as in …-mxfp8-bw.py:167-171. */
MX8_API int mx8_swiglu_bwd_quantize(const void* gate_fp8, const void* gate_sc, const void* up_fp8, const void* up_sc,
                                    const void* d_hidden, int rows, int cols, const void* num_rows, int which, void* out_fp8,
                                    void* out_sc, void* out_fp8_t, void* out_sc_t, void* out_bf16, void* stream);
/* Both gradients (same arithmetic, same bytes) from one pass over gate, up and d_hidden: each input is
 * read once, as in the reference's single task (same file :1250-1353). */
MX8_API int mx8_swiglu_bwd_quantize_both(const void* gate_fp8, const void* gate_sc, const void* up_fp8, const void* up_sc,
                                         const void* d_hidden, int rows, int cols, const void* num_rows,
                                         void* d_gate_fp8, void* d_gate_sc, void* d_gate_fp8_t, void* d_gate_sc_t,
                                         void* d_up_fp8, void* d_up_sc, void* d_up_fp8_t, void* d_up_sc_t, void* stream);

/* d_combine_buffer[t*topk + j] = bf16( d_output[t] * topk_weights[t][j] ) (bf16 [tokens][hidden] in,
 * [tokens*topk][hidden] out).  Replaces bwd_prologue, blackwell-ultra/022-…-mxfp8-bw.cu:2881-2923. */
MX8_API int mx8_moe_bwd_prologue(const void* d_output, const void* topk_weights, void* d_combine_buffer, int tokens, int hidden,
                                 int topk, void* stream);

/* d_x[t] = bf16( d_x_shared[t] + sum_j d_x_routed_buffer[t*topk + j] ), fp32 sum, j ascending; d_x_shared
 * may be NULL.  Replaces bwd_epilogue, blackwell-ultra/022-…-mxfp8-bw.cu:2945-2993. */
MX8_API int mx8_moe_bwd_epilogue(const void* d_x_shared, const void* d_x_routed_buffer, void* d_x, int tokens, int hidden,
                                 int topk, void* stream);

/* Expert-parallel MoE routing schedule for the calling rank (int32 everywhere).
 *   topk_all [world][tokens][topk]: global expert ids chosen by every rank's tokens;
 *   this rank owns experts [rank*num_local_experts, (rank+1)*num_local_experts).
 * Outputs: peer_rank[capacity] (source rank per row, -1 = padding/unused), peer_token_idx[capacity]
 * (token*topk + k on the source rank), num_tokens[1] (rows used, every expert padded to 256),
 * tokens_per_expert[num_local_experts] (padded).  Rows of an expert: round j holds the j-th pair of every
 * source rank that still has one, ranks ascending, where the pairs of one source rank are counted in the
 * reference kernel's order: entry idx = token*topk + k belongs to thread idx % 1024 of a 1024-thread
 * block and threads number their hits one after the other, i.e. by (idx % 1024, idx / 1024)
 * (blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.cu:99-146).  `scratch` is `scratch_bytes` of device memory,
 * overwritten: with mx8_moe_schedule_scratch_bytes(...) bytes the schedule is a counting sort that reads
 * the routing table twice; with at least num_local_experts*(world+1) ints it still works, scanning the
 * table once per local expert; less is MX8_ERR_LIMIT.  capacity is a multiple of 256; a schedule that
 * does not fit sets the device status word (mx8_device_status) instead of trapping.
 * Replaces scheduler::schedule, blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.cu:149-183. */
MX8_API size_t mx8_moe_schedule_scratch_bytes(int world, int tokens, int topk, int num_local_experts);
MX8_API int mx8_moe_schedule(const void* topk_all, int world, int tokens, int topk, int num_local_experts,
                             int capacity, int rank, void* peer_rank, void* peer_token_idx, void* num_tokens,
                             void* tokens_per_expert, void* scratch, size_t scratch_bytes, void* stream);

/* Same schedule, same outputs, for callers that cannot provide scratch memory.  It has no counterpart
 * in the reference.  Hosts whose memory plan is fixed after start-up, or that run under a foreign
 * allocator and must not call cudaMalloc on the request path, use this form: the counting scratch is
 * a fixed 64 KiB array inside the library (one copy per device, held until the process exits), and
 * the call allocates nothing.  Limit: num_local_experts * (world + 1) <= 16384, otherwise
 * MX8_ERR_LIMIT.  The first call on a device looks the array's address up; make that call before
 * starting any stream capture.  Every call on a device uses the same array (cleared at the start of
 * each call), so calls that can overlap on the GPU must be ordered by the caller. */
MX8_API int mx8_moe_schedule_static(const void* topk_all, int world, int tokens, int topk, int num_local_experts,
                                    int capacity, int rank, void* peer_rank, void* peer_token_idx, void* num_tokens,
                                    void* tokens_per_expert, void* stream);

/* C[M][N] = A[M][K] . B[N][K]^T with bf16 operands (K contiguous, a multiple of 64), fp32 accumulation
 * on the tensor cores (tcgen05.mma kind::f16), C bf16 or float.  The dual form adds a second product
 * A2[M][K2] . B2[N][K2]^T into the same accumulator (K2 = 0: none).
 * Replaces the shared-expert GEMMs, expert_grouped_gemm<true> of
 * blackwell-ultra/022-moe-dispatch-mlp-swiglu-combine-mxfp8-bw.cu:1399-1736 (forward gate / up / down,
 * backward dgrad with two accumulated products; the weight gradients take explicitly transposed
 * operands, see mx8_transpose_bf16). */
MX8_API int mx8_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int c_dtype, void* stream);
MX8_API int mx8_gemm_bf16_dual(const void* A1, const void* B1, const void* A2, const void* B2, void* C, int M, int N,
                               int K1, int K2, int c_dtype, void* stream);

/* Element-wise pieces of the shared expert (bf16 in, fp32 arithmetic, bf16 out; n elements):
 *   mx8_swiglu_bf16      hidden = silu(gate) * up       (swiglu_fwd<true>, same file :1097-1110)
 *   mx8_swiglu_bwd_bf16  d_gate = d_hidden * dsilu(gate) * up, d_up = d_hidden * silu(gate)
 *                        (swiglu_bwd<true>, same file :1354-1375)
 *   mx8_transpose_bf16   out[cols][rows] = in[rows][cols]^T (rows, cols multiples of 64): operands of the
 *                        shared expert's weight-gradient GEMMs, which the reference reads token-major
 *                        (same file :1547-1550). */
MX8_API int mx8_swiglu_bf16(const void* gate, const void* up, void* hidden, long long n, void* stream);
MX8_API int mx8_swiglu_bwd_bf16(const void* d_hidden, const void* gate, const void* up, void* d_gate, void* d_up,
                                long long n, void* stream);
MX8_API int mx8_transpose_bf16(const void* in, void* out, int rows, int cols, void* stream);

/* Row windows: the MoE layer cut into minibatches of consecutive local experts, so that the transfer
 * legs (dispatch, combine) of one minibatch can run beside the GEMMs of another on a second stream.
 * The reference does this inside one kernel with a task queue and dedicated communication SMs
 * (blackwell-ultra/022-…-mxfp8-bw.cu:1738-2010, arguments num_comm_sms / minibatch_size); here every
 * kernel of the layer has a form that works on rows [*row_begin, *row_end) only, on at most max_sms
 * multiprocessors, and the host orders the pieces with streams and events.
 *   row_begin, row_end: device ints (multiples of 256), NULL = 0 / the entry point's own row count;
 *   max_sms: 0 = the whole device;
 *   own_sms: 0, or 1 in mx8_moe_combine_window to give the combine max_sms multiprocessors of its own: bulk-copy blocks
 *   whose shared memory keeps GEMM and dispatch blocks off them (the caller launches its GEMMs on max_sms fewer
 *   multiprocessors).  Without it a throttled combine shares multiprocessors with the GEMMs.  Other entry points ignore
 *   the field.
 * mx8_moe_minibatch_bounds fills bounds[0..minibatches] with the row at which each group of
 * num_local_experts / minibatches consecutive experts starts (from tokens_per_expert). */
typedef struct mx8_window {
    const void* row_begin;
    const void* row_end;
    int max_sms;
    int own_sms;
} mx8_window;
MX8_API int mx8_moe_minibatch_bounds(const void* tokens_per_expert, int num_local_experts, int minibatches, void* bounds,
                                     void* stream);
MX8_API int mx8_moe_dispatch_quantize_window(const void* const* x_ptrs, int world, int hidden, int topk, const void* peer_rank,
                                             const void* peer_token_idx, const void* num_tokens, int capacity, void* fp8,
                                             void* sc, void* fp8_t, void* sc_t, const mx8_window* window, void* stream);
MX8_API int mx8_gemm_grouped_window(const void* A, const void* A_sc, const void* B, const void* B_sc, void* C, void* C_sc,
                                    int M, int N, int K, int c_dtype, const void* num_rows, const void* group_rows,
                                    int num_groups, const mx8_window* window, void* stream);
/* Two grouped products of the same A in one launch: C1 = A . B1_g^T and C2 = A . B2_g^T (B1, B2 of one shape, C1, C2 of
 * one type; other arguments as mx8_gemm_grouped_window; N a multiple of 256).  The reference's task queue interleaves
 * the gate and up projections of a minibatch the same way (blackwell-ultra/022-…-mxfp8-bw.cu:1876-1992); one launch has
 * one partial last round instead of two and reads every A panel once for both. */
MX8_API int mx8_gemm_grouped_pair_window(const void* A, const void* A_sc, const void* B1, const void* B1_sc, const void* B2,
                                         const void* B2_sc, void* C1, void* C1_sc, void* C2, void* C2_sc, int M, int N, int K,
                                         int c_dtype, const void* num_rows, const void* group_rows, int num_groups,
                                         const mx8_window* window, void* stream);
/* Gate and up projections of the MoE layer with SwiGLU in the epilogue, one launch: per 256-row x 128-column tile one CTA
 * of the pair holds the gate weights' rows and the other the up weights' rows, so the epilogue has gate and up of the
 * same columns side by side.  It writes gate and up as MXFP8 (bytes [M][N] + scale tiles, exactly what two
 * mx8_gemm_grouped calls with MX8_C_MXFP8 write), and hidden = bf16( silu(dequant(gate)) * dequant(up) ) as MXFP8 in both
 * orientations (exactly what mx8_swiglu_quantize writes from those): hidden_fp8 [M][N] / hidden_sc and hidden_fp8_t
 * [N][M] / hidden_sc_t.  A [M][K], B_gate / B_up [num_groups][N][K]; M a multiple of 256, N and K of 128; grouping, num_rows
 * and window as in mx8_gemm_grouped_window.  Replaces the quantizing epilogue of expert_grouped_gemm plus swiglu_fwd<false>,
 * blackwell-ultra/022-…-mxfp8-bw.cu:1644-1700 and :924-1129, which the reference runs as separate tasks. */
MX8_API int mx8_gemm_grouped_swiglu_window(const void* A, const void* A_sc, const void* B_gate, const void* B_gate_sc,
                                           const void* B_up, const void* B_up_sc, void* gate_fp8, void* gate_sc, void* up_fp8,
                                           void* up_sc, void* hidden_fp8, void* hidden_sc, void* hidden_fp8_t, void* hidden_sc_t,
                                           int M, int N, int K, const void* num_rows, const void* group_rows, int num_groups,
                                           const mx8_window* window, void* stream);
MX8_API int mx8_swiglu_quantize_window(const void* gate_fp8, const void* gate_sc, const void* up_fp8, const void* up_sc,
                                       int rows, int cols, const void* num_rows, void* hidden_fp8, void* hidden_sc,
                                       void* hidden_fp8_t, void* hidden_sc_t, void* hidden_bf16, const mx8_window* window,
                                       void* stream);
MX8_API int mx8_swiglu_bwd_quantize_both_window(const void* gate_fp8, const void* gate_sc, const void* up_fp8, const void* up_sc,
                                                const void* d_hidden, int rows, int cols, const void* num_rows,
                                                void* d_gate_fp8, void* d_gate_sc, void* d_gate_fp8_t, void* d_gate_sc_t,
                                                void* d_up_fp8, void* d_up_sc, void* d_up_fp8_t, void* d_up_sc_t,
                                                const mx8_window* window, void* stream);
MX8_API int mx8_gemm_grouped_dual_window(const void* A1, const void* A1_sc, const void* B1, const void* B1_sc, const void* A2,
                                         const void* A2_sc, const void* B2, const void* B2_sc, void* C, int M, int N, int K1,
                                         int K2, const void* num_rows, const void* group_rows, int num_groups,
                                         const mx8_window* window, void* stream);
MX8_API int mx8_moe_combine_window(const void* y_routed, const void* peer_rank, const void* peer_token_idx,
                                   const void* num_tokens, int capacity, int hidden, void* const* combine_ptrs, int world,
                                   long long combine_rows, const mx8_window* window, void* stream);
/* As mx8_moe_minibatch_bounds with the groups given explicitly: first_expert is a HOST array of minibatches + 1
 * ascending expert indices, first_expert[0] = 0, first_expert[minibatches] = num_local_experts (NULL = even split);
 * at most 64 minibatches. */
MX8_API int mx8_moe_minibatch_bounds_split(const void* tokens_per_expert, int num_local_experts, int minibatches,
                                           const int* first_expert, void* bounds, void* stream);

/* The whole layer in one call.
 *
 * mx8_moe_fwd = the reference's dispatch_mlp_swiglu_combine_fwd (blackwell-ultra/022-…-mxfp8-bw.cu:2016-2136): tokens
 * are pulled from every rank's x (x_ptrs), quantized, run through the local experts' gate / up / SwiGLU / down, and
 * the result rows are pushed into the owners' combine buffers (combine_ptrs); the shared expert (bf16) runs on this
 * rank's own tokens when shared_intermediate > 0.  The reference allocates its outputs itself; here the caller
 * passes them (the thirteen tensors its binding returns, same names, capacity rows for the routed ones) plus a
 * workspace of mx8_moe_fwd_workspace_bytes(dims) bytes of device memory for the tensors it keeps internal.
 *   num_comm_sms, minibatch_size: the reference's arguments.  Both > 0: the local experts are cut into
 *   ceil(capacity / minibatch_size) minibatches whose transfers overlap the other minibatches' GEMMs on two side
 *   streams the library creates once per device; outputs do not depend on the split.  Otherwise one launch
 *   sequence on `stream`.  Tuning (all may be 0): minibatches overrides the count; ramp = 1 makes the first and
 *   last minibatch half as large, ramp > 100 lets the minibatches grow by ramp percent from both ends toward the middle; combine_sms caps a combine that runs beside GEMMs (default num_comm_sms / 4);
 *   combine_own_sms > 0 instead gives such a combine that many multiprocessors of its own and the GEMMs beside it as many fewer;
 *   split_swiglu = 1 runs SwiGLU as its own kernel after the gate / up projections instead of in their epilogue, and
 *   then split_gate_up = 1 launches the two projections separately instead of as one pair launch.
 *   fuse_combine = 1: the down projection's epilogue writes the owners' buffers directly (one sequence; y_routed
 *   may be NULL).
 * mx8_moe_bwd = dispatch_mlp_swiglu_combine_bwd (same file :2556-2760) in the same style: the eighteen tensors its
 * binding returns are passed by the caller, the transposed gradients live in the workspace.
 * Both return after queueing; `stream` waits for the side streams' last work.  x_ptrs / combine_ptrs /
 * d_combine_ptrs / d_x_routed_ptrs are HOST arrays of `world` device pointers. */
typedef struct mx8_moe_dims {
    int world, tokens, hidden, intermediate, shared_intermediate, num_local_experts, topk, capacity;
    int num_comm_sms, minibatch_size;
    int minibatches, ramp, combine_sms, split_gate_up, split_swiglu, combine_own_sms;
} mx8_moe_dims;
typedef struct mx8_moe_fwd_args {
    mx8_moe_dims dims;
    int fuse_combine;
    const void* x;                          /* this rank's [tokens][hidden] bf16 (shared expert input) */
    const void* const* x_ptrs;
    void* const* combine_ptrs;
    const void *w_shared_gate, *w_shared_up, *w_shared_down;       /* bf16 [Is][H], [Is][H], [H][Is] or NULL */
    const void *w_gate, *w_gate_sc, *w_up, *w_up_sc, *w_down, *w_down_sc;
    const void *peer_rank, *peer_token_idx, *num_tokens, *tokens_per_expert;
    void *x_fp8_t, *x_sc_t, *gate_shared, *gate_fp8, *gate_sc, *up_shared, *up_fp8, *up_sc, *hidden_shared, *hidden_fp8_t,
         *hidden_sc_t, *y_shared, *y_routed;
    void* workspace;
    size_t workspace_bytes;
} mx8_moe_fwd_args;
typedef struct mx8_moe_bwd_args {
    mx8_moe_dims dims;
    const void* d_y_shared;                 /* [tokens][hidden] bf16 or NULL */
    const void* const* d_combine_ptrs;
    void* const* d_x_routed_ptrs;
    const void *w_shared_gate_T, *w_shared_up_T, *w_shared_down_T;
    const void *w_gate_T, *w_gate_T_sc, *w_up_T, *w_up_T_sc, *w_down_T, *w_down_T_sc;
    const void *x_fp8_t, *x_sc_t, *gate_shared, *gate_fp8, *gate_sc, *up_shared, *up_fp8, *up_sc, *hidden_shared, *hidden_fp8_t,
               *hidden_sc_t;
    const void* x;                          /* this rank's tokens (shared expert weight gradients) */
    const void *peer_rank, *peer_token_idx, *num_tokens, *tokens_per_expert;
    void *d_x_shared, *d_x_routed, *d_gate_shared, *d_gate_fp8, *d_gate_sc, *d_up_shared, *d_up_fp8, *d_up_sc, *d_hidden_shared,
         *d_hidden_routed, *d_y_fp8, *d_y_sc, *d_w_shared_gate, *d_w_gate, *d_w_shared_up, *d_w_up, *d_w_shared_down, *d_w_down;
    void* workspace;
    size_t workspace_bytes;
} mx8_moe_bwd_args;
MX8_API size_t mx8_moe_fwd_workspace_bytes(const mx8_moe_dims* dims);
MX8_API int mx8_moe_fwd(const mx8_moe_fwd_args* args, void* stream);
MX8_API size_t mx8_moe_bwd_workspace_bytes(const mx8_moe_dims* dims);
MX8_API int mx8_moe_bwd(const mx8_moe_bwd_args* args, void* stream);

/* Host-buffer forms.  The reference's harnesses keep tensors on the device and never move them
 * inside a timed region (blackwell-ultra/019-mxfp8-quantize.py:59-84,
 * blackwell/047-mxfp8-mma-2cta-MNK128-polished.py:127-176); a caller whose data lives in host
 * memory uses these instead of three serial steps (copy in, kernel, copy out).  The matrix is cut
 * into bands of `band_rows` rows (a multiple of 128); inbound copy, kernel and outbound copy of
 * successive bands overlap on three streams, so both directions of the PCIe link are busy at once.
 *   - `*_host` pointers are HOST memory with the layouts of mx8_quantize / mx8_gemm (page-locked
 *     memory is needed for the copies to be asynchronous);
 *   - `workspace` is DEVICE memory of at least mx8_*_host_workspace(...) bytes, used for two
 *     alternating band buffers (and, for the GEMM, B with its scales); the call allocates no memory;
 *   - the GEMM form computes C in blocks of band_rows rows of A by band_rows rows of B and sends A band 0
 *     and the B bands first, so its outbound copies begin once two bands have arrived;
 *   - earlier work on `stream` precedes the first copy and `stream` waits for the last one.  Two
 *     copy streams per device are created on first use and kept. */
MX8_API size_t mx8_quantize_host_workspace(int N, int band_rows);
MX8_API int mx8_quantize_host(const void* x_host, int M, int N, void* fp8_host, void* sc_host, void* fp8_t_host,
                              void* sc_t_host, int scale_mode, int band_rows, void* workspace,
                              size_t workspace_bytes, void* stream);
MX8_API size_t mx8_gemm_host_workspace(int N, int K, int band_rows, int c_dtype);
MX8_API int mx8_gemm_host(const void* A_host, const void* A_sc_host, const void* B_host, const void* B_sc_host,
                          void* C_host, int M, int N, int K, int c_dtype, int band_rows, void* workspace,
                          size_t workspace_bytes, void* stream);

/* C = dequant(quantize(A_bf16)) . dequant(B)^T: the GEMM for an activation that is still bf16 [M][K].
 * A is quantized row-wise (reference rule) into `workspace` (DEVICE memory, mx8_gemm_a_bf16_workspace(M, K)
 * bytes: the E4M3 bytes, then the scale tiles), then mx8_gemm runs; two launches on `stream`, same result
 * as calling mx8_quantize and mx8_gemm.  Stands in for a GEMM with a quantizing prologue; the reference
 * quantizes in separate kernels too (blackwell-ultra/022-…-mxfp8-bw.cu:717-828 before :1399-1736).
 * mx8_gemm_a_bf16_fused is the same product with the quantization done inside the GEMM's main loop (eight
 * converter warps turn every bf16 A tile, fetched into a two-slot staging ring, into E4M3 + scale bytes in shared
 * memory): no workspace and one launch, bit-identical output, at the price of four pipeline stages instead of
 * six; measured at about a third of the two-launch form's rate, so nothing in the library calls it. */
MX8_API int mx8_gemm_a_bf16_fused(const void* A_bf16, const void* B, const void* B_sc, void* C, int M, int N, int K,
                                  int c_dtype, void* stream);
MX8_API size_t mx8_gemm_a_bf16_workspace(int M, int K);
MX8_API int mx8_gemm_a_bf16(const void* A_bf16, const void* B, const void* B_sc, void* C, int M, int N, int K, int c_dtype,
                            void* workspace, size_t workspace_bytes, void* stream);

/* Measurement aid, no counterpart in the reference: queues one launch in which every CTA pair of the device
 * issues k_steps (a multiple of 8) K steps of the GEMM's main loop, four tcgen05.mma.cta_group::2.kind::mxf8f6f4
 * .block_scale of a 256 x 256 tile each, on operands resident in shared memory; no global traffic, no epilogue.
 * *flops_out = operations of the launch; timed by the caller with events it gives the tensor-core roof the
 * benchmark reports the GEMM against (the data sheet's 4.5 PFLOP/s assumes a clock the power cap does not allow). */
MX8_API int mx8_probe_mma_peak(int k_steps, double* flops_out, void* stream);

/* Exercises the library's failure reporting without a fault: queues a one-block kernel that waits, through the
 * bounded wait all kernels here use, on a barrier nothing ever signals.  After limit_us microseconds (1 .. 1 000 000)
 * the wait gives up, the kernel records code 8 in the device status word and returns normally; the next
 * mx8_device_status call then answers MX8_ERR_DEVICE_TIMEOUT with status 8 and clears the word, and the device
 * stays usable.  The reference's waits are unbounded (blackwell-ultra/022-…-mxfp8-bw.cu:703-711); no counterpart. */
MX8_API int mx8_selftest_bounded_wait(unsigned limit_us, void* stream);

/* Synchronizes `stream`, then reads and clears the current device's status word: 0 = healthy,
 * otherwise the code of the first bounded wait that expired (see csrc/mx8_ptx.cuh).
 * Returns MX8_OK, MX8_ERR_DEVICE_TIMEOUT (status != 0) or MX8_ERR_CUDA. */
MX8_API int mx8_device_status(int* status_out, void* stream);

MX8_API const char* mx8_strerror(int code);
MX8_API const char* mx8_last_cuda_error(void); /* text of the last CUDA failure seen by this thread */
MX8_API const char* mx8_version(void);

#ifdef __cplusplus
}
#endif
#endif /* MX8_H_ */
