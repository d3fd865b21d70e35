// Host-buffer forms of the quantizer and the GEMM: the matrix is cut into bands of rows (the GEMM's C
// into blocks of an A band by a B band) and the three legs of every band (host -> device copy, kernel,
// device -> host copy) run on three streams,
// so that the inbound copy of band b+1 and the outbound copy of band b-1 share the PCIe link's two
// directions with the kernel of band b.  Two device buffer sets alternate between bands.
//
// Ordering contract: work already queued on `stream` precedes the first copy, and `stream` waits for
// the last outbound copy, so the caller synchronises (or keeps queueing on) `stream` as with every
// other entry point.  The two copy streams are created once per device and kept.
#include <cstddef>
#include <mutex>
#include <vector>

#include "mx8_host.cuh"

namespace mx8 {
namespace {

struct CopyStreams {
    cudaStream_t in = nullptr, out = nullptr, out2 = nullptr;   // out2: strided copies of transposed outputs
};

int copy_streams(CopyStreams** out) {
    static CopyStreams per_device[64];
    static std::mutex mu;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        note_cuda_error("cudaGetDevice", cudaGetErrorString(e));
        return MX8_ERR_CUDA;
    }
    std::lock_guard<std::mutex> lock(mu);
    CopyStreams& cs = per_device[dev];
    if (!cs.in) {
        e = cudaStreamCreateWithFlags(&cs.in, cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&cs.out, cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&cs.out2, cudaStreamNonBlocking);
        if (e != cudaSuccess) {
            note_cuda_error("cudaStreamCreateWithFlags", cudaGetErrorString(e));
            cs = CopyStreams{};
            return MX8_ERR_CUDA;
        }
    }
    *out = &cs;
    return MX8_OK;
}

// Events of one call.  They are destroyed when the object goes out of scope; the runtime keeps an
// event alive until the work that references it has finished.
struct Events {
    std::vector<cudaEvent_t> ev;
    cudaError_t err = cudaSuccess;
    cudaEvent_t make() {
        cudaEvent_t e = nullptr;
        cudaError_t r = cudaEventCreateWithFlags(&e, cudaEventDisableTiming);
        if (r != cudaSuccess) { err = r; return nullptr; }
        ev.push_back(e);
        return e;
    }
    ~Events() {
        for (cudaEvent_t e : ev) cudaEventDestroy(e);
    }
};

struct Check {
    cudaError_t err = cudaSuccess;
    const char* what = "";
    void operator()(cudaError_t e, const char* w) {
        if (err == cudaSuccess && e != cudaSuccess) { err = e; what = w; }
    }
    int status() const {
        if (err == cudaSuccess) return MX8_OK;
        note_cuda_error(what, cudaGetErrorString(err));
        return MX8_ERR_CUDA;
    }
};

inline size_t align_up(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

// Row bounds of the bands: equal bands of R rows, the last one shorter when R does not divide M.  (Shorter
// bands at both ends, to shorten the fill and drain of the pipeline, were measured and gained nothing: with
// eight bands the link is already busy in both directions for all but a few percent of the time.)
std::vector<size_t> band_plan(size_t M, size_t R) {
    std::vector<size_t> edges{0};
    for (size_t r = R; r < M; r += R) edges.push_back(r);
    edges.push_back(M);
    return edges;
}

struct QuantBand {      // device buffers of one band (R rows)
    uint8_t *x, *q, *sc, *qt, *sct;
};

size_t quant_band_bytes(size_t R, size_t N) {
    return align_up(R * N * 2) + 2 * (align_up(R * N) + align_up(R * N / 32));
}

}  // namespace
}  // namespace mx8

extern "C" {

MX8_API size_t mx8_quantize_host_workspace(int N, int band_rows) {
    if (N <= 0 || band_rows <= 0) return 0;
    return 2 * mx8::quant_band_bytes(static_cast<size_t>(band_rows), static_cast<size_t>(N));
}

int mx8_quantize_host(const void* x_host, int M, int N, void* fp8_host, void* sc_host, void* fp8_t_host,
                      void* sc_t_host, int scale_mode, int band_rows, void* workspace, size_t workspace_bytes,
                      void* stream) {
    using namespace mx8;
    const bool want_n = fp8_host && sc_host, want_t = fp8_t_host && sc_t_host;
    if (!x_host || !workspace || (!want_n && !want_t)) return MX8_ERR_ARG;
    if ((fp8_host == nullptr) != (sc_host == nullptr) || (fp8_t_host == nullptr) != (sc_t_host == nullptr)) return MX8_ERR_ARG;
    if (M <= 0 || N <= 0 || M % 128 || N % 128 || band_rows <= 0 || band_rows % 128) return MX8_ERR_SHAPE;
    if (!aligned16(workspace)) return MX8_ERR_ALIGN;
    const size_t R = static_cast<size_t>(band_rows < M ? band_rows : M), Nn = static_cast<size_t>(N), Mm = static_cast<size_t>(M);
    if (workspace_bytes < 2 * quant_band_bytes(R, Nn)) {
        note_cuda_error("mx8_quantize_host", "workspace smaller than mx8_quantize_host_workspace(N, band_rows)");
        return MX8_ERR_LIMIT;
    }
    CopyStreams* cs = nullptr;
    int rc = copy_streams(&cs);
    if (rc != MX8_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    QuantBand buf[2];
    uint8_t* w = static_cast<uint8_t*>(workspace);
    for (int i = 0; i < 2; ++i) {
        buf[i].x = w;   w += align_up(R * Nn * 2);
        buf[i].q = w;   w += align_up(R * Nn);
        buf[i].sc = w;  w += align_up(R * Nn / 32);
        buf[i].qt = w;  w += align_up(R * Nn);
        buf[i].sct = w; w += align_up(R * Nn / 32);
    }
    const std::vector<size_t> edges = band_plan(Mm, R);
    const int bands = static_cast<int>(edges.size()) - 1;
    Events evs;
    Check ck;
    std::vector<cudaEvent_t> in_ready(bands), done(bands), out_done(bands), out2_done(bands);
    cudaEvent_t start = evs.make();
    for (int b = 0; b < bands; ++b) { in_ready[b] = evs.make(); done[b] = evs.make(); out_done[b] = evs.make(); out2_done[b] = evs.make(); }
    if (evs.err != cudaSuccess) { note_cuda_error("cudaEventCreateWithFlags", cudaGetErrorString(evs.err)); return MX8_ERR_CUDA; }

    ck(cudaEventRecord(start, s), "cudaEventRecord");
    ck(cudaStreamWaitEvent(cs->in, start, 0), "cudaStreamWaitEvent");
    ck(cudaStreamWaitEvent(cs->out, start, 0), "cudaStreamWaitEvent");
    ck(cudaStreamWaitEvent(cs->out2, start, 0), "cudaStreamWaitEvent");
    const uint8_t* xh = static_cast<const uint8_t*>(x_host);
    for (int b = 0; b < bands && ck.err == cudaSuccess; ++b) {
        const QuantBand& B = buf[b & 1];
        const size_t r0 = edges[b], rows = edges[b + 1] - edges[b];
        // inbound: the buffer is free once the kernel of band b-2 has read it
        if (b >= 2) ck(cudaStreamWaitEvent(cs->in, done[b - 2], 0), "cudaStreamWaitEvent");
        ck(cudaMemcpyAsync(B.x, xh + r0 * Nn * 2, rows * Nn * 2, cudaMemcpyHostToDevice, cs->in), "cudaMemcpyAsync(h2d)");
        ck(cudaEventRecord(in_ready[b], cs->in), "cudaEventRecord");
        // kernel: outputs of band b-2 must have left the buffers
        ck(cudaStreamWaitEvent(s, in_ready[b], 0), "cudaStreamWaitEvent");
        if (b >= 2) ck(cudaStreamWaitEvent(s, out_done[b - 2], 0), "cudaStreamWaitEvent");
        if (b >= 2) ck(cudaStreamWaitEvent(s, out2_done[b - 2], 0), "cudaStreamWaitEvent");
        if (ck.err != cudaSuccess) break;
        rc = mx8_quantize(B.x, 1, static_cast<int>(rows), N, want_n ? B.q : nullptr, want_n ? B.sc : nullptr,
                          want_t ? B.qt : nullptr, want_t ? B.sct : nullptr, scale_mode, s);
        if (rc != MX8_OK) break;
        ck(cudaEventRecord(done[b], s), "cudaEventRecord");
        // outbound: contiguous row-wise outputs on one stream, the strided transposed ones on
        // another, so that the per-row overhead of the strided copies hides behind the bulk ones
        ck(cudaStreamWaitEvent(cs->out, done[b], 0), "cudaStreamWaitEvent");
        ck(cudaStreamWaitEvent(cs->out2, done[b], 0), "cudaStreamWaitEvent");
        if (want_n) {
            ck(cudaMemcpyAsync(static_cast<uint8_t*>(fp8_host) + r0 * Nn, B.q, rows * Nn, cudaMemcpyDeviceToHost, cs->out), "cudaMemcpyAsync(d2h)");
            ck(cudaMemcpyAsync(static_cast<uint8_t*>(sc_host) + r0 * Nn / 32, B.sc, rows * Nn / 32, cudaMemcpyDeviceToHost, cs->out), "cudaMemcpyAsync(d2h)");
        }
        if (want_t) {
            // the band is a block of `rows` columns of the transposed outputs
            ck(cudaMemcpy2DAsync(static_cast<uint8_t*>(fp8_t_host) + r0, Mm, B.qt, rows, rows, Nn, cudaMemcpyDeviceToHost, cs->out2), "cudaMemcpy2DAsync(d2h)");
            ck(cudaMemcpy2DAsync(static_cast<uint8_t*>(sc_t_host) + r0 / 128 * 512, Mm / 128 * 512, B.sct, rows / 128 * 512, rows / 128 * 512,
                                 Nn / 128, cudaMemcpyDeviceToHost, cs->out2), "cudaMemcpy2DAsync(d2h)");
        }
        ck(cudaEventRecord(out_done[b], cs->out), "cudaEventRecord");
        ck(cudaEventRecord(out2_done[b], cs->out2), "cudaEventRecord");
    }
    // whatever was queued must finish before the caller's stream moves on (also on the error path,
    // where the buffers may be released by the caller right after the return)
    cudaEvent_t tail_in = evs.make(), tail_out = evs.make(), tail_out2 = evs.make();
    if (tail_in && tail_out && tail_out2) {
        ck(cudaEventRecord(tail_in, cs->in), "cudaEventRecord");
        ck(cudaEventRecord(tail_out, cs->out), "cudaEventRecord");
        ck(cudaEventRecord(tail_out2, cs->out2), "cudaEventRecord");
        ck(cudaStreamWaitEvent(s, tail_in, 0), "cudaStreamWaitEvent");
        ck(cudaStreamWaitEvent(s, tail_out, 0), "cudaStreamWaitEvent");
        ck(cudaStreamWaitEvent(s, tail_out2, 0), "cudaStreamWaitEvent");
    }
    if (rc != MX8_OK) return rc;
    return ck.status();
}

size_t mx8_gemm_host_workspace(int N, int K, int band_rows, int c_dtype) {
    if (N <= 0 || K <= 0 || band_rows <= 0) return 0;
    using mx8::align_up;
    const size_t R = band_rows, Nn = N, Kk = K, es = c_dtype == MX8_C_F32 ? 4 : 2;
    return align_up(Nn * Kk) + align_up(Nn * Kk / 32) + 2 * (align_up(R * Kk) + align_up(R * Kk / 32) + align_up(R * Nn * es));
}

int mx8_gemm_host(const void* A_host, const void* A_sc_host, const void* B_host, const void* B_sc_host, void* C_host,
                  int M, int N, int K, int c_dtype, int band_rows, void* workspace, size_t workspace_bytes, void* stream) {
    using namespace mx8;
    if (!A_host || !A_sc_host || !B_host || !B_sc_host || !C_host || !workspace) return MX8_ERR_ARG;
    if (c_dtype != MX8_C_BF16 && c_dtype != MX8_C_F32) return MX8_ERR_ARG;
    if (M <= 0 || N <= 0 || K <= 0 || M % 128 || N % 128 || K % 128 || band_rows <= 0 || band_rows % 128) return MX8_ERR_SHAPE;
    if (!aligned16(workspace)) return MX8_ERR_ALIGN;
    const size_t R = static_cast<size_t>(band_rows < M ? band_rows : M), Nn = N, Kk = K, Mm = M, es = c_dtype == MX8_C_F32 ? 4 : 2;
    if (workspace_bytes < mx8_gemm_host_workspace(N, K, static_cast<int>(R), c_dtype)) {
        note_cuda_error("mx8_gemm_host", "workspace smaller than mx8_gemm_host_workspace(N, K, band_rows, c_dtype)");
        return MX8_ERR_LIMIT;
    }
    CopyStreams* cs = nullptr;
    int rc = copy_streams(&cs);
    if (rc != MX8_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    uint8_t* w = static_cast<uint8_t*>(workspace);
    uint8_t* b_dev = w;    w += align_up(Nn * Kk);
    uint8_t* bsc_dev = w;  w += align_up(Nn * Kk / 32);
    uint8_t *a_dev[2], *asc_dev[2], *c_dev[2];
    for (int i = 0; i < 2; ++i) {
        a_dev[i] = w;   w += align_up(R * Kk);
        asc_dev[i] = w; w += align_up(R * Kk / 32);
        c_dev[i] = w;   w += align_up(R * Nn * es);
    }
    // C is computed in blocks of (band of A rows) x (band of B rows): the first block needs only one band of
    // each operand, so the outbound copies start after 2 bands have arrived instead of after all of B.
    // Inbound order: A band 0, every B band, then the other A bands; B stays resident.
    const std::vector<size_t> edges = band_plan(Mm, R);
    const size_t Nb = R < Nn ? R : Nn;
    const std::vector<size_t> nedges = band_plan(Nn, Nb);
    const int bands = static_cast<int>(edges.size()) - 1, nbands = static_cast<int>(nedges.size()) - 1;
    const int blocks = bands * nbands;
    Events evs;
    Check ck;
    std::vector<cudaEvent_t> a_ready(bands), band_done(bands), b_ready(nbands), done(blocks), out_done(blocks);
    cudaEvent_t start = evs.make();
    for (auto* v : {&a_ready, &band_done, &b_ready, &done, &out_done})
        for (cudaEvent_t& e : *v) e = evs.make();
    if (evs.err != cudaSuccess) { note_cuda_error("cudaEventCreateWithFlags", cudaGetErrorString(evs.err)); return MX8_ERR_CUDA; }

    ck(cudaEventRecord(start, s), "cudaEventRecord");
    ck(cudaStreamWaitEvent(cs->in, start, 0), "cudaStreamWaitEvent");
    ck(cudaStreamWaitEvent(cs->out, start, 0), "cudaStreamWaitEvent");
    for (int b = 0; b < bands && ck.err == cudaSuccess && rc == MX8_OK; ++b) {
        const int i = b & 1;
        const size_t r0 = edges[b], rows = edges[b + 1] - edges[b];
        // the A buffer is free once every block of band b-2 has been computed
        if (b >= 2) ck(cudaStreamWaitEvent(cs->in, band_done[b - 2], 0), "cudaStreamWaitEvent");
        ck(cudaMemcpyAsync(a_dev[i], static_cast<const uint8_t*>(A_host) + r0 * Kk, rows * Kk, cudaMemcpyHostToDevice, cs->in), "cudaMemcpyAsync(h2d)");
        ck(cudaMemcpyAsync(asc_dev[i], static_cast<const uint8_t*>(A_sc_host) + r0 * Kk / 32, rows * Kk / 32, cudaMemcpyHostToDevice, cs->in), "cudaMemcpyAsync(h2d)");
        ck(cudaEventRecord(a_ready[b], cs->in), "cudaEventRecord");
        if (b == 0) {
            for (int j = 0; j < nbands; ++j) {
                const size_t c0 = nedges[j], cols = nedges[j + 1] - nedges[j];
                ck(cudaMemcpyAsync(b_dev + c0 * Kk, static_cast<const uint8_t*>(B_host) + c0 * Kk, cols * Kk, cudaMemcpyHostToDevice, cs->in), "cudaMemcpyAsync(h2d)");
                ck(cudaMemcpyAsync(bsc_dev + c0 * Kk / 32, static_cast<const uint8_t*>(B_sc_host) + c0 * Kk / 32, cols * Kk / 32, cudaMemcpyHostToDevice, cs->in), "cudaMemcpyAsync(h2d)");
                ck(cudaEventRecord(b_ready[j], cs->in), "cudaEventRecord");
            }
        }
        ck(cudaStreamWaitEvent(s, a_ready[b], 0), "cudaStreamWaitEvent");
        for (int j = 0; j < nbands && ck.err == cudaSuccess; ++j) {
            const int k = b * nbands + j, cb = k & 1;
            const size_t c0 = nedges[j], cols = nedges[j + 1] - nedges[j];
            if (b == 0) ck(cudaStreamWaitEvent(s, b_ready[j], 0), "cudaStreamWaitEvent");
            if (k >= 2) ck(cudaStreamWaitEvent(s, out_done[k - 2], 0), "cudaStreamWaitEvent");   // the C buffer has left the device
            if (ck.err != cudaSuccess) break;
            rc = mx8_gemm(a_dev[i], asc_dev[i], b_dev + c0 * Kk, bsc_dev + c0 * Kk / 32, c_dev[cb], static_cast<int>(rows), static_cast<int>(cols), K,
                          c_dtype, s);
            if (rc != MX8_OK) break;
            ck(cudaEventRecord(done[k], s), "cudaEventRecord");
            ck(cudaStreamWaitEvent(cs->out, done[k], 0), "cudaStreamWaitEvent");
            ck(cudaMemcpy2DAsync(static_cast<uint8_t*>(C_host) + (r0 * Nn + c0) * es, Nn * es, c_dev[cb], cols * es, cols * es, rows,
                                 cudaMemcpyDeviceToHost, cs->out), "cudaMemcpy2DAsync(d2h)");
            ck(cudaEventRecord(out_done[k], cs->out), "cudaEventRecord");
        }
        ck(cudaEventRecord(band_done[b], s), "cudaEventRecord");
    }
    cudaEvent_t tail_in = evs.make(), tail_out = evs.make();
    if (tail_in && tail_out) {
        ck(cudaEventRecord(tail_in, cs->in), "cudaEventRecord");
        ck(cudaEventRecord(tail_out, cs->out), "cudaEventRecord");
        ck(cudaStreamWaitEvent(s, tail_in, 0), "cudaStreamWaitEvent");
        ck(cudaStreamWaitEvent(s, tail_out, 0), "cudaStreamWaitEvent");
    }
    if (rc != MX8_OK) return rc;
    return ck.status();
}

// GEMM whose A operand is still bf16: quantize A row-wise into the caller's workspace, then the block-scaled
// GEMM, both on `stream`.  Two launches; the quantize pass costs about 1 % of the product at the shapes this
// library is measured on.  The form with the conversion inside the GEMM's main loop exists as well
// (mx8_gemm_a_bf16_fused); it gives the same bytes at about a third of this form's rate.
size_t mx8_gemm_a_bf16_workspace(int M, int K) {
    if (M <= 0 || K <= 0) return 0;
    return mx8::align_up(static_cast<size_t>(M) * K) + mx8::align_up(static_cast<size_t>(M) * K / 32);
}

int mx8_gemm_a_bf16(const void* A_bf16, const void* B, const void* B_sc, void* C, int M, int N, int K, int c_dtype,
                    void* workspace, size_t workspace_bytes, void* stream) {
    using namespace mx8;
    if (!A_bf16 || !B || !B_sc || !C || !workspace) return MX8_ERR_ARG;
    if (M <= 0 || N <= 0 || K <= 0 || M % 128 || N % 128 || K % 128) return MX8_ERR_SHAPE;
    if (!aligned16(workspace)) return MX8_ERR_ALIGN;
    if (workspace_bytes < mx8_gemm_a_bf16_workspace(M, K)) {
        note_cuda_error("mx8_gemm_a_bf16", "workspace smaller than mx8_gemm_a_bf16_workspace(M, K)");
        return MX8_ERR_LIMIT;
    }
    uint8_t* a_fp8 = static_cast<uint8_t*>(workspace);
    uint8_t* a_sc = a_fp8 + align_up(static_cast<size_t>(M) * K);
    int rc = mx8_quantize(A_bf16, 1, M, K, a_fp8, a_sc, nullptr, nullptr, MX8_SCALE_RCEIL, stream);
    if (rc != MX8_OK) return rc;
    return mx8_gemm(a_fp8, a_sc, B, B_sc, C, M, N, K, c_dtype, stream);
}

}  // extern "C"
