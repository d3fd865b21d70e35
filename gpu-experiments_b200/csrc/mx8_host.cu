// Host-side plumbing behind the C ABI: error text, device checks, tensor-map encoding and the
// per-device status word that bounded device waits report into.
#include <cstdio>
#include <cstring>
#include <mutex>

#include <atomic>

#include "mx8_host.cuh"
#include "mx8_ptx.cuh"

namespace mx8 {

static thread_local char g_cuda_err[256] = "";

void note_cuda_error(const char* what, const char* detail) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", what, detail ? detail : "?");
}

// The status word lives in a file-scope device variable: no allocation, one per device that
// loads the library.
__device__ int g_device_status = 0;

int* device_status_ptr() {
    int* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_device_status);
    if (e != cudaSuccess) {
        note_cuda_error("cudaGetSymbolAddress", cudaGetErrorString(e));
        return nullptr;
    }
    return p;
}

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
        if (e == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(p);
        else note_cuda_error("cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)", cudaGetErrorString(e));
    });
    return fn;
}

int make_tmap(CUtensorMap* out, CUtensorMapDataType dt, int rank, const void* base, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swz, CUtensorMapL2promotion l2) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return MX8_ERR_CUDA;
    cuuint64_t d[5];
    cuuint64_t s[4];
    cuuint32_t b[5];
    cuuint32_t es[5];
    for (int i = 0; i < rank; ++i) {
        d[i] = dims[i];
        b[i] = box[i];
        es[i] = 1;
        if (i + 1 < rank) s[i] = strides_bytes[i];
    }
    CUresult r = fn(out, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), d, s, b, es,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swz, l2, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char msg[64];
        snprintf(msg, sizeof(msg), "CUresult %d", static_cast<int>(r));
        note_cuda_error("cuTensorMapEncodeTiled", msg);
        return MX8_ERR_CUDA;
    }
    return MX8_OK;
}

// filled on first use; two threads racing here write the same values
static std::atomic<int> g_sm_count[64];
static std::atomic<int> g_cc_major[64];

static int query_device(int* sm, int* major) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        note_cuda_error("cudaGetDevice", cudaGetErrorString(e));
        return MX8_ERR_CUDA;
    }
    if (dev < 0 || dev >= 64) return MX8_ERR_UNSUPPORTED;
    if (g_sm_count[dev].load(std::memory_order_acquire) == 0) {
        int s = 0, m = 0;
        e = cudaDeviceGetAttribute(&s, cudaDevAttrMultiProcessorCount, dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&m, cudaDevAttrComputeCapabilityMajor, dev);
        if (e != cudaSuccess) {
            note_cuda_error("cudaDeviceGetAttribute", cudaGetErrorString(e));
            return MX8_ERR_CUDA;
        }
        g_cc_major[dev].store(m, std::memory_order_relaxed);
        g_sm_count[dev].store(s, std::memory_order_release);
    }
    *sm = g_sm_count[dev].load(std::memory_order_acquire);
    *major = g_cc_major[dev].load(std::memory_order_relaxed);
    return MX8_OK;
}

int sm_count() {
    int s = 0, m = 0;
    return query_device(&s, &m) == MX8_OK ? s : 0;
}

int check_device_sm100() {
    int s = 0, m = 0;
    int rc = query_device(&s, &m);
    if (rc != MX8_OK) return rc;
    return m == 10 ? MX8_OK : MX8_ERR_UNSUPPORTED;
}

}  // namespace mx8

namespace mx8 {
// One CTA waits on an mbarrier nobody will ever arrive on, through the same bounded wait every kernel of the
// library uses, with a short limit: the wait gives up, records DEV_TIMEOUT_SELFTEST in the status word and the
// kernel returns normally.
__global__ void selftest_wait_kernel(unsigned long long limit_ns, int* status) {
    __shared__ alignas(8) unsigned long long bar_storage;
    __shared__ int abort_flag;
    const uint32_t bar = smem_u32(&bar_storage);
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(bar, 1);
        fence_mbar_init();
    }
    __syncthreads();
    const AbortCtl ab{&abort_flag, status};
    if (threadIdx.x == 0) mbar_wait(bar, 0, ab, DEV_TIMEOUT_SELFTEST, limit_ns);
    __syncthreads();
}
}  // namespace mx8

extern "C" {

int mx8_selftest_bounded_wait(unsigned limit_us, void* stream) {
    using namespace mx8;
    if (limit_us == 0 || limit_us > 1000000u) return MX8_ERR_ARG;       // at most a second
    int rc = check_device_sm100();
    if (rc != MX8_OK) return rc;
    int* status = device_status_ptr();
    if (!status) return MX8_ERR_CUDA;
    selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<unsigned long long>(limit_us) * 1000ull, status);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        note_cuda_error("selftest launch", cudaGetErrorString(e));
        return MX8_ERR_CUDA;
    }
    return MX8_OK;
}

int mx8_device_status(int* status_out, void* stream) {
    cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) {
        mx8::note_cuda_error("cudaStreamSynchronize", cudaGetErrorString(e));
        return MX8_ERR_CUDA;
    }
    int v = 0;
    e = cudaMemcpyFromSymbol(&v, mx8::g_device_status, sizeof(int));
    if (e == cudaSuccess && v != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(mx8::g_device_status, &zero, sizeof(int));
    }
    if (e != cudaSuccess) {
        mx8::note_cuda_error("cudaMemcpy{From,To}Symbol", cudaGetErrorString(e));
        return MX8_ERR_CUDA;
    }
    if (status_out) *status_out = v;
    return v == 0 ? MX8_OK : MX8_ERR_DEVICE_TIMEOUT;
}

const char* mx8_strerror(int code) {
    switch (code) {
        case MX8_OK: return "ok";
        case MX8_ERR_ARG: return "invalid argument (null pointer, bad enum value or no output requested)";
        case MX8_ERR_SHAPE: return "dimension is not a positive multiple of 128";
        case MX8_ERR_ALIGN: return "pointer is not 16-byte aligned";
        case MX8_ERR_CUDA: return "CUDA call failed (see mx8_last_cuda_error)";
        case MX8_ERR_UNSUPPORTED: return "current device is not compute capability 10.x (sm_100a required)";
        case MX8_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel expired (see mx8_device_status)";
        case MX8_ERR_LIMIT: return "problem exceeds a built-in size limit (see mx8_last_cuda_error)";
        default: return "unknown mx8 status code";
    }
}

const char* mx8_last_cuda_error(void) { return mx8::g_cuda_err; }

const char* mx8_version(void) { return "mx8 0.1 (sm_100a)"; }

}  // extern "C"
