// Per-device state of the library (SM count, status word), error strings, and a self-test of the
// bounded-wait mechanism that every kernel's pipeline relies on.
#include <cuda_runtime.h>
#include <cudaTypedefs.h>
#include <stdlib.h>

#include <mutex>

#include "nvfp4_internal.h"
#include "ptx_sm100.cuh"

namespace nvfp4 {

namespace {
constexpr int MAX_DEV = 64;
std::mutex g_mu;
int g_sms[MAX_DEV] = {};
int* g_status_host[MAX_DEV] = {};
int* g_status_dev[MAX_DEV] = {};
}  // namespace

int sm_count(int dev) {
    if (dev < 0 || dev >= MAX_DEV) return 1;
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_sms[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
        g_sms[dev] = n;
    }
    return g_sms[dev];
}

int* status_word(int dev) {
    if (dev < 0 || dev >= MAX_DEV) return nullptr;
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_status_dev[dev]) {
        int* h = nullptr;
        if (cudaHostAlloc((void**)&h, sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess)
            return nullptr;
        *h = 0;
        int* d = nullptr;
        if (cudaHostGetDevicePointer((void**)&d, h, 0) != cudaSuccess) {
            cudaFreeHost(h);
            return nullptr;
        }
        g_status_host[dev] = h;
        g_status_dev[dev] = d;
    }
    return g_status_dev[dev];
}

int* status_word_if_allocated(int dev) {
    if (dev < 0 || dev >= MAX_DEV) return nullptr;
    std::lock_guard<std::mutex> lk(g_mu);
    return g_status_dev[dev];
}

void free_status_words() {
    std::lock_guard<std::mutex> lk(g_mu);
    for (int dev = 0; dev < MAX_DEV; dev++) {
        if (g_status_host[dev]) cudaFreeHost(g_status_host[dev]);
        g_status_host[dev] = nullptr;
        g_status_dev[dev] = nullptr;
    }
}

unsigned long long wait_budget_ns() {
    static unsigned long long v = [] {
        const char* e = getenv("NVFP4_WAIT_BUDGET_MS");
        long ms = e ? atol(e) : 2000;
        if (ms < 1) ms = 1;
        if (ms > 60000) ms = 60000;
        return (unsigned long long)ms * 1000000ull;
    }();
    return v;
}

int encode_tiled(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base, const uint64_t* dims,
                 const uint64_t* strides, const uint32_t* box, CUtensorMapSwizzle swizzle) {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            f = nullptr;
        return (PFN_cuTensorMapEncodeTiled_v12000)f;
    }();
    if (!fn || rank < 1 || rank > 5) return NVFP4_ERR_TENSORMAP;
    cuuint64_t d[5], s[4];
    cuuint32_t b[5], es[5] = {1, 1, 1, 1, 1};
    for (int i = 0; i < rank; i++) { d[i] = dims[i]; b[i] = box[i]; }
    for (int i = 0; i + 1 < rank; i++) s[i] = strides[i];
    CUresult r = fn(map, dtype, (cuuint32_t)rank, const_cast<void*>(base), d, s, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? NVFP4_OK : NVFP4_ERR_TENSORMAP;
}

// One thread waits on an mbarrier that nothing ever arrives on: the wait must expire within the
// budget and leave DEV_SELFTEST_TIMEOUT in the status word, with the context still usable.
__global__ void wait_selftest_kernel(int* status, unsigned long long budget_ns, unsigned long long* elapsed_ns) {
    __shared__ __align__(8) uint64_t bar;
    const uint32_t b = smem_u32(&bar);
    mbar_init(b, 1);
    fence_mbar_init();
    const uint64_t t0 = globaltimer_ns();
    const bool ok = mbar_wait(b, 0, budget_ns);
    *elapsed_ns = globaltimer_ns() - t0;
    if (!ok) report_status(status, DEV_SELFTEST_TIMEOUT);
}

}  // namespace nvfp4

using namespace nvfp4;

extern "C" int nvfp4_device_status(int dev, int clear) {
    if (dev < 0 || dev >= MAX_DEV) return NVFP4_ERR_SHAPE;
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_status_host[dev]) return 0;
    int v = *(volatile int*)g_status_host[dev];
    if (clear) *(volatile int*)g_status_host[dev] = 0;
    return v;
}

extern "C" int nvfp4_wait_selftest(int budget_ms, double* elapsed_ms, void* stream) {
    if (budget_ms < 1 || budget_ms > 2000) return NVFP4_ERR_SHAPE;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    int* st = status_word(dev);
    if (!st) return NVFP4_ERR_INTERNAL;
    unsigned long long* el = nullptr;
    e = cudaMalloc((void**)&el, sizeof(*el));
    if (e != cudaSuccess) return (int)e;
    wait_selftest_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(st, (unsigned long long)budget_ms * 1000000ull, el);
    unsigned long long h = 0;
    e = cudaMemcpyAsync(&h, el, sizeof(h), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    cudaFree(el);
    if (e != cudaSuccess) return (int)e;
    if (elapsed_ms) *elapsed_ms = (double)h * 1e-6;
    return NVFP4_OK;
}

extern "C" const char* nvfp4_strerror(int code) {
    switch (code) {
        case NVFP4_OK: return "ok";
        case NVFP4_ERR_NULL: return "null pointer argument";
        case NVFP4_ERR_SHAPE: return "invalid shape argument";
        case NVFP4_ERR_K_MULTIPLE: return "K is not a multiple of the kernel's K granularity";
        case NVFP4_ERR_N_MULTIPLE: return "N is not a multiple of 128";
        case NVFP4_ERR_ALIGN: return "pointer is not sufficiently aligned";
        case NVFP4_ERR_UNSUPPORTED: return "size outside the supported range";
        case NVFP4_ERR_TENSORMAP: return "cuTensorMapEncodeTiled failed";
        case NVFP4_ERR_INTERNAL: return "internal error";
        case NVFP4_ERR_TOO_MANY_GROUPS: return "too many groups";
        case DEV_TIMEOUT_PRODUCER: return "device: producer wait expired";
        case DEV_TIMEOUT_CONSUMER: return "device: consumer wait expired";
        case DEV_TIMEOUT_EPILOGUE: return "device: epilogue wait expired";
        case DEV_TIMEOUT_MMA_ACC: return "device: accumulator wait expired";
        case DEV_SELFTEST_TIMEOUT: return "device: self-test wait expired (expected)";
        default: break;
    }
    if (code > 0) return cudaGetErrorString((cudaError_t)code);
    return "unknown error";
}

extern "C" int nvfp4_abi_version(void) { return NVFP4_ABI_VERSION; }
