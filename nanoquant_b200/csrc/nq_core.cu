// Library-wide pieces of the C ABI: status strings, CUDA error text, device info.
#include <cstdio>
#include <cstring>

#include "nq_common.cuh"

namespace nq {

static thread_local char g_cuda_error[512] = "";

void set_cuda_error(cudaError_t e, const char* where) {
    snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s (%s)", where, cudaGetErrorName(e),
             cudaGetErrorString(e));
    // clear the sticky-free error state so that the next call starts clean
    (void)cudaGetLastError();
}

int sm_count() {
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace nq

extern "C" {

int nq_abi_version(void) { return 2; }

const char* nq_strerror(int status) {
    switch (status) {
        case NQ_OK: return "ok";
        case NQ_ERR_NULL: return "a required pointer is NULL";
        case NQ_ERR_SHAPE: return "invalid shape (non-positive or not a required multiple)";
        case NQ_ERR_DTYPE: return "unsupported dtype or layout id";
        case NQ_ERR_ALIGN: return "pointer not 16-byte aligned";
        case NQ_ERR_SCRATCH: return "scratch or workspace buffer too small";
        case NQ_ERR_CUDA: return "CUDA runtime error (see nq_last_cuda_error)";
        case NQ_ERR_TIMEOUT: return "a bounded device-side wait gave up";
        case NQ_ERR_UNSUPPORTED: return "shape not supported by the kernels";
        case NQ_ERR_TOO_LARGE: return "size beyond the fixed maximum of this entry point";
        default: return "unknown status";
    }
}

const char* nq_last_cuda_error(void) { return nq::g_cuda_error; }

}  // extern "C"
