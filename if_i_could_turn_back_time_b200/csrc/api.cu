// Version, error text, device queries, workspace sizing.
#include "common.cuh"
#include <mutex>

int jq_sm_count() {
    static int cache[64];
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return JQ_SM_COUNT_FALLBACK;
    std::lock_guard<std::mutex> lk(mu);
    if (cache[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = JQ_SM_COUNT_FALLBACK;
        cache[dev] = n;
    }
    return cache[dev];
}

extern "C" int jq_version(void) { return JQ_VERSION; }

extern "C" const char *jq_strerror(int status) {
    switch (status) {
        case JQ_OK: return "ok";
        case JQ_ERR_NULL_PTR: return "null pointer argument";
        case JQ_ERR_BAD_SHAPE: return "bad shape (N, K, B, group size or rotation block)";
        case JQ_ERR_BAD_ALIGN: return "pointer not aligned (packed weights need 16 bytes)";
        case JQ_ERR_BAD_DTYPE: return "unsupported element type";
        case JQ_ERR_UNSUPPORTED: return "combination not supported by this build";
        case JQ_ERR_WORKSPACE: return "workspace too small";
        case JQ_ERR_TIMEOUT: return "device-side wait gave up";
        case JQ_ERR_NOMEM: return "host allocation failed";
        case JQ_ERR_SCRATCH_LIMIT: return "problem needs more than the library's built-in scratch array (JQ_NOALLOC_SCRATCH_BYTES)";
        default: break;
    }
    if (status <= JQ_ERR_CUDA_BASE) return cudaGetErrorString((cudaError_t)(JQ_ERR_CUDA_BASE - status));
    return "unknown status";
}

