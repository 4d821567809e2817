// Error channel and device queries of the kernel library.
#include "common.cuh"

#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include <mutex>

static thread_local char g_last_error[512] = "";

void llm_set_error(const char* format, ...) {
    va_list args;
    va_start(args, format);
    vsnprintf(g_last_error, sizeof(g_last_error), format, args);
    va_end(args);
}

int llm_check_launch(const char* what) {
    cudaError_t status = cudaGetLastError();
    if (status != cudaSuccess) {
        llm_set_error("%s: %s", what, cudaGetErrorString(status));
        return (int)status;
    }
    return LLM_OK;
}

bool llm_pdl_enabled() {
    static int enabled = -1;
    if (enabled < 0) {
        const char* value = getenv("LLMSERVER_B200_PDL");
        enabled = (value != nullptr && value[0] == '0') ? 0 : 1;
    }
    return enabled == 1;
}

namespace {
struct SharedLimit {
    const void* kernel;
    int device;
    size_t bytes;
};
constexpr int kMaxLimits = 256;
SharedLimit g_limits[kMaxLimits];
int g_limit_count = 0;
std::mutex g_limit_lock;
}  // namespace

int llm_raise_shared_limit(const void* kernel, size_t bytes, const char* what, bool max_carveout) {
    int device = 0;
    cudaError_t status = cudaGetDevice(&device);
    if (status != cudaSuccess) {
        llm_set_error("%s: cannot tell the current device: %s", what, cudaGetErrorString(status));
        return (int)status;
    }
    std::lock_guard<std::mutex> guard(g_limit_lock);
    SharedLimit* entry = nullptr;
    for (int i = 0; i < g_limit_count; ++i)
        if (g_limits[i].kernel == kernel && g_limits[i].device == device) entry = &g_limits[i];
    if (entry != nullptr && entry->bytes >= bytes) return LLM_OK;
    status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (status != cudaSuccess) {
        llm_set_error("%s: cannot get %zu bytes of shared memory: %s", what, bytes, cudaGetErrorString(status));
        return (int)status;
    }
    if (max_carveout) cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (entry == nullptr && g_limit_count < kMaxLimits) entry = &g_limits[g_limit_count++];
    if (entry != nullptr) *entry = SharedLimit{kernel, device, bytes};
    return LLM_OK;
}

LLM_EXPORT const char* llm_last_error() { return g_last_error; }

// Compute capability of the current device as major * 10 + minor, or a negative CUDA error.
LLM_EXPORT int llm_device_arch() {
    int device = 0, major = 0, minor = 0;
    cudaError_t status = cudaGetDevice(&device);
    if (status == cudaSuccess) status = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
    if (status == cudaSuccess) status = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device);
    if (status != cudaSuccess) {
        llm_set_error("device query: %s", cudaGetErrorString(status));
        return -(int)status;
    }
    return major * 10 + minor;
}

LLM_EXPORT int llm_sm_count() {
    int device = 0, count = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return -1;
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return -1;
    return count;
}
