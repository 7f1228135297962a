// Status strings, thread-local last-error text and the per-device property cache.
#include "ko_internal.h"

#include <mutex>
#include <string>

namespace ko {
namespace {
thread_local std::string g_last_error;
std::mutex g_info_mutex;
DeviceInfo g_info[64];
}  // namespace

int fail(int status, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    std::vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return status;
}

int fail_cuda(cudaError_t err, const char *what) {
    return fail(KO_ERR_CUDA, "%s failed: %s (%s)", what, cudaGetErrorName(err), cudaGetErrorString(err));
}

int current_device_info(DeviceInfo *out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(KO_ERR_NO_DEVICE, "cudaGetDevice failed: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return fail(KO_ERR_NO_DEVICE, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_info_mutex);
    DeviceInfo &info = g_info[dev];
    if (info.device != dev) {
        DeviceInfo fresh;
        KO_CUDA(cudaDeviceGetAttribute(&fresh.sm_count, cudaDevAttrMultiProcessorCount, dev));
        KO_CUDA(cudaDeviceGetAttribute(&fresh.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
        KO_CUDA(cudaDeviceGetAttribute(&fresh.cc_minor, cudaDevAttrComputeCapabilityMinor, dev));
        KO_CUDA(cudaDeviceGetAttribute(&fresh.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        if (fresh.cc_major != 10)
            return fail(KO_ERR_NO_DEVICE, "device %d is sm_%d%d; this library contains sm_100a code only", dev,
                        fresh.cc_major, fresh.cc_minor);
        fresh.device = dev;
        info = fresh;
    }
    *out = info;
    return KO_OK;
}
}  // namespace ko

#include <map>
#include <utility>

#include "row_launch.h"

namespace ko {
int ensure_dynamic_smem(const void *kernel, size_t bytes) {
    static std::mutex mu;
    static std::map<std::pair<const void *, int>, size_t> configured;
    int dev = 0;
    KO_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    size_t &have = configured[{kernel, dev}];
    if (bytes > have) {
        KO_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
        have = bytes;
    }
    return KO_OK;
}
}  // namespace ko

extern "C" {

const char *ko_status_string(int status) {
    switch (status) {
        case KO_OK: return "KO_OK";
        case KO_ERR_INVALID_ARG: return "KO_ERR_INVALID_ARG";
        case KO_ERR_ALIGN: return "KO_ERR_ALIGN";
        case KO_ERR_SHAPE: return "KO_ERR_SHAPE";
        case KO_ERR_CUDA: return "KO_ERR_CUDA";
        case KO_ERR_TIMEOUT: return "KO_ERR_TIMEOUT";
        case KO_ERR_NO_DEVICE: return "KO_ERR_NO_DEVICE";
        default: return "KO_ERR_UNKNOWN";
    }
}

const char *ko_last_error_string(void) { return ko::g_last_error.c_str(); }

int ko_version(void) { return 100; /* 0.1.0 */ }

}  // extern "C"
