// Internal helpers shared by the C-ABI translation units: thread-local error text, argument
// checks, per-device property cache.  Not part of the public interface.
#pragma once

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include <cuda_runtime.h>

#include "../../include/ko_b200.h"

namespace ko {

// records the message for ko_last_error_string() and returns `status`
int fail(int status, const char *fmt, ...) __attribute__((format(printf, 2, 3)));
int fail_cuda(cudaError_t err, const char *what);

struct DeviceInfo {
    int device = -1;
    int sm_count = 0;
    int cc_major = 0, cc_minor = 0;
    int max_smem_optin = 0;
};
// properties of the current device (cached per device ordinal); status != KO_OK on failure
int current_device_info(DeviceInfo *out);

// device status words (device_status.cu): 0 = tensor-core GEMM, 1 = staged row operators
constexpr int kStatusWordCount = 4;
int device_status_word(int which, unsigned int **out);

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace ko

#define KO_REQUIRE(cond, status, ...)                         \
    do {                                                      \
        if (!(cond)) return ::ko::fail((status), __VA_ARGS__); \
    } while (0)

#define KO_CUDA(call)                                                   \
    do {                                                                \
        cudaError_t ko_err__ = (call);                                  \
        if (ko_err__ != cudaSuccess) return ::ko::fail_cuda(ko_err__, #call); \
    } while (0)

// checks the launch that was just enqueued
#define KO_CHECK_LAUNCH(name)                                                  \
    do {                                                                       \
        cudaError_t ko_err__ = cudaGetLastError();                             \
        if (ko_err__ != cudaSuccess) return ::ko::fail_cuda(ko_err__, name);   \
    } while (0)
