// Shared pieces of the three stand-alone drivers: argument parsing, event timing, result lines.
// The drivers follow the reference's (fill -> H2D -> launch -> time -> report) shape
// (nn_operators/softmax/main.cu:14-74) with what it lacks: warm-up, several timed launches over
// rotating buffers (so that inputs come from HBM, not L2), a seeded fill and a result check.
#pragma once

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../common/common.h"
#include "../common/tensor.h"
#include "ko_b200.h"

namespace driver {

inline long long arg_int(int argc, char **argv, const char *name, long long fallback) {
    for (int i = 1; i + 1 < argc; ++i)
        if (std::strcmp(argv[i], name) == 0) return std::atoll(argv[i + 1]);
    return fallback;
}
inline bool arg_flag(int argc, char **argv, const char *name) {
    for (int i = 1; i < argc; ++i)
        if (std::strcmp(argv[i], name) == 0) return true;
    return false;
}

inline void require_ok(int status, const char *what) {
    if (status != KO_OK) {
        std::fprintf(stderr, "%s failed: %s (%s)\n", what, ko_status_string(status), ko_last_error_string());
        std::exit(EXIT_FAILURE);
    }
}

// median time of `iters` launches in microseconds; launch(i) enqueues the i-th call on `stream`
template <typename Launch>
double time_us(cudaStream_t stream, int warmup, int iters, Launch &&launch) {
    for (int i = 0; i < warmup; ++i) launch(i);
    checkCudaErrors(cudaStreamSynchronize(stream));
    std::vector<cudaEvent_t> ev(iters + 1);
    for (auto &e : ev) checkCudaErrors(cudaEventCreate(&e));
    checkCudaErrors(cudaEventRecord(ev[0], stream));
    for (int i = 0; i < iters; ++i) {
        launch(warmup + i);
        checkCudaErrors(cudaEventRecord(ev[i + 1], stream));
    }
    checkCudaErrors(cudaStreamSynchronize(stream));
    std::vector<float> ms(iters);
    for (int i = 0; i < iters; ++i) checkCudaErrors(cudaEventElapsedTime(&ms[i], ev[i], ev[i + 1]));
    for (auto &e : ev) cudaEventDestroy(e);
    std::sort(ms.begin(), ms.end());
    return 1e3 * ms[iters / 2];
}

}  // namespace driver
