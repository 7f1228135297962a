// C-ABI launcher of the row softmax: picks the tier and the launch geometry from the runtime shape.
#include "ko_internal.h"
#include "ko_tuning.h"

#include "../nn_operators/softmax/softmax.h"

namespace {

using ko::DeviceInfo;

template <int kVecs, int kRows>
int launch_warp(const float *in, float *out, long long rows, int cols, int block, long long grid_cap,
                cudaStream_t s) {
    const int warps_per_block = block / 32;
    const long long groups = (rows + kRows - 1) / kRows;
    long long grid = (groups + warps_per_block - 1) / warps_per_block;
    if (grid_cap > 0 && grid > grid_cap) grid = grid_cap;
    if (grid > 0x7fffffffLL) grid = 0x7fffffffLL;
    ko::softmax_warp_kernel<kVecs, kRows><<<(unsigned)grid, block, 0, s>>>(in, out, rows, cols);
    KO_CHECK_LAUNCH("softmax_warp_kernel");
    return KO_OK;
}

template <int kVecs, int kThreads>
int launch_block(const float *in, float *out, long long rows, int cols, long long grid_cap, cudaStream_t s) {
    long long grid = rows;
    if (grid_cap > 0 && grid > grid_cap) grid = grid_cap;
    if (grid > 0x7fffffffLL) grid = 0x7fffffffLL;
    ko::softmax_block_kernel<kVecs, kThreads><<<(unsigned)grid, kThreads, 0, s>>>(in, out, rows, cols);
    KO_CHECK_LAUNCH("softmax_block_kernel");
    return KO_OK;
}

int validate(const float *in, float *out, long long rows, int cols) {
    KO_REQUIRE(rows >= 0 && cols >= 0, KO_ERR_INVALID_ARG, "softmax: negative shape [%lld, %d]", rows, cols);
    if (rows == 0 || cols == 0) return KO_OK;
    KO_REQUIRE(in != nullptr && out != nullptr, KO_ERR_INVALID_ARG, "softmax: NULL pointer");
    return KO_OK;
}

}  // namespace

extern "C" {

int ko_softmax_f32_tuned(const float *in, float *out, int64_t rows, int32_t cols, int rows_per_warp, int block,
                         int64_t grid_cap, void *stream) {
    if (int st = validate(in, out, rows, cols)) return st;
    if (rows == 0 || cols == 0) return KO_OK;
    DeviceInfo info;
    if (int st = ko::current_device_info(&info)) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool vec_ok = (cols % 4 == 0) && ko::aligned16(in) && ko::aligned16(out);
    const int nvec = cols / 4;
    if (block <= 0) block = 256;
    KO_REQUIRE(block % 32 == 0 && block <= 256, KO_ERR_INVALID_ARG, "softmax: block %d must be a multiple of 32, <= 256", block);

    if (vec_ok && nvec <= 32 * 16) {
        const int vecs = (nvec + 31) / 32;
#define KO_WARP(V, R) return launch_warp<V, R>(in, out, rows, cols, block, grid_cap, s)
        if (vecs == 1) {
            switch (rows_per_warp) { case 1: KO_WARP(1, 1); case 2: KO_WARP(1, 2); case 8: KO_WARP(1, 8); default: KO_WARP(1, 4); }
        } else if (vecs == 2) {
            switch (rows_per_warp) { case 1: KO_WARP(2, 1); case 4: KO_WARP(2, 4); default: KO_WARP(2, 2); }
        } else if (vecs <= 4) {
            switch (rows_per_warp) { case 1: KO_WARP(4, 1); case 4: KO_WARP(4, 4); default: KO_WARP(4, 2); }
        } else if (vecs <= 6) {
            switch (rows_per_warp) { case 2: KO_WARP(6, 2); default: KO_WARP(6, 1); }
        } else if (vecs <= 8) {
            switch (rows_per_warp) { case 2: KO_WARP(8, 2); default: KO_WARP(8, 1); }
        } else if (vecs <= 12) {
            KO_WARP(12, 1);
        } else {
            KO_WARP(16, 1);
        }
#undef KO_WARP
    }
    if (vec_ok && nvec <= 1024 * 8) {
        // one row per block, <= 8 vectors per thread
        if (nvec <= 256 * 4) return launch_block<4, 256>(in, out, rows, cols, grid_cap, s);
        if (nvec <= 512 * 4) return launch_block<4, 512>(in, out, rows, cols, grid_cap, s);
        if (nvec <= 1024 * 4) return launch_block<4, 1024>(in, out, rows, cols, grid_cap, s);
        return launch_block<8, 1024>(in, out, rows, cols, grid_cap, s);
    }
    long long grid = rows;
    const long long cap = grid_cap > 0 ? grid_cap : (long long)info.sm_count * 8;
    if (grid > cap) grid = cap;
    ko::softmax_stream_kernel<<<(unsigned)grid, 256, 0, s>>>(in, out, rows, cols);
    KO_CHECK_LAUNCH("softmax_stream_kernel");
    return KO_OK;
}

int ko_softmax_f32(const float *in, float *out, int64_t rows, int32_t cols, void *stream) {
    return ko_softmax_f32_tuned(in, out, rows, cols, /*rows_per_warp=*/0, /*block=*/0, /*grid_cap=*/0, stream);
}

}  // extern "C"
