// C-ABI launchers of the LayerNorm forward: tier and launch geometry from the runtime shape.
#include "ko_internal.h"
#include "ko_tuning.h"

#include "../nn_operators/layernorm/layernorm.h"

namespace {

template <typename T, int kVecs, int kRows>
int launch_warp(const T *in, T *out, long long rows, int cols, float eps, const T *g, const T *b, int ddof,
                int block, long long grid_cap, cudaStream_t s) {
    const int warps_per_block = block / 32;
    const long long groups = (rows + kRows - 1) / kRows;
    long long grid = (groups + warps_per_block - 1) / warps_per_block;
    if (grid_cap > 0 && grid > grid_cap) grid = grid_cap;
    if (grid > 0x7fffffffLL) grid = 0x7fffffffLL;
    ko::layernorm_warp_kernel<T, kVecs, kRows><<<(unsigned)grid, block, 0, s>>>(in, out, rows, cols, eps, g, b, ddof);
    KO_CHECK_LAUNCH("layernorm_warp_kernel");
    return KO_OK;
}

template <typename T, int kVecs, int kThreads>
int launch_block(const T *in, T *out, long long rows, int cols, float eps, const T *g, const T *b, int ddof,
                 long long grid_cap, cudaStream_t s) {
    long long grid = rows;
    if (grid_cap > 0 && grid > grid_cap) grid = grid_cap;
    if (grid > 0x7fffffffLL) grid = 0x7fffffffLL;
    ko::layernorm_block_kernel<T, kVecs, kThreads><<<(unsigned)grid, kThreads, 0, s>>>(in, out, rows, cols, eps, g, b, ddof);
    KO_CHECK_LAUNCH("layernorm_block_kernel");
    return KO_OK;
}

template <typename T, int kThreads>
int launch_block_vecs(int vecs, const T *in, T *out, long long rows, int cols, float eps, const T *g, const T *b,
                      int ddof, long long grid_cap, cudaStream_t s) {
    if (vecs <= 1) return launch_block<T, 1, kThreads>(in, out, rows, cols, eps, g, b, ddof, grid_cap, s);
    if (vecs <= 2) return launch_block<T, 2, kThreads>(in, out, rows, cols, eps, g, b, ddof, grid_cap, s);
    if (vecs <= 4) return launch_block<T, 4, kThreads>(in, out, rows, cols, eps, g, b, ddof, grid_cap, s);
    return launch_block<T, 8, kThreads>(in, out, rows, cols, eps, g, b, ddof, grid_cap, s);
}

template <typename T>
int layernorm_dispatch(const T *in, T *out, long long rows, int cols, float eps, const T *gamma, const T *beta,
                       int ddof, int rows_per_warp, int block, long long grid_cap, cudaStream_t s) {
    KO_REQUIRE(rows >= 0 && cols >= 0, KO_ERR_INVALID_ARG, "layernorm: negative shape [%lld, %d]", rows, cols);
    KO_REQUIRE(ddof == 0 || ddof == 1, KO_ERR_INVALID_ARG, "layernorm: ddof must be 0 or 1, got %d", ddof);
    if (rows == 0 || cols == 0) return KO_OK;
    KO_REQUIRE(in != nullptr && out != nullptr, KO_ERR_INVALID_ARG, "layernorm: NULL pointer");
    ko::DeviceInfo info;
    if (int st = ko::current_device_info(&info)) return st;

    constexpr int kPer = ko::RowIo<T>::kPerVec;
    constexpr int kMaxVecsPerThread = 32 / kPer;  // 32 FP32 values per thread
    const bool vec_ok = cols % kPer == 0 && ko::aligned16(in) && ko::aligned16(out) && ko::aligned16(gamma) &&
                        ko::aligned16(beta);
    const int nvec = cols / kPer;
    KO_REQUIRE(block >= 0 && block % 32 == 0 && block <= 1024, KO_ERR_INVALID_ARG,
               "layernorm: block %d must be a multiple of 32, <= 1024", block);

    if (vec_ok && nvec <= 32 * kMaxVecsPerThread) {
        const int vecs = (nvec + 31) / 32;
        const int wb = (block > 0 && block <= 256) ? block : 256;
#define KO_WARP(V, R) return launch_warp<T, V, R>(in, out, rows, cols, eps, gamma, beta, ddof, wb, grid_cap, s)
        if (vecs == 1) { if (rows_per_warp == 1) KO_WARP(1, 1); if (rows_per_warp == 2) KO_WARP(1, 2); KO_WARP(1, 4); }
        if (vecs == 2) { if (rows_per_warp == 1) KO_WARP(2, 1); if (rows_per_warp == 4) KO_WARP(2, 4); KO_WARP(2, 2); }
        if (vecs <= 4) { if (rows_per_warp == 1) KO_WARP(4, 1); KO_WARP(4, 2); }
        if constexpr (kMaxVecsPerThread >= 8) {
            if (vecs <= 6) { if (rows_per_warp == 1) KO_WARP(6, 1); KO_WARP(6, 2); }
            if (rows_per_warp == 2) KO_WARP(8, 2);
            KO_WARP(8, 1);
        }
#undef KO_WARP
    }
    if (vec_ok && nvec <= 1024 * kMaxVecsPerThread) {
        // threads per row: aim at 2 vectors per thread unless the caller picks the block size
        int threads = block;
        if (threads == 0) {
            threads = 128;
            while (threads < 1024 && nvec > threads * 2) threads *= 2;
        }
        while (threads < 1024 && nvec > threads * kMaxVecsPerThread) threads *= 2;
        const int vecs = (nvec + threads - 1) / threads;
        switch (threads) {
            case 128: return launch_block_vecs<T, 128>(vecs, in, out, rows, cols, eps, gamma, beta, ddof, grid_cap, s);
            case 256: return launch_block_vecs<T, 256>(vecs, in, out, rows, cols, eps, gamma, beta, ddof, grid_cap, s);
            case 512: return launch_block_vecs<T, 512>(vecs, in, out, rows, cols, eps, gamma, beta, ddof, grid_cap, s);
            case 1024: return launch_block_vecs<T, 1024>(vecs, in, out, rows, cols, eps, gamma, beta, ddof, grid_cap, s);
            default: return ko::fail(KO_ERR_INVALID_ARG, "layernorm: block tier needs 128/256/512/1024 threads, got %d", threads);
        }
    }
    long long grid = rows;
    const long long cap = grid_cap > 0 ? grid_cap : (long long)info.sm_count * 8;
    if (grid > cap) grid = cap;
    ko::layernorm_stream_kernel<T><<<(unsigned)grid, 256, 0, s>>>(in, out, rows, cols, eps, gamma, beta, ddof);
    KO_CHECK_LAUNCH("layernorm_stream_kernel");
    return KO_OK;
}

}  // namespace

extern "C" {

int ko_layernorm_f32_tuned(const float *in, float *out, int64_t rows, int32_t cols, float eps, const float *gamma,
                           const float *beta, int ddof, int rows_per_warp, int block, int64_t grid_cap, void *stream) {
    return layernorm_dispatch<float>(in, out, rows, cols, eps, gamma, beta, ddof, rows_per_warp, block, grid_cap,
                                     static_cast<cudaStream_t>(stream));
}

int ko_layernorm_bf16_tuned(const uint16_t *in, uint16_t *out, int64_t rows, int32_t cols, float eps,
                            const uint16_t *gamma, const uint16_t *beta, int ddof, int rows_per_warp, int block,
                            int64_t grid_cap, void *stream) {
    using B = __nv_bfloat16;
    return layernorm_dispatch<B>(reinterpret_cast<const B *>(in), reinterpret_cast<B *>(out), rows, cols, eps,
                                 reinterpret_cast<const B *>(gamma), reinterpret_cast<const B *>(beta), ddof,
                                 rows_per_warp, block, grid_cap, static_cast<cudaStream_t>(stream));
}

int ko_layernorm_f32(const float *in, float *out, int64_t rows, int32_t cols, float eps, const float *gamma,
                     const float *beta, int ddof, void *stream) {
    return ko_layernorm_f32_tuned(in, out, rows, cols, eps, gamma, beta, ddof, 0, 0, 0, stream);
}

int ko_layernorm_bf16(const uint16_t *in, uint16_t *out, int64_t rows, int32_t cols, float eps, const uint16_t *gamma,
                      const uint16_t *beta, int ddof, void *stream) {
    return ko_layernorm_bf16_tuned(in, out, rows, cols, eps, gamma, beta, ddof, 0, 0, 0, stream);
}

}  // extern "C"
