// C-ABI launcher of the FFMA SGEMM: picks the tile configuration from the problem shape.
#include "ko_internal.h"
#include "ko_tuning.h"

#include "../nn_operators/gemm/simt_gemm.h"

namespace {

//                              BM   BN  BK  WM  WN LM
using CfgBig = ko::SgemmConfig<128, 128, 16, 32, 64, 4>;   // 256 threads, 8x8 per lane
using CfgWide = ko::SgemmConfig<128, 64, 16, 32, 32, 4>;   // 256 threads, 8x4 per lane
using CfgSmall = ko::SgemmConfig<64, 64, 16, 32, 32, 4>;   // 128 threads, 8x4 per lane

template <typename Cfg>
int launch(int M, int N, int K, const float *A, const float *B, const float *C, float *D, bool aligned,
           cudaStream_t s) {
    const long long tiles = (long long)((M + Cfg::BM - 1) / Cfg::BM) * ((N + Cfg::BN - 1) / Cfg::BN);
    KO_REQUIRE(tiles <= 0x7fffffffLL, KO_ERR_SHAPE, "sgemm: %lld tiles exceed the grid limit", tiles);
    if (aligned)
        ko::sgemm_kernel<Cfg, true><<<(unsigned)tiles, Cfg::kThreads, Cfg::kSmemBytes, s>>>(M, N, K, A, B, C, D);
    else
        ko::sgemm_kernel<Cfg, false><<<(unsigned)tiles, Cfg::kThreads, Cfg::kSmemBytes, s>>>(M, N, K, A, B, C, D);
    KO_CHECK_LAUNCH("sgemm_kernel");
    return KO_OK;
}

template <typename Cfg>
double wave_efficiency(long long M, long long N, int sm_count, int blocks_per_sm) {
    const long long tiles = ((M + Cfg::BM - 1) / Cfg::BM) * ((N + Cfg::BN - 1) / Cfg::BN);
    const long long slots = (long long)sm_count * blocks_per_sm;
    const long long waves = (tiles + slots - 1) / slots;
    const double fill = (double)tiles / (double)(waves * slots);
    const double useful = (double)(M * N) / (double)(tiles * Cfg::BM * Cfg::BN);
    return fill * useful;
}

}  // namespace

extern "C" {

// variant: 0 = choose, 1 = 128x128 tiles, 2 = 128x64, 3 = 64x64
int ko_sgemm_f32_tuned(int64_t M, int64_t N, int64_t K, const float *A, const float *B, const float *C, float *D,
                       int variant, void *stream) {
    KO_REQUIRE(M >= 0 && N >= 0 && K >= 0, KO_ERR_INVALID_ARG, "sgemm: negative shape {%lld,%lld,%lld}",
               (long long)M, (long long)N, (long long)K);
    if (M == 0 || N == 0) return KO_OK;
    KO_REQUIRE(M <= 0x7fffffff && N <= 0x7fffffff && K <= 0x7fffffff, KO_ERR_SHAPE, "sgemm: dimension exceeds 2^31-1");
    KO_REQUIRE(D != nullptr && (K == 0 || (A != nullptr && B != nullptr)), KO_ERR_INVALID_ARG, "sgemm: NULL pointer");
    KO_REQUIRE(D != A && D != B, KO_ERR_INVALID_ARG, "sgemm: D must not alias A or B");
    ko::DeviceInfo info;
    if (int st = ko::current_device_info(&info)) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool aligned = K % 4 == 0 && N % 4 == 0 && ko::aligned16(A) && ko::aligned16(B);

    if (variant == 0) {
        // weigh wave quantisation against the better FFMA:LDS ratio of the larger tiles
        const double big = 1.00 * wave_efficiency<CfgBig>(M, N, info.sm_count, 1);
        const double wide = 0.92 * wave_efficiency<CfgWide>(M, N, info.sm_count, 2);
        const double small = 0.85 * wave_efficiency<CfgSmall>(M, N, info.sm_count, 4);
        variant = (big >= wide && big >= small) ? 1 : (wide >= small ? 2 : 3);
    }
    const int m = (int)M, n = (int)N, k = (int)K;
    switch (variant) {
        case 1: return launch<CfgBig>(m, n, k, A, B, C, D, aligned, s);
        case 2: return launch<CfgWide>(m, n, k, A, B, C, D, aligned, s);
        case 3: return launch<CfgSmall>(m, n, k, A, B, C, D, aligned, s);
        default: return ko::fail(KO_ERR_INVALID_ARG, "sgemm: unknown variant %d", variant);
    }
}

int ko_sgemm_f32(int64_t M, int64_t N, int64_t K, const float *A, const float *B, const float *C, float *D,
                 void *stream) {
    return ko_sgemm_f32_tuned(M, N, K, A, B, C, D, 0, stream);
}

}  // extern "C"
