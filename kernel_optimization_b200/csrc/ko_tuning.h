// Launch-geometry overrides of the operator entry points (same semantics as the public calls;
// 0 selects the library's default for that knob).  Used by the sweep tooling and the tests that
// pin every instantiated variant; applications call the plain entry points of ko_b200.h.
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

int ko_softmax_f32_tuned(const float *in, float *out, int64_t rows, int32_t cols, int rows_per_warp, int block,
                         int64_t grid_cap, void *stream);
/* block: warp tier -> threads per block (<= 256); block tier -> threads per row (128..1024) */
int ko_layernorm_f32_tuned(const float *in, float *out, int64_t rows, int32_t cols, float eps, const float *gamma,
                           const float *beta, int ddof, int rows_per_warp, int block, int64_t grid_cap, void *stream);
int ko_layernorm_bf16_tuned(const uint16_t *in, uint16_t *out, int64_t rows, int32_t cols, float eps,
                            const uint16_t *gamma, const uint16_t *beta, int ddof, int rows_per_warp, int block,
                            int64_t grid_cap, void *stream);
/* variant: 0 = choose, 1 = 128x128 tiles, 2 = 128x64, 3 = 64x64 */
int ko_sgemm_f32_tuned(int64_t M, int64_t N, int64_t K, const float *A, const float *B, const float *C, float *D,
                       int variant, void *stream);
/* fmt: 0 = F16, 1 = BF16; bn: 0 = choose, else 64 / 128 / 256 columns of D per tile */
int ko_gemm_tc_tuned(int fmt, int64_t M, int64_t N, int64_t K, const uint16_t *A, const uint16_t *B, const float *C,
                     float *D, int bn, void *stream);

#ifdef __cplusplus
}
#endif
