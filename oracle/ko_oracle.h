/*
 * CPU oracle for the row-softmax / Welford-LayerNorm / SGEMM / mixed-precision GEMM path.
 *
 * TEST INFRASTRUCTURE ONLY.  This library is the checker: the parity tests, the smoke
 * check and the benchmark's CPU-baseline leg load it.  The product library never links,
 * loads or calls it, and there is no CPU fallback behind the CUDA kernels.
 *
 * Every routine is a restatement, in plain C, of arithmetic found in the reference
 * project donglinz/kernel_optimization.  The cited file:line ranges are paths inside
 * that project.  Where the reference's arithmetic is defective (Subtract adds,
 * WelfordMerge divides at every level) a `literal` switch reproduces the defect so that
 * the restatement can be pinned against the reference's own kernels; the default
 * (`literal == 0`) is the mathematically intended operator the product implements.
 *
 * Parity pinning: the reference ships no golden vectors, known-answer tests or fixtures
 * for softmax, LayerNorm or the tensor-core GEMM ("parity unpinned" by its own tests);
 * its only live check is SGEMM against cuBLAS at |err| <= 1e-3
 * (nn_operators/gemm/main.cu:144-176).  The literal modes here are pinned against outputs
 * of the reference kernels themselves, recompiled unmodified for sm_100a and run on a
 * B200 (see oracle/ref_shim.cu and tests/golden/).
 */
#ifndef KO_ORACLE_H
#define KO_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- seeded, counter-based input generator (Philox4x32-10, Salmon et al., SC'11) ---- */
void ko_oracle_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]);
/* element i of tensor `tensor_id` under `seed` depends on (seed, tensor_id, elem_offset + i) only */
void ko_oracle_fill_uniform_f32(float *dst, int64_t n, uint32_t seed, uint32_t tensor_id,
                                int64_t elem_offset, float lo, float hi);
void ko_oracle_fill_normal_f32(float *dst, int64_t n, uint32_t seed, uint32_t tensor_id,
                               int64_t elem_offset, float mean, float stddev);
/* rows are numbered row_offset + r; inside every `block` consecutive rows, col > (row % block) := value */
void ko_oracle_causal_mask_f32(float *dst, int64_t rows, int32_t cols, int64_t row_offset,
                               int32_t block, float value);

/* ---- 16-bit float conversions (round to nearest even) ---- */
uint16_t ko_oracle_f32_to_bf16(float x);
float ko_oracle_bf16_to_f32(uint16_t h);
uint16_t ko_oracle_f32_to_f16(float x);
float ko_oracle_f16_to_f32(uint16_t h);
void ko_oracle_round_f32_to_bf16(const float *src, uint16_t *dst, int64_t n);
void ko_oracle_round_f32_to_f16(const float *src, uint16_t *dst, int64_t n);
void ko_oracle_widen_bf16(const uint16_t *src, float *dst, int64_t n);
void ko_oracle_widen_f16(const uint16_t *src, float *dst, int64_t n);

/* ---- softmax over the last dimension ---- */
/* float64 oracle: exp(x - max) / sum */
void ko_oracle_softmax_f64(const float *in, double *out, int64_t rows, int32_t cols);
/* FP32 port in the warp kernel's operation order (softmax.h:32-58); literal => exp(x + max) */
void ko_oracle_softmax_f32(const float *in, float *out, int64_t rows, int32_t cols,
                           int literal, int threads);

/* ---- LayerNorm forward over the last dimension ---- */
/* float64 oracle; gamma/beta may be NULL; ddof 0 (population) or 1 (sample) */
void ko_oracle_layernorm_f64(const float *in, double *out, int64_t rows, int32_t cols, double eps,
                             const float *gamma, const float *beta, int ddof);
/* FP32 port in the warp kernel's order (layernorm.h:13-23 update, :36-50 merge, :184-198 write).
 * literal => the reference's arithmetic verbatim: merge divides M2 by (n-1) at every level and
 * the normalisation adds the mean (functors.h:164-170); ddof is ignored in that mode. */
void ko_oracle_layernorm_f32(const float *in, float *out, int64_t rows, int32_t cols, float eps,
                             const float *gamma, const float *beta, int ddof, int literal,
                             int threads);

/* (count, mean, M2 = sum of squared deviations) per row, out[rows, 3]: FP32 in the warp kernel's
 * update / merge order without the per-level division (layernorm.h:13-91), and two-pass float64 */
void ko_oracle_welford_stats_f32(const float *in, float *out, int64_t rows, int32_t cols);
void ko_oracle_welford_stats_f64(const float *in, double *out, int64_t rows, int32_t cols);

/* ---- GEMM ---- */
/* D[M,N] = A[M,K] B[K,N] (+ C), all row-major FP32; FP32 fused multiply-add in ascending k
 * (simt_gemm.h:202-222, epilogue :325-373; commented CPU loop gemm/main.cu:162-167) */
void ko_oracle_sgemm_f32(int64_t M, int64_t N, int64_t K, const float *A, const float *B,
                         const float *C, float *D, int threads);
/* same product accumulated in float64 */
void ko_oracle_sgemm_f64(int64_t M, int64_t N, int64_t K, const float *A, const float *B,
                         const float *C, double *D, int threads);
/* 16-bit inputs already widened to FP32 by the caller: A row-major [M,K], B column-major [K,N]
 * (element (k,n) at B[n*K + k]), optional FP32 C, FP32 / float64 accumulate */
void ko_oracle_gemm_tn_f32(int64_t M, int64_t N, int64_t K, const float *A, const float *Bt,
                           const float *C, float *D, int threads);
void ko_oracle_gemm_tn_f64(int64_t M, int64_t N, int64_t K, const float *A, const float *Bt,
                           const float *C, double *D, int threads);

/* ---- error metrics (got is FP32, want is float64) ---- */
double ko_oracle_max_abs_err(const float *got, const double *want, int64_t n);
/* max |got - want| / max(|want|, floor) */
double ko_oracle_max_rel_err(const float *got, const double *want, int64_t n, double floor);
/* ||got - want||_F / ||want||_F */
double ko_oracle_rel_frobenius(const float *got, const double *want, int64_t n);
/* max over rows of |sum(row) - 1| */
double ko_oracle_max_rowsum_err(const float *got, int64_t rows, int32_t cols);

int ko_oracle_max_threads(void);

#ifdef __cplusplus
}
#endif
#endif /* KO_ORACLE_H */
