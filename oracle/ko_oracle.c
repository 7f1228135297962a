/*
 * CPU oracle -- TEST INFRASTRUCTURE ONLY (see ko_oracle.h).  Plain C11 + OpenMP.
 * Build: make -C oracle        (gcc -O2 -fopenmp -ffp-contract=off -shared -fPIC)
 *
 * Citations are file:line inside the reference project donglinz/kernel_optimization.
 */
#include "ko_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define KO_CLONES __attribute__((target_clones("default", "arch=x86-64-v3")))

static int resolve_threads(int threads) {
#ifdef _OPENMP
    return threads > 0 ? threads : omp_get_max_threads();
#else
    (void)threads;
    return 1;
#endif
}

int ko_oracle_max_threads(void) { return resolve_threads(0); }

/* ------------------------------------------------------------------------------------------
 * Philox4x32-10 (J. Salmon, M. Moraes, R. Dror, D. Shaw, "Parallel random numbers: as easy as
 * 1, 2, 3", SC'11).  Published algorithm restated; known-answer vectors are checked in
 * tests/test_oracle_generator.py.
 * ---------------------------------------------------------------------------------------- */
void ko_oracle_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]) {
    uint32_t c0 = ctr[0], c1 = ctr[1], c2 = ctr[2], c3 = ctr[3];
    uint32_t k0 = key[0], k1 = key[1];
    for (int round = 0; round < 10; ++round) {
        uint64_t p0 = (uint64_t)0xD2511F53u * c0;
        uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
        uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
        uint32_t n1 = (uint32_t)p1;
        uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
        uint32_t n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

static inline void philox_block(uint32_t seed, uint32_t tensor_id, uint64_t block, uint32_t out[4]) {
    uint32_t ctr[4] = {(uint32_t)block, (uint32_t)(block >> 32), 0u, 0u};
    uint32_t key[2] = {seed, tensor_id};
    ko_oracle_philox4x32_10(ctr, key, out);
}

/* word -> (0,1): top 24 bits plus half a step, so neither end point is produced */
static inline double unit_open24(uint32_t w) { return ((double)(w >> 8) + 0.5) * (1.0 / 16777216.0); }
/* word -> (0,1) using all 32 bits (for the Box-Muller radius/angle) */
static inline double unit_open32(uint32_t w) { return ((double)w + 0.5) * (1.0 / 4294967296.0); }

void ko_oracle_fill_uniform_f32(float *dst, int64_t n, uint32_t seed, uint32_t tensor_id,
                                int64_t elem_offset, float lo, float hi) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        uint64_t e = (uint64_t)(elem_offset + i);
        uint32_t w[4];
        philox_block(seed, tensor_id, e >> 2, w);
        dst[i] = (float)((double)lo + ((double)hi - (double)lo) * unit_open24(w[e & 3]));
    }
}

void ko_oracle_fill_normal_f32(float *dst, int64_t n, uint32_t seed, uint32_t tensor_id,
                               int64_t elem_offset, float mean, float stddev) {
    /* elements 4b+0,4b+1 come from words (0,1) of block b; 4b+2,4b+3 from words (2,3) */
    const double two_pi = 6.283185307179586476925286766559;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        uint64_t e = (uint64_t)(elem_offset + i);
        uint32_t w[4];
        philox_block(seed, tensor_id, e >> 2, w);
        int pair = (int)((e >> 1) & 1);
        double u1 = unit_open32(w[2 * pair]);
        double u2 = unit_open32(w[2 * pair + 1]);
        double r = sqrt(-2.0 * log(u1));
        double z = (e & 1) ? r * sin(two_pi * u2) : r * cos(two_pi * u2);
        dst[i] = (float)((double)mean + (double)stddev * z);
    }
}

void ko_oracle_causal_mask_f32(float *dst, int64_t rows, int32_t cols, int64_t row_offset,
                               int32_t block, float value) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        int64_t rb = (row_offset + r) % block;
        for (int64_t c = rb + 1; c < cols; ++c) dst[r * (int64_t)cols + c] = value;
    }
}

/* ------------------------------- 16-bit float conversions -------------------------------- */
static inline uint32_t f32_bits(float x) { uint32_t u; memcpy(&u, &x, 4); return u; }
static inline float bits_f32(uint32_t u) { float x; memcpy(&x, &u, 4); return x; }

uint16_t ko_oracle_f32_to_bf16(float x) {
    uint32_t u = f32_bits(x);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* quiet NaN */
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
float ko_oracle_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

uint16_t ko_oracle_f32_to_f16(float x) {
    uint32_t u = f32_bits(x);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);          /* NaN */
    if (a >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);         /* rounds to >= 65520 -> inf */
    if (a < 0x33000001u) return (uint16_t)sign;                      /* <= 2^-25 -> 0 (ties to even) */
    int32_t e = (int32_t)(a >> 23) - 127;
    uint32_t m = (a & 0x7fffffu) | 0x800000u;                        /* 24-bit significand */
    int shift = (e < -14) ? (13 + (-14 - e)) : 13;                   /* bits dropped */
    uint32_t kept = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (kept & 1u))) kept += 1u;
    uint32_t h;
    if (e < -14) h = kept;                                           /* subnormal (may carry to normal) */
    else h = ((uint32_t)(e + 15) << 10) + (kept - 0x400u);           /* carry propagates into exponent */
    return (uint16_t)(sign | h);
}
float ko_oracle_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1fu, m = h & 0x3ffu;
    if (e == 0x1fu) return bits_f32(sign | 0x7f800000u | (m << 13));
    if (e == 0) {
        float v = (float)m * (1.0f / 16777216.0f);                   /* m * 2^-24 */
        return sign ? -v : v;
    }
    return bits_f32(sign | ((e + 112u) << 23) | (m << 13));
}
void ko_oracle_round_f32_to_bf16(const float *src, uint16_t *dst, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) dst[i] = ko_oracle_f32_to_bf16(src[i]);
}
void ko_oracle_round_f32_to_f16(const float *src, uint16_t *dst, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) dst[i] = ko_oracle_f32_to_f16(src[i]);
}
void ko_oracle_widen_bf16(const uint16_t *src, float *dst, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) dst[i] = ko_oracle_bf16_to_f32(src[i]);
}
void ko_oracle_widen_f16(const uint16_t *src, float *dst, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) dst[i] = ko_oracle_f16_to_f32(src[i]);
}

/* ---------------------------------------- softmax ---------------------------------------- */
void ko_oracle_softmax_f64(const float *in, double *out, int64_t rows, int32_t cols) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const float *x = in + r * (int64_t)cols;
        double *y = out + r * (int64_t)cols;
        double mx = -INFINITY, sum = 0.0;
        for (int c = 0; c < cols; ++c) if ((double)x[c] > mx) mx = (double)x[c];
        for (int c = 0; c < cols; ++c) { y[c] = exp((double)x[c] - mx); sum += y[c]; }
        for (int c = 0; c < cols; ++c) y[c] /= sum;
    }
}

/* The warp kernel's data layout (softmax.h:19-32): lane l of a warp owns the vec_len-wide
 * vectors l, l+32, l+64, ... of the row; each of the vec_len slots reduces on its own over
 * those vectors, the slots are folded sequentially (common.h:138-149), and the 32 lane values
 * go through a shfl_down tree 16,8,4,2,1 whose lane-0 result is broadcast (common.h:37-46). */
static float tree32_max(float *v) {
    for (int off = 16; off > 0; off >>= 1)
        for (int i = 0; i < off; ++i) v[i] = v[i] > v[i + off] ? v[i] : v[i + off];
    return v[0];
}
static float tree32_sum(float *v) {
    for (int off = 16; off > 0; off >>= 1)
        for (int i = 0; i < off; ++i) v[i] = v[i] + v[i + off];
    return v[0];
}

void ko_oracle_softmax_f32(const float *in, float *out, int64_t rows, int32_t cols, int literal,
                           int threads) {
    const int vec = (cols % 4 == 0) ? 4 : 1;
    const int nvec = cols / vec;
#pragma omp parallel for schedule(static) num_threads(resolve_threads(threads))
    for (int64_t r = 0; r < rows; ++r) {
        const float *x = in + r * (int64_t)cols;
        float *y = out + r * (int64_t)cols;
        float lane_val[32];
        /* softmax.h:33-42  row maximum */
        for (int l = 0; l < 32; ++l) {
            float slot[4] = {-__FLT_MAX__, -__FLT_MAX__, -__FLT_MAX__, -__FLT_MAX__};
            for (int v = l; v < nvec; v += 32)
                for (int s = 0; s < vec; ++s) {
                    float e = x[v * vec + s];
                    slot[s] = slot[s] > e ? slot[s] : e;
                }
            float m = slot[0];
            for (int s = 1; s < vec; ++s) m = m > slot[s] ? m : slot[s];
            lane_val[l] = m;
        }
        const float row_max = tree32_max(lane_val);
        /* softmax.h:44-52  exp of the shifted logits and their sum */
        for (int l = 0; l < 32; ++l) {
            float slot[4] = {0.f, 0.f, 0.f, 0.f};
            for (int v = l; v < nvec; v += 32)
                for (int s = 0; s < vec; ++s) {
                    float shifted = literal ? x[v * vec + s] + row_max   /* functors.h:164-170 */
                                            : x[v * vec + s] - row_max;
                    float e = expf(shifted);
                    y[v * vec + s] = e;
                    slot[s] += e;
                }
            float t = slot[0];
            for (int s = 1; s < vec; ++s) t += slot[s];
            lane_val[l] = t;
        }
        const float row_sum = tree32_sum(lane_val);
        /* softmax.h:54-57  normalise */
        for (int c = 0; c < cols; ++c) y[c] = y[c] / row_sum;
    }
}

/* --------------------------------------- LayerNorm --------------------------------------- */
void ko_oracle_layernorm_f64(const float *in, double *out, int64_t rows, int32_t cols, double eps,
                             const float *gamma, const float *beta, int ddof) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const float *x = in + r * (int64_t)cols;
        double *y = out + r * (int64_t)cols;
        double mean = 0.0, m2 = 0.0;
        for (int c = 0; c < cols; ++c) mean += (double)x[c];
        mean /= (double)cols;
        for (int c = 0; c < cols; ++c) { double d = (double)x[c] - mean; m2 += d * d; }
        double denom = (double)(cols - ddof);
        double var = denom > 0.0 ? m2 / denom : 0.0;
        double rstd = 1.0 / sqrt(var + eps);
        for (int c = 0; c < cols; ++c) {
            double v = ((double)x[c] - mean) * rstd;
            if (gamma) v *= (double)gamma[c];
            if (beta) v += (double)beta[c];
            y[c] = v;
        }
    }
}

typedef struct { float n, mean, m2; } welford_t;

/* layernorm.h:13-23 */
static inline void welford_update(welford_t *w, float x) {
    w->n += 1.0f;
    float delta = x - w->mean;
    w->mean += delta / w->n;
    float delta2 = x - w->mean;
    w->m2 += delta * delta2;
}

/* layernorm.h:36-50.  literal: the result's m2 is divided by (n_ab - 1) at every call, as the
 * reference does (:48).  Otherwise m2 stays the sum of squared deviations (Chan et al.). */
static inline void welford_merge(welford_t *a, const welford_t *b, int literal) {
    float n_ab = a->n + b->n;
    if (!literal && n_ab == 0.0f) return;
    float delta = b->mean - a->mean;
    float b_over_ab = b->n / n_ab;
    float m2 = a->m2 + b->m2 + delta * delta * a->n * b_over_ab;
    a->mean += delta * b_over_ab;
    a->m2 = literal ? m2 / (n_ab - 1.0f) : m2;
    a->n = n_ab;
}

void ko_oracle_layernorm_f32(const float *in, float *out, int64_t rows, int32_t cols, float eps,
                             const float *gamma, const float *beta, int ddof, int literal,
                             int threads) {
    const int vec = (cols % 4 == 0) ? 4 : 1;
    const int nvec = cols / vec;
#pragma omp parallel for schedule(static) num_threads(resolve_threads(threads))
    for (int64_t r = 0; r < rows; ++r) {
        const float *x = in + r * (int64_t)cols;
        float *y = out + r * (int64_t)cols;
        welford_t lane[32];
        /* layernorm.h:168-179: one Welford stream per vector slot per lane */
        for (int l = 0; l < 32; ++l) {
            welford_t slot[4];
            memset(slot, 0, sizeof slot);
            for (int v = l; v < nvec; v += 32)
                for (int s = 0; s < vec; ++s) welford_update(&slot[s], x[v * vec + s]);
            /* layernorm.h:64-75: fold slots 1..N-1 into slot 0 */
            lane[l] = slot[0];
            for (int s = 1; s < vec; ++s) welford_merge(&lane[l], &slot[s], literal);
        }
        /* layernorm.h:52-62: shfl_down tree; lane 0 holds the row statistics */
        for (int off = 16; off > 0; off >>= 1)
            for (int i = 0; i < off; ++i) welford_merge(&lane[i], &lane[i + off], literal);
        const float mean = lane[0].mean;
        float var;
        if (literal) var = lane[0].m2;                                /* layernorm.h:184 uses m2 as is */
        else {
            float denom = (float)(cols - ddof);
            var = denom > 0.f ? lane[0].m2 / denom : 0.f;
        }
        const float rstd = 1.0f / sqrtf(var + eps);                   /* functors.h:97-103 rsqrtf */
        /* layernorm.h:185-198 */
        for (int c = 0; c < cols; ++c) {
            float centred = literal ? x[c] + mean : x[c] - mean;      /* functors.h:164-170 */
            float v = centred * rstd;
            if (gamma) v = v * gamma[c];
            if (beta) v = v + beta[c];
            y[c] = v;
        }
    }
}

/* Row statistics alone, as (count, mean, M2) with M2 the sum of squared deviations: what the
 * Welford helpers of layernorm.h:13-143 are meant to deliver before the single division.
 * stats_f32: FP32 in the warp kernel's order (per-slot streams :25-34, slot fold :64-75, tree :52-62,
 * merge without the per-level division); stats_f64: two-pass float64. */
void ko_oracle_welford_stats_f32(const float *in, float *out, int64_t rows, int32_t cols) {
    const int vec = (cols % 4 == 0) ? 4 : 1;
    const int nvec = cols / vec;
    for (int64_t r = 0; r < rows; ++r) {
        const float *x = in + r * (int64_t)cols;
        welford_t lane[32];
        for (int l = 0; l < 32; ++l) {
            welford_t slot[4];
            memset(slot, 0, sizeof slot);
            for (int v = l; v < nvec; v += 32)
                for (int s = 0; s < vec; ++s) welford_update(&slot[s], x[v * vec + s]);
            lane[l] = slot[0];
            for (int s = 1; s < vec; ++s) welford_merge(&lane[l], &slot[s], 0);
        }
        for (int off = 16; off > 0; off >>= 1)
            for (int i = 0; i < off; ++i) welford_merge(&lane[i], &lane[i + off], 0);
        out[r * 3 + 0] = lane[0].n;
        out[r * 3 + 1] = lane[0].mean;
        out[r * 3 + 2] = lane[0].m2;
    }
}

void ko_oracle_welford_stats_f64(const float *in, double *out, int64_t rows, int32_t cols) {
    for (int64_t r = 0; r < rows; ++r) {
        const float *x = in + r * (int64_t)cols;
        double sum = 0.0, m2 = 0.0;
        for (int c = 0; c < cols; ++c) sum += (double)x[c];
        const double mean = sum / (double)cols;
        for (int c = 0; c < cols; ++c) m2 += ((double)x[c] - mean) * ((double)x[c] - mean);
        out[r * 3 + 0] = (double)cols;
        out[r * 3 + 1] = mean;
        out[r * 3 + 2] = m2;
    }
}

/* ------------------------------------------ GEMM ----------------------------------------- */
/* Row-major SGEMM; every output accumulates a[i,k]*b[k,j] with one fused multiply-add per k in
 * ascending k, starting from zero (simt_gemm.h:202-222: `accum += a * b` compiles to FFMA),
 * then C is added once at the end (simt_gemm.h:325-354). */
KO_CLONES
static void sgemm_rows_f32(int64_t i0, int64_t i1, int64_t N, int64_t K, const float *A,
                           const float *B, const float *C, float *D) {
    int64_t i = i0;
    for (; i + 4 <= i1; i += 4) {
        float *d0 = D + (i + 0) * N, *d1 = D + (i + 1) * N, *d2 = D + (i + 2) * N, *d3 = D + (i + 3) * N;
        for (int64_t j = 0; j < N; ++j) d0[j] = d1[j] = d2[j] = d3[j] = 0.f;
        for (int64_t k = 0; k < K; ++k) {
            const float a0 = A[(i + 0) * K + k], a1 = A[(i + 1) * K + k];
            const float a2 = A[(i + 2) * K + k], a3 = A[(i + 3) * K + k];
            const float *b = B + k * N;
#pragma omp simd
            for (int64_t j = 0; j < N; ++j) {
                d0[j] = __builtin_fmaf(a0, b[j], d0[j]);
                d1[j] = __builtin_fmaf(a1, b[j], d1[j]);
                d2[j] = __builtin_fmaf(a2, b[j], d2[j]);
                d3[j] = __builtin_fmaf(a3, b[j], d3[j]);
            }
        }
    }
    for (; i < i1; ++i) {
        float *d = D + i * N;
        for (int64_t j = 0; j < N; ++j) d[j] = 0.f;
        for (int64_t k = 0; k < K; ++k) {
            const float a = A[i * K + k];
            const float *b = B + k * N;
#pragma omp simd
            for (int64_t j = 0; j < N; ++j) d[j] = __builtin_fmaf(a, b[j], d[j]);
        }
    }
    if (C)
        for (int64_t r = i0; r < i1; ++r)
            for (int64_t j = 0; j < N; ++j) D[r * N + j] = D[r * N + j] + C[r * N + j];
}

void ko_oracle_sgemm_f32(int64_t M, int64_t N, int64_t K, const float *A, const float *B,
                         const float *C, float *D, int threads) {
    const int64_t chunk = 16;
    const int64_t nchunks = (M + chunk - 1) / chunk;
#pragma omp parallel for schedule(dynamic) num_threads(resolve_threads(threads))
    for (int64_t c = 0; c < nchunks; ++c) {
        int64_t i0 = c * chunk, i1 = i0 + chunk < M ? i0 + chunk : M;
        sgemm_rows_f32(i0, i1, N, K, A, B, C, D);
    }
}

KO_CLONES
static void sgemm_row_f64(int64_t i, int64_t N, int64_t K, const float *A, const float *B,
                          const float *C, double *D) {
    double *d = D + i * N;
    for (int64_t j = 0; j < N; ++j) d[j] = 0.0;
    for (int64_t k = 0; k < K; ++k) {
        const double a = (double)A[i * K + k];
        const float *b = B + k * N;
#pragma omp simd
        for (int64_t j = 0; j < N; ++j) d[j] += a * (double)b[j];
    }
    if (C) for (int64_t j = 0; j < N; ++j) d[j] += (double)C[i * N + j];
}

void ko_oracle_sgemm_f64(int64_t M, int64_t N, int64_t K, const float *A, const float *B,
                         const float *C, double *D, int threads) {
#pragma omp parallel for schedule(dynamic, 8) num_threads(resolve_threads(threads))
    for (int64_t i = 0; i < M; ++i) sgemm_row_f64(i, N, K, A, B, C, D);
}

/* A row-major [M,K], B column-major [K,N] (both K-contiguous): dot products.  The tensor-core
 * path accumulates in FP32 in a hardware-defined order, so the FP32 port keeps 16 partial sums
 * per dot product (vectorisable); the float64 version is the oracle. */
KO_CLONES
static void gemm_tn_row_f32(int64_t m, int64_t N, int64_t K, const float *A, const float *Bt,
                            const float *C, float *D) {
    const float *a = A + m * K;
    for (int64_t n = 0; n < N; ++n) {
        const float *b = Bt + n * K;
        float acc = 0.f;
#pragma omp simd reduction(+ : acc)
        for (int64_t k = 0; k < K; ++k) acc += a[k] * b[k];
        D[m * N + n] = C ? acc + C[m * N + n] : acc;
    }
}
KO_CLONES
static void gemm_tn_row_f64(int64_t m, int64_t N, int64_t K, const float *A, const float *Bt,
                            const float *C, double *D) {
    const float *a = A + m * K;
    for (int64_t n = 0; n < N; ++n) {
        const float *b = Bt + n * K;
        double acc = 0.0;
#pragma omp simd reduction(+ : acc)
        for (int64_t k = 0; k < K; ++k) acc += (double)a[k] * (double)b[k];
        D[m * N + n] = C ? acc + (double)C[m * N + n] : acc;
    }
}
void ko_oracle_gemm_tn_f32(int64_t M, int64_t N, int64_t K, const float *A, const float *Bt,
                           const float *C, float *D, int threads) {
#pragma omp parallel for schedule(dynamic, 4) num_threads(resolve_threads(threads))
    for (int64_t m = 0; m < M; ++m) gemm_tn_row_f32(m, N, K, A, Bt, C, D);
}
void ko_oracle_gemm_tn_f64(int64_t M, int64_t N, int64_t K, const float *A, const float *Bt,
                           const float *C, double *D, int threads) {
#pragma omp parallel for schedule(dynamic, 4) num_threads(resolve_threads(threads))
    for (int64_t m = 0; m < M; ++m) gemm_tn_row_f64(m, N, K, A, Bt, C, D);
}

/* ----------------------------------------- metrics --------------------------------------- */
double ko_oracle_max_abs_err(const float *got, const double *want, int64_t n) {
    double worst = 0.0;
#pragma omp parallel for reduction(max : worst)
    for (int64_t i = 0; i < n; ++i) {
        double e = fabs((double)got[i] - want[i]);
        if (!(e <= worst)) worst = isnan(e) ? INFINITY : e;
    }
    return worst;
}
double ko_oracle_max_rel_err(const float *got, const double *want, int64_t n, double floor_) {
    double worst = 0.0;
#pragma omp parallel for reduction(max : worst)
    for (int64_t i = 0; i < n; ++i) {
        double den = fabs(want[i]) > floor_ ? fabs(want[i]) : floor_;
        double e = fabs((double)got[i] - want[i]) / den;
        if (!(e <= worst)) worst = isnan(e) ? INFINITY : e;
    }
    return worst;
}
double ko_oracle_rel_frobenius(const float *got, const double *want, int64_t n) {
    double num = 0.0, den = 0.0;
#pragma omp parallel for reduction(+ : num, den)
    for (int64_t i = 0; i < n; ++i) {
        double d = (double)got[i] - want[i];
        num += d * d;
        den += want[i] * want[i];
    }
    return den > 0.0 ? sqrt(num / den) : sqrt(num);
}
double ko_oracle_max_rowsum_err(const float *got, int64_t rows, int32_t cols) {
    double worst = 0.0;
#pragma omp parallel for reduction(max : worst)
    for (int64_t r = 0; r < rows; ++r) {
        double s = 0.0;
        for (int c = 0; c < cols; ++c) s += (double)got[r * (int64_t)cols + c];
        double e = fabs(s - 1.0);
        if (!(e <= worst)) worst = isnan(e) ? INFINITY : e;
    }
    return worst;
}
