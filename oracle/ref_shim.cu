// Thin extern "C" launchers around the REFERENCE project's own kernels, compiled unmodified for
// sm_100a from the reference checkout (-I<reference root>; nothing is copied into this tree).
//
// TEST INFRASTRUCTURE ONLY.  The resulting library (oracle/_ref/libko_ref_kernels.so) is used
//   * to pin the CPU oracle's `literal` modes against what the reference really computes, and
//   * as the informational "reference kernel on B200" timing row of the benchmark.
// The product library never loads it.
//
// The reference fixes shapes at compile time (softmax.h:11, layernorm.h:145), so only the
// shapes instantiated below can be launched; the launch geometry is the reference driver's
// (softmax/main.cu:77, layernorm/main.cu:75-76, gemm/main.cu:84,343).
#include <cstdint>
#include <cstdio>
#include <string>

#include <cuda_runtime.h>

// The row-op headers and the GEMM headers declare the same dynamic shared-memory symbol with
// different element types (softmax.h:73 vs simt_gemm.h:226), so this file is compiled twice:
// once with -DKO_REF_PART_ROWOPS and once with -DKO_REF_PART_GEMM.
#if defined(KO_REF_PART_ROWOPS)
#include "nn_operators/softmax/softmax.h"
#include "nn_operators/layernorm/layernorm.h"
#elif defined(KO_REF_PART_GEMM)
#include "nn_operators/gemm/gemm.h"
#else
#error "compile with -DKO_REF_PART_ROWOPS or -DKO_REF_PART_GEMM"
#endif

#if defined(KO_REF_PART_ROWOPS)
namespace {

template <int R, int C>
int launch_softmax(float *in, float *out, cudaStream_t s) {
    using K = SoftMaxWarpImpl<float, 4, R, C>;
    softmax<K><<<40 * 8, 128, K::smem_in_bytes, s>>>(in, out);
    return (int)cudaGetLastError();
}

template <int R, int C, bool AFFINE>
int launch_ln_warp(float *in, float *out, float eps, float *g, float *b, cudaStream_t s) {
    using K = LayerNormWarpImpl<float, 4, R, C, AFFINE>;
    layer_normalization<K><<<40 * 8, 128, K::smem_in_bytes, s>>>(in, out, eps, g, b);
    return (int)cudaGetLastError();
}

template <int R, int C>
int launch_ln_block(float *in, float *out, float eps, cudaStream_t s) {
    using K = LayerNormBlockImpl<float, 4, R, C, false>;
    layer_normalization<K><<<40 * 16, 64, K::smem_in_bytes, s>>>(in, out, eps);
    return (int)cudaGetLastError();
}

}  // namespace

extern "C" {

// returns a cudaError_t value, or -1 when the (rows, cols) pair was not instantiated
int ko_ref_softmax_f32(float *in, float *out, long long rows, int cols, void *stream) {
    cudaStream_t s = (cudaStream_t)stream;
#define KO_CASE(R, C) if (rows == (R) && cols == (C)) return launch_softmax<R, C>(in, out, s);
    KO_CASE(196608, 128)
    KO_CASE(196608, 512)
    KO_CASE(32, 128)
    KO_CASE(1000, 128)
    KO_CASE(16, 512)
#undef KO_CASE
    return -1;
}

// variant: 0 = LayerNormWarpImpl without affine, 1 = LayerNormWarpImpl with gamma/beta,
//          2 = LayerNormBlockImpl (block 64) without affine
int ko_ref_layernorm_f32(float *in, float *out, long long rows, int cols, float eps, float *gamma,
                         float *beta, int variant, void *stream) {
    cudaStream_t s = (cudaStream_t)stream;
#define KO_CASE(R, C)                                                                          \
    if (rows == (R) && cols == (C)) {                                                          \
        if (variant == 0) return launch_ln_warp<R, C, false>(in, out, eps, nullptr, nullptr, s); \
        if (variant == 1) return launch_ln_warp<R, C, true>(in, out, eps, gamma, beta, s);     \
        if (variant == 2) return launch_ln_block<R, C>(in, out, eps, s);                       \
        return -1;                                                                             \
    }
    KO_CASE(16384, 768)
    KO_CASE(8, 768)
    KO_CASE(100, 768)
#undef KO_CASE
    return -1;
}

}  // extern "C"
#endif  // KO_REF_PART_ROWOPS

#if defined(KO_REF_PART_GEMM)
extern "C" {

// The reference SGEMM prefetches one K-tile past the end of A and B on its last iteration
// (simt_gemm.h:287-292), so the caller must own at least 8 floats past A[M*K] and 8*N floats
// past B[K*N]; the capacities (in elements) are checked here and the launch is refused otherwise.
int ko_ref_sgemm_f32(long long M, long long N, long long K, float *A, long long a_capacity,
                     float *B, long long b_capacity, float *C, float *D, void *stream) {
    using Kern = GemmKernelSimt<float, float, float, shape::GemmShape<64, 64, 8>,
                                shape::GemmShape<32, 32, 8>, 4, 4, 4>;
    if (M <= 0 || N <= 0 || K <= 0 || M % 64 || N % 64 || K % 8) return -1;
    if (a_capacity < M * K + 8 || b_capacity < K * N + 8 * N) return -2;
    int grid = (int)((M / 64) * (N / 64));
    gemm<Kern><<<grid, Kern::thread_per_block, Kern::smem_total_size_in_bytes, (cudaStream_t)stream>>>(
        shape::GemmCoord((size_t)M, (size_t)N, (size_t)K), A, B, C, D);
    return (int)cudaGetLastError();
}

}  // extern "C"
#endif  // KO_REF_PART_GEMM
