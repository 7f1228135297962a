// FP32 SGEMM on the FFMA pipe for sm_100a: D[M,N] = A[M,K] * B[K,N] (+ C), all row-major.
//
// Structure (a from-scratch design; the reference's kernel is nn_operators/gemm/simt_gemm.h:46-375):
//   * a thread block owns a BM x BN tile of D and walks K in steps of BK;
//   * the A tile is stored TRANSPOSED in shared memory (As[k][m]) so that both operands are read
//     with conflict-free 128-bit shared loads (the reference keeps A untransposed and issues eight
//     32-bit loads per k, simt_gemm.h:154-170);
//   * shared memory is double buffered and the next global tile is prefetched into registers while
//     the current one is multiplied: one __syncthreads per K step;
//   * every global access is predicated, so any M, N, K is legal (the reference prefetches one tile
//     past the end of A and B, simt_gemm.h:287-292, and needs M, N % 64 == 0, K % 8 == 0);
//   * each output is accumulated with one FFMA per k in ascending k starting from zero, and C is
//     added once at the end -- the same order as the reference (simt_gemm.h:202-222, :325-354),
//     so results agree with it bit for bit.  FFMA only: no TF32, no tensor cores.
//
// A warp's 32 lanes form an LM x LN grid; a lane owns QM x QN quads of 4x4 outputs, quads being
// LM*4 rows / LN*4 columns apart so that neighbouring lanes read neighbouring 16-byte words.
#pragma once

#include "../../common/common.h"
#include "../../common/functors.h"

namespace ko {

template <int BM_, int BN_, int BK_, int WM_, int WN_, int LM_>
struct SgemmConfig {
    static constexpr int BM = BM_, BN = BN_, BK = BK_, WM = WM_, WN = WN_, LM = LM_, LN = 32 / LM_;
    static constexpr int kWarpsM = BM / WM, kWarpsN = BN / WN;
    static constexpr int kThreads = kWarpsM * kWarpsN * 32;
    static constexpr int TM = WM / LM, TN = WN / LN;  // outputs per lane
    static constexpr int QM = TM / 4, QN = TN / 4;    // 4x4 quads per lane
    static constexpr int kPadA = 4, kPadB = 4;
    static constexpr int kStrideA = BM + kPadA, kStrideB = BN + kPadB;
    static constexpr int kStageFloats = BK * kStrideA + BK * kStrideB;
    static constexpr int kSmemBytes = 2 * kStageFloats * (int)sizeof(float);
    static constexpr int kVecA = BM * BK / 4, kVecB = BK * BN / 4;  // float4 per tile
    static constexpr int kLoadsA = (kVecA + kThreads - 1) / kThreads;
    static constexpr int kLoadsB = (kVecB + kThreads - 1) / kThreads;
    static_assert(LM * LN == 32 && TM % 4 == 0 && TN % 4 == 0 && BK % 4 == 0, "bad SGEMM tiling");
    static_assert(BM % WM == 0 && BN % WN == 0 && WM % (LM * 4) == 0 && WN % (LN * 4) == 0, "bad SGEMM tiling");
};

// kAligned: K % 4 == 0, N % 4 == 0 and 16-byte aligned A, B (128-bit global loads);
// otherwise every element is fetched with a predicated 32-bit load.
template <typename Cfg, bool kAligned>
__device__ __forceinline__ void sgemm_tile(int M, int N, int K, const float *__restrict__ A,
                                           const float *__restrict__ B, const float *C, float *D, int tile_m,
                                           int tile_n, float *smem) {
    constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int warp_m = warp / Cfg::kWarpsN, warp_n = warp % Cfg::kWarpsN;
    const int lane_m = lane / Cfg::LN, lane_n = lane % Cfg::LN;
    const int m_base = tile_m * BM, n_base = tile_n * BN;

    auto As = [&](int buf) { return smem + buf * Cfg::kStageFloats; };
    auto Bs = [&](int buf) { return smem + buf * Cfg::kStageFloats + BK * Cfg::kStrideA; };

    float4 stage_a[Cfg::kLoadsA], stage_b[Cfg::kLoadsB];

    auto fetch = [&](int k0) {
#pragma unroll
        for (int s = 0; s < Cfg::kLoadsA; ++s) {
            const int i = tid + s * Cfg::kThreads;
            const int m = i % BM, kq = (i / BM) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i < Cfg::kVecA && m_base + m < M) {
                const float *src = A + (size_t)(m_base + m) * K + (k0 + kq);
                if (kAligned) {
                    if (k0 + kq < K) v = *reinterpret_cast<const float4 *>(src);
                } else {
                    if (k0 + kq + 0 < K) v.x = src[0];
                    if (k0 + kq + 1 < K) v.y = src[1];
                    if (k0 + kq + 2 < K) v.z = src[2];
                    if (k0 + kq + 3 < K) v.w = src[3];
                }
            }
            stage_a[s] = v;
        }
#pragma unroll
        for (int s = 0; s < Cfg::kLoadsB; ++s) {
            const int i = tid + s * Cfg::kThreads;
            const int k = i / (BN / 4), n = (i % (BN / 4)) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i < Cfg::kVecB && k0 + k < K) {
                const float *src = B + (size_t)(k0 + k) * N + (n_base + n);
                if (kAligned) {
                    if (n_base + n < N) v = *reinterpret_cast<const float4 *>(src);
                } else {
                    if (n_base + n + 0 < N) v.x = src[0];
                    if (n_base + n + 1 < N) v.y = src[1];
                    if (n_base + n + 2 < N) v.z = src[2];
                    if (n_base + n + 3 < N) v.w = src[3];
                }
            }
            stage_b[s] = v;
        }
    };
    auto commit = [&](int buf) {
#pragma unroll
        for (int s = 0; s < Cfg::kLoadsA; ++s) {
            const int i = tid + s * Cfg::kThreads;
            if (i < Cfg::kVecA) {
                const int m = i % BM, kq = (i / BM) * 4;
                float *dst = As(buf) + kq * Cfg::kStrideA + m;
                dst[0] = stage_a[s].x;
                dst[Cfg::kStrideA] = stage_a[s].y;
                dst[2 * Cfg::kStrideA] = stage_a[s].z;
                dst[3 * Cfg::kStrideA] = stage_a[s].w;
            }
        }
#pragma unroll
        for (int s = 0; s < Cfg::kLoadsB; ++s) {
            const int i = tid + s * Cfg::kThreads;
            if (i < Cfg::kVecB) {
                const int k = i / (BN / 4), n = (i % (BN / 4)) * 4;
                *reinterpret_cast<float4 *>(Bs(buf) + k * Cfg::kStrideB + n) = stage_b[s];
            }
        }
    };

    float acc[Cfg::QM][Cfg::QN][4][4];
#pragma unroll
    for (int a = 0; a < Cfg::QM; ++a)
#pragma unroll
        for (int b = 0; b < Cfg::QN; ++b)
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[a][b][i][j] = 0.f;

    const int a_off = warp_m * Cfg::WM + lane_m * 4;  // + qm * LM*4
    const int b_off = warp_n * Cfg::WN + lane_n * 4;  // + qn * LN*4

    fetch(0);
    commit(0);
    __syncthreads();

    const int ktiles = (K + BK - 1) / BK;
    for (int kt = 0; kt < ktiles; ++kt) {
        const int cur = kt & 1;
        if (kt + 1 < ktiles) fetch((kt + 1) * BK);

        const float *as = As(cur) + a_off;
        const float *bs = Bs(cur) + b_off;
        float4 fa[2][Cfg::QM], fb[2][Cfg::QN];
#pragma unroll
        for (int q = 0; q < Cfg::QM; ++q) fa[0][q] = *reinterpret_cast<const float4 *>(as + q * Cfg::LM * 4);
#pragma unroll
        for (int q = 0; q < Cfg::QN; ++q) fb[0][q] = *reinterpret_cast<const float4 *>(bs + q * Cfg::LN * 4);
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            const int now = kk & 1, nxt = now ^ 1;
            if (kk + 1 < BK) {
#pragma unroll
                for (int q = 0; q < Cfg::QM; ++q)
                    fa[nxt][q] = *reinterpret_cast<const float4 *>(as + (kk + 1) * Cfg::kStrideA + q * Cfg::LM * 4);
#pragma unroll
                for (int q = 0; q < Cfg::QN; ++q)
                    fb[nxt][q] = *reinterpret_cast<const float4 *>(bs + (kk + 1) * Cfg::kStrideB + q * Cfg::LN * 4);
            }
#pragma unroll
            for (int a = 0; a < Cfg::QM; ++a) {
                const float av[4] = {fa[now][a].x, fa[now][a].y, fa[now][a].z, fa[now][a].w};
#pragma unroll
                for (int b = 0; b < Cfg::QN; ++b) {
                    const float bv[4] = {fb[now][b].x, fb[now][b].y, fb[now][b].z, fb[now][b].w};
#pragma unroll
                    for (int i = 0; i < 4; ++i)
#pragma unroll
                        for (int j = 0; j < 4; ++j) acc[a][b][i][j] = fmaf(av[i], bv[j], acc[a][b][i][j]);
                }
            }
        }
        if (kt + 1 < ktiles) {
            commit(cur ^ 1);
            __syncthreads();
        }
    }

    // epilogue: D = acc (+ C), 128-bit stores where the row pitch allows
    const bool vec_out = (N % 4 == 0) && ((reinterpret_cast<uintptr_t>(D) & 15u) == 0) &&
                         (C == nullptr || (reinterpret_cast<uintptr_t>(C) & 15u) == 0);
#pragma unroll
    for (int a = 0; a < Cfg::QM; ++a) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int m = m_base + a_off + a * Cfg::LM * 4 + i;
            if (m >= M) continue;
#pragma unroll
            for (int b = 0; b < Cfg::QN; ++b) {
                const int n = n_base + b_off + b * Cfg::LN * 4;
                if (n >= N) continue;
                float4 v = make_float4(acc[a][b][i][0], acc[a][b][i][1], acc[a][b][i][2], acc[a][b][i][3]);
                const size_t off = (size_t)m * N + n;
                if (vec_out) {
                    if (C) {
                        const float4 c = *reinterpret_cast<const float4 *>(C + off);
                        v.x += c.x; v.y += c.y; v.z += c.z; v.w += c.w;
                    }
                    *reinterpret_cast<float4 *>(D + off) = v;
                } else {
                    const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (n + j < N) D[off + j] = C ? vv[j] + C[off + j] : vv[j];
                }
            }
        }
    }
}

// runtime-shape kernel used by the C ABI: one tile per block, 1-D grid, tiles ordered so that
// blocks running together share A rows / B columns in L2
template <typename Cfg, bool kAligned>
__global__ void __launch_bounds__(Cfg::kThreads) sgemm_kernel(int M, int N, int K, const float *A, const float *B,
                                                              const float *C, float *D) {
    extern __shared__ __align__(16) float ko_sgemm_smem[];
    const int tiles_n = (N + Cfg::BN - 1) / Cfg::BN;
    sgemm_tile<Cfg, kAligned>(M, N, K, A, B, C, D, blockIdx.x / tiles_n, blockIdx.x % tiles_n, ko_sgemm_smem);
}

}  // namespace ko

// ---------------------------------------------------------------------------------------------
// source-level drop-in for the reference's GemmKernelSimt (same template parameters and static
// members; ThreadBlockShape / WarpShape choose the tiling, lanes form a 4 x 8 grid as in the
// reference's WarpThreadMap, simt_gemm.h:21-27)
// ---------------------------------------------------------------------------------------------
namespace thread_mapping {
template <typename ThreadBlockShape, typename WarpShape>
struct ThreadBlockThreadMap {
    static constexpr int warp_count_m = ThreadBlockShape::kM / WarpShape::kM;
    static constexpr int warp_count_n = ThreadBlockShape::kN / WarpShape::kN;
};
}  // namespace thread_mapping

template <typename ElementA_, typename ElementB_, typename ElementC_, typename ThreadBlockShape_, typename WarpShape_,
          int AlignmentA, int AlignmentB, int AlignmentC>
struct GemmKernelSimt {
    using ElementA = ElementA_;
    using ElementB = ElementB_;
    using ElementC = ElementC_;
    using ThreadBlockShape = ThreadBlockShape_;
    using WarpShape = WarpShape_;
    // shared-memory K step: at least 8 and a multiple of 4, whatever ThreadBlockShape::kK says
    static constexpr int kStepK = ThreadBlockShape::kK >= 8 ? (ThreadBlockShape::kK / 4) * 4 : 8;
    using Cfg = ko::SgemmConfig<ThreadBlockShape::kM, ThreadBlockShape::kN, kStepK, WarpShape::kM, WarpShape::kN, 4>;

    static constexpr int smem_A_total_size_in_bytes = 2 * Cfg::BK * Cfg::kStrideA * (int)sizeof(float);
    static constexpr int smem_B_total_size_in_bytes = 2 * Cfg::BK * Cfg::kStrideB * (int)sizeof(float);
    static constexpr int smem_total_size_in_bytes = Cfg::kSmemBytes;
    static constexpr int warp_count_m = Cfg::kWarpsM, warp_count_n = Cfg::kWarpsN;
    static constexpr int warp_count = warp_count_m * warp_count_n;
    static constexpr int thread_per_block = Cfg::kThreads;

    __device__ __forceinline__ void operator()(const shape::GemmCoord &problem_size, ElementA *ptr_A, ElementB *ptr_B,
                                               ElementC *ptr_C, ElementC *ptr_D) const {
        static_assert(sizeof(ElementA) == 4 && sizeof(ElementB) == 4 && sizeof(ElementC) == 4, "FP32 only");
        extern __shared__ __align__(16) float ko_sgemm_smem[];
        const int M = (int)problem_size.m(), N = (int)problem_size.n(), K = (int)problem_size.k();
        const int tiles_n = (N + Cfg::BN - 1) / Cfg::BN, tiles_m = (M + Cfg::BM - 1) / Cfg::BM;
        const bool aligned = K % 4 == 0 && N % 4 == 0 && ((reinterpret_cast<uintptr_t>(ptr_A) & 15u) == 0) &&
                             ((reinterpret_cast<uintptr_t>(ptr_B) & 15u) == 0);
        for (int tile = blockIdx.x; tile < tiles_m * tiles_n; tile += gridDim.x) {
            if (aligned)
                ko::sgemm_tile<Cfg, true>(M, N, K, ptr_A, ptr_B, ptr_C, ptr_D, tile / tiles_n, tile % tiles_n, ko_sgemm_smem);
            else
                ko::sgemm_tile<Cfg, false>(M, N, K, ptr_A, ptr_B, ptr_C, ptr_D, tile / tiles_n, tile % tiles_n, ko_sgemm_smem);
            __syncthreads();
        }
    }
};
