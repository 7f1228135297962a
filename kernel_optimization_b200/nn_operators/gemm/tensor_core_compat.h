// Source-level stand-in for the reference's GemmKernelTensorCore template
// (nn_operators/gemm/tensor_core_gemm.h:101-399): same template parameters, static members and call
// operator, so `gemm<GemmKernelTensorCore<half, half, half, GemmShape<128,128,32>, GemmShape<64,64,32>,
// GemmShape<16,8,8>, 8, 8, 8>><<<grid, K::thread_per_block, K::smem_total_size_in_bytes>>>(...)` compiles
// and produces D = A * B (+ C) for row-major A [M,K], B [K,N], C/D [M,N] as the reference intends.
//
// The reference's kernel is an unfinished Turing mma.sync design (FP16 accumulate, wrong epilogue,
// call disabled at nn_operators/gemm/main.cu:344).  The Blackwell tensor-core path of this library
// (tcgen05 + TMEM + TMA, tensor_core_gemm.h) needs host-built TMA descriptors and therefore lives
// behind the C ABI (ko_gemm_f16_f32 / ko_gemm_bf16_f32).  This template exists for source
// compatibility only: it multiplies on the FP32 pipe with FP32 accumulation (more accurate than the
// reference's FP16 accumulation) through a shared-memory tile, for any M, N, K and any grid.
#pragma once

#include "../../common/common.h"

template <typename ElementA_, typename ElementB_, typename ElementC_, typename ThreadBlockShape_, typename WarpShape_,
          typename InstructionShape_, int AlignmentA, int AlignmentB, int AlignmentC>
struct GemmKernelTensorCore {
    using ElementA = ElementA_;
    using ElementB = ElementB_;
    using ElementC = ElementC_;
    using ThreadBlockShape = ThreadBlockShape_;
    using WarpShape = WarpShape_;
    using InstructionShape = InstructionShape_;

    static constexpr int kTileK = 16;
    static constexpr int smem_A_total_size_in_bytes = ThreadBlockShape::kM * kTileK * (int)sizeof(float);
    static constexpr int smem_B_total_size_in_bytes = kTileK * ThreadBlockShape::kN * (int)sizeof(float);
    static constexpr int smem_total_size_in_bytes = smem_A_total_size_in_bytes + smem_B_total_size_in_bytes;
    static constexpr int warp_count_m = ThreadBlockShape::kM / WarpShape::kM;
    static constexpr int warp_count_n = ThreadBlockShape::kN / WarpShape::kN;
    static constexpr int warp_count = warp_count_m * warp_count_n;
    static constexpr int thread_per_block = warp_count * 32;

    __device__ static float widen(const float &v) { return v; }
    __device__ static float widen(const half &v) { return __half2float(v); }
    __device__ static float widen(const __nv_bfloat16 &v) { return __bfloat162float(v); }
    template <typename T>
    __device__ static T narrow(float v) {
        if constexpr (sizeof(T) == 4) return v;
        else if constexpr (std::is_same<T, half>::value) return __float2half_rn(v);
        else return __float2bfloat16_rn(v);
    }

    __device__ __forceinline__ void operator()(const shape::GemmCoord &problem_size, ElementA *ptr_A, ElementB *ptr_B,
                                               ElementC *ptr_C, ElementC *ptr_D) const {
        constexpr int BM = ThreadBlockShape::kM, BN = ThreadBlockShape::kN;
        extern __shared__ __align__(16) float ko_tc_compat_smem[];
        float *As = ko_tc_compat_smem;           // [BM][kTileK]
        float *Bs = ko_tc_compat_smem + BM * kTileK;  // [kTileK][BN]
        const int M = (int)problem_size.m(), N = (int)problem_size.n(), K = (int)problem_size.k();
        const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
        constexpr int kOutputs = BM * BN;
        constexpr int kPerThread = (kOutputs + thread_per_block - 1) / thread_per_block;
        for (int tile = blockIdx.x; tile < tiles_m * tiles_n; tile += gridDim.x) {
            const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
            float acc[kPerThread];
#pragma unroll
            for (int i = 0; i < kPerThread; ++i) acc[i] = 0.f;
            for (int k0 = 0; k0 < K; k0 += kTileK) {
                __syncthreads();
                for (int e = threadIdx.x; e < BM * kTileK; e += blockDim.x) {
                    const int m = e / kTileK, k = e % kTileK;
                    As[e] = (m0 + m < M && k0 + k < K) ? widen(ptr_A[(size_t)(m0 + m) * K + k0 + k]) : 0.f;
                }
                for (int e = threadIdx.x; e < kTileK * BN; e += blockDim.x) {
                    const int k = e / BN, n = e % BN;
                    Bs[e] = (k0 + k < K && n0 + n < N) ? widen(ptr_B[(size_t)(k0 + k) * N + n0 + n]) : 0.f;
                }
                __syncthreads();
#pragma unroll
                for (int i = 0; i < kPerThread; ++i) {
                    const int o = threadIdx.x + i * blockDim.x;
                    if (o < kOutputs) {
                        const int m = o / BN, n = o % BN;
#pragma unroll
                        for (int k = 0; k < kTileK; ++k) acc[i] = fmaf(As[m * kTileK + k], Bs[k * BN + n], acc[i]);
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < kPerThread; ++i) {
                const int o = threadIdx.x + i * blockDim.x;
                const int m = m0 + o / BN, n = n0 + o % BN;
                if (o < kOutputs && m < M && n < N) {
                    float v = acc[i];
                    if (ptr_C) v += widen(ptr_C[(size_t)m * N + n]);
                    ptr_D[(size_t)m * N + n] = narrow<ElementC>(v);
                }
            }
        }
    }
};
