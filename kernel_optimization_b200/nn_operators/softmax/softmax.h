// Row softmax over the last dimension for sm_100a.
//
// Three tiers, chosen by row length (the reference's warp / block-cached / block-no-cache split,
// nn_operators/softmax/softmax.h:11-60, :62-113, :116-166, re-thought for B200):
//
//   warp tier   one warp owns kRows consecutive rows per step; each row sits in registers as
//               kVecs 128-bit vectors per lane; every load of the step is issued before the
//               first use, so a warp keeps kRows*kVecs*512 B in flight.  Max and sum are
//               butterfly all-reduces.  Reads and writes each byte once.
//   block tier  one thread block per row, the row in registers (kVecs vectors per thread),
//               warp all-reduce + one shared-memory exchange per statistic.
//   stream tier one thread block per row, three passes over global memory with scalar
//               accesses; any column count and any alignment (correctness path).
//
// All tiers compute exp(x - rowmax) / sum in FP32 (the reference's Subtract functor adds,
// common/functors.h:168, so it evaluates exp(x + rowmax); the two agree mathematically but the
// reference overflows once 2*rowmax > 88.7).
//
// The reference's class templates SoftMaxWarpImpl / SoftMaxBlockImpl / SoftMaxBlockNoCacheImpl and
// the softmax<Kernel> __global__ wrapper keep their names, template parameters and static members,
// so `softmax<SoftMaxWarpImpl<float, 4, R, C>><<<grid, block, smem, stream>>>(in, out)` still
// compiles; every tier is a grid-stride loop and therefore correct for any launch geometry.
#pragma once

#include "../../common/common.h"
#include "../../common/functors.h"

namespace ko {

constexpr float kNegInf = -__builtin_huge_valf();

__device__ __forceinline__ float max4(const float4 &v) { return fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)); }

// ---------------------------------------------------------------------------------------------
// warp tier
// ---------------------------------------------------------------------------------------------
template <int kVecs, int kRows>
__device__ __forceinline__ void softmax_warp_tier(const float *in, float *out, long long rows, int cols) {
    const int lane = threadIdx.x & 31;
    const int nvec = cols >> 2;  // 128-bit vectors per row
    const long long warps_per_grid = (long long)gridDim.x * (blockDim.x >> 5);
    const long long warp_global = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const float4 *in4 = reinterpret_cast<const float4 *>(in);
    float4 *out4 = reinterpret_cast<float4 *>(out);

    for (long long row0 = warp_global * kRows; row0 < rows; row0 += warps_per_grid * kRows) {
        float4 x[kRows][kVecs];
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            const bool row_ok = row0 + r < rows;
#pragma unroll
            for (int j = 0; j < kVecs; ++j) {
                const int v = lane + 32 * j;
                x[r][j] = (row_ok && v < nvec) ? ld_stream(in4 + (row0 + r) * nvec + v)
                                               : make_float4(kNegInf, kNegInf, kNegInf, kNegInf);
            }
        }
        float mx[kRows];
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            float m = max4(x[r][0]);
#pragma unroll
            for (int j = 1; j < kVecs; ++j) m = fmaxf(m, max4(x[r][j]));
            mx[r] = m;
        }
#pragma unroll
        for (int r = 0; r < kRows; ++r) mx[r] = warp_allreduce_max(mx[r]);

        float sum[kRows];
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            float s = 0.f;
#pragma unroll
            for (int j = 0; j < kVecs; ++j) {
                x[r][j].x = expf(x[r][j].x - mx[r]);
                x[r][j].y = expf(x[r][j].y - mx[r]);
                x[r][j].z = expf(x[r][j].z - mx[r]);
                x[r][j].w = expf(x[r][j].w - mx[r]);
                s += (x[r][j].x + x[r][j].y) + (x[r][j].z + x[r][j].w);
            }
            sum[r] = s;
        }
#pragma unroll
        for (int r = 0; r < kRows; ++r) sum[r] = warp_allreduce_sum(sum[r]);

#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            const float inv = 1.0f / sum[r];
            const bool row_ok = row0 + r < rows;
#pragma unroll
            for (int j = 0; j < kVecs; ++j) {
                const int v = lane + 32 * j;
                if (row_ok && v < nvec) {
                    float4 y = x[r][j];
                    y.x *= inv; y.y *= inv; y.z *= inv; y.w *= inv;
                    st_stream(out4 + (row0 + r) * nvec + v, y);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// block tier: one row per thread block, row in registers
// ---------------------------------------------------------------------------------------------
// s_exchange: at least 33 floats
template <bool kIsMax>
__device__ __forceinline__ float block_allreduce(float v, float *s_exchange) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    v = kIsMax ? warp_allreduce_max(v) : warp_allreduce_sum(v);
    __syncthreads();
    if (lane == 0) s_exchange[warp] = v;
    __syncthreads();
    float t = lane < nwarps ? s_exchange[lane] : (kIsMax ? kNegInf : 0.f);
    return kIsMax ? warp_allreduce_max(t) : warp_allreduce_sum(t);
}

template <int kVecs>
__device__ __forceinline__ void softmax_block_tier(const float *in, float *out, long long rows, int cols,
                                                   float *s_exchange) {
    const int nvec = cols >> 2;
    const float4 *in4 = reinterpret_cast<const float4 *>(in);
    float4 *out4 = reinterpret_cast<float4 *>(out);
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        float4 x[kVecs];
        float m = kNegInf;
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            const int v = threadIdx.x + blockDim.x * j;
            x[j] = v < nvec ? ld_stream(in4 + row * nvec + v) : make_float4(kNegInf, kNegInf, kNegInf, kNegInf);
            m = fmaxf(m, max4(x[j]));
        }
        m = block_allreduce<true>(m, s_exchange);
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            x[j].x = expf(x[j].x - m); x[j].y = expf(x[j].y - m);
            x[j].z = expf(x[j].z - m); x[j].w = expf(x[j].w - m);
            s += (x[j].x + x[j].y) + (x[j].z + x[j].w);
        }
        s = block_allreduce<false>(s, s_exchange);
        const float inv = 1.0f / s;
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            const int v = threadIdx.x + blockDim.x * j;
            if (v < nvec) {
                float4 y = x[j];
                y.x *= inv; y.y *= inv; y.z *= inv; y.w *= inv;
                st_stream(out4 + row * nvec + v, y);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// stream tier: any cols, any alignment; three passes over global memory
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void softmax_stream_tier(const float *in, float *out, long long rows, int cols,
                                                    float *s_exchange) {
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const float *x = in + row * cols;
        float *y = out + row * cols;
        float m = kNegInf;
        for (int c = threadIdx.x; c < cols; c += blockDim.x) m = fmaxf(m, x[c]);
        m = block_allreduce<true>(m, s_exchange);
        float s = 0.f;
        for (int c = threadIdx.x; c < cols; c += blockDim.x) s += expf(x[c] - m);
        s = block_allreduce<false>(s, s_exchange);
        const float inv = 1.0f / s;
        for (int c = threadIdx.x; c < cols; c += blockDim.x) y[c] = expf(x[c] - m) * inv;
        __syncthreads();
    }
}

// runtime-shape kernels used by the C ABI
template <int kVecs, int kRows>
__global__ void __launch_bounds__(256) softmax_warp_kernel(const float *in, float *out, long long rows, int cols) {
    softmax_warp_tier<kVecs, kRows>(in, out, rows, cols);
}
template <int kVecs, int kThreads>
__global__ void __launch_bounds__(kThreads) softmax_block_kernel(const float *in, float *out, long long rows, int cols) {
    __shared__ float s_exchange[33];
    softmax_block_tier<kVecs>(in, out, rows, cols, s_exchange);
}
__global__ void __launch_bounds__(256) softmax_stream_kernel(const float *in, float *out, long long rows, int cols) {
    __shared__ float s_exchange[33];
    softmax_stream_tier(in, out, rows, cols, s_exchange);
}

}  // namespace ko

// ---------------------------------------------------------------------------------------------
// source-level drop-in for the reference's launch syntax (compile-time shapes, FP32)
// ---------------------------------------------------------------------------------------------
template <typename T_, int vec_len_, int num_row_, int num_column_>
struct SoftMaxWarpImpl {
    using T = T_;
    static constexpr int vec_len = vec_len_, num_row = num_row_, num_column = num_column_;
    static constexpr int smem_in_bytes = 0;
    static_assert(num_column % 4 == 0, "the warp tier moves 128-bit vectors");
    static constexpr int kVecs = (num_column / 4 + 31) / 32;
    static_assert(kVecs <= 16, "row too long for the warp tier; use SoftMaxBlockImpl");
    static constexpr int kRows = kVecs >= 8 ? 1 : (kVecs >= 4 ? 2 : 4);
    __device__ __forceinline__ static void run(T *in_data, T *out_data) {
        ko::softmax_warp_tier<kVecs, kRows>(in_data, out_data, num_row, num_column);
    }
};

template <typename T_, int vec_len_, int num_row_, int num_column_>
struct SoftMaxBlockImpl {
    using T = T_;
    static constexpr int vec_len = vec_len_, num_row = num_row_, num_column = num_column_;
    // the row lives in registers, not shared memory; 33 floats are used for the exchange
    static constexpr int smem_in_bytes = 33 * sizeof(float);
    __device__ __forceinline__ static void run(T *in_data, T *out_data) {
        extern __shared__ float ko_softmax_dyn_smem[];
        // up to 16 vectors per thread; longer rows (or tiny blocks) fall through to the stream tier
        if (num_column % 4 == 0 && num_column / 4 <= 16 * (int)blockDim.x)
            ko::softmax_block_tier<16>(in_data, out_data, num_row, num_column, ko_softmax_dyn_smem);
        else
            ko::softmax_stream_tier(in_data, out_data, num_row, num_column, ko_softmax_dyn_smem);
    }
};

template <typename T_, int vec_len_, int num_row_, int num_column_>
struct SoftMaxBlockNoCacheImpl {
    using T = T_;
    static constexpr int vec_len = vec_len_, num_row = num_row_, num_column = num_column_;
    static constexpr int smem_in_bytes = 33 * sizeof(float);
    __device__ __forceinline__ static void run(T *in_data, T *out_data) {
        extern __shared__ float ko_softmax_dyn_smem[];
        ko::softmax_stream_tier(in_data, out_data, num_row, num_column, ko_softmax_dyn_smem);
    }
};

template <typename SoftMaxKernel>
__global__ void softmax(typename SoftMaxKernel::T *in_data, typename SoftMaxKernel::T *out_data) {
    SoftMaxKernel::run(in_data, out_data);
}
