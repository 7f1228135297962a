// Row softmax with FP16 or BF16 input and output, FP32 arithmetic, for sm_100a.
//
// The reference gives its row operators `half` building blocks -- Exp<half> (common/functors.h:71-77),
// numeric_limits<half> (common/common.h:171-177) -- but only ever instantiates them for float
// (nn_operators/softmax/main.cu:78-79).  Here 16-bit rows are read as 16-byte vectors of 8 elements,
// widened to FP32, pushed through the same max / 2^((x - max) log2 e) / sum / scale steps as the FP32
// tiers (softmax.h), and rounded to nearest even once on the way out: the statistics never see 16-bit
// precision, so a row of 65504s or of -65504s is exact.  (As in the FP32 tiers the exponent is formed as
// fma(x, log2 e, -fl(max log2 e)): the rounding of the shift is the same for every element of the row and
// cancels in the quotient, but it grows with |max| -- half an ulp of max log2 e -- and must stay far below
// the exponent range, which holds for |x| < 1e9: all of FP16, not all of BF16.)
//
//   warp tier   a row over a group of 8, 16 or 32 lanes, up to 8 vectors (64 elements) per lane,
//               two rows per lane group in flight; columns a multiple of 8, up to 2048
//   block tier  one row per block of exactly the threads it needs (a multiple of 32, at most 512) with three or six
//               vectors per thread: up to 24576 columns
//   reread tier one row per block in two passes, the second from the L2: rows beyond 24576 columns
//   stream tier any column count and alignment, scalar accesses, three passes
#pragma once

#include "softmax.h"

namespace ko {

template <typename T>
struct Half8;  // 16-byte vector of 8 T <-> 8 floats

template <>
struct Half8<__half> {
    __device__ __forceinline__ static void unpack(const uint4 &r, float (&f)[8]) {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 p = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
            f[2 * i] = p.x;
            f[2 * i + 1] = p.y;
        }
    }
    __device__ __forceinline__ static uint4 pack(const float (&f)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t *>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    __device__ __forceinline__ static float widen(__half v) { return __half2float(v); }
    __device__ __forceinline__ static __half narrow(float v) { return __float2half_rn(v); }
};

template <>
struct Half8<__nv_bfloat16> {
    __device__ __forceinline__ static void unpack(const uint4 &r, float (&f)[8]) {
        f[0] = bf16_lo(r.x); f[1] = bf16_hi(r.x); f[2] = bf16_lo(r.y); f[3] = bf16_hi(r.y);
        f[4] = bf16_lo(r.z); f[5] = bf16_hi(r.z); f[6] = bf16_lo(r.w); f[7] = bf16_hi(r.w);
    }
    __device__ __forceinline__ static uint4 pack(const float (&f)[8]) {
        return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
    }
    __device__ __forceinline__ static float widen(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ __forceinline__ static __nv_bfloat16 narrow(float v) { return __float2bfloat16_rn(v); }
};

// max of 8, then in place to 2^(x log2e + neg) with the sum returned, then scaled
__device__ __forceinline__ float max8(const float (&f)[8]) {
    return fmaxf(fmaxf(fmaxf(f[0], f[1]), fmaxf(f[2], f[3])), fmaxf(fmaxf(f[4], f[5]), fmaxf(f[6], f[7])));
}
__device__ __forceinline__ float exp_shifted8(float (&f)[8], float neg_m_log2e) {
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = exp2_approx(fmaf(f[e], kLog2e, neg_m_log2e));
    return ((f[0] + f[1]) + (f[2] + f[3])) + ((f[4] + f[5]) + (f[6] + f[7]));
}

// ---------------------------------------------------------------------------------------------
// warp tier: kSlots rows per lane group in flight, kVecs 16-byte vectors per lane and row
// ---------------------------------------------------------------------------------------------
template <typename T, int kVecs, int kSlots, int G>
__global__ void __launch_bounds__(256) softmax16_warp_kernel(const T *in, T *out, long long rows, int cols) {
    using Io = Half8<T>;
    constexpr int kRowsPerSlot = 32 / G, kRowsPerStep = kSlots * kRowsPerSlot;
    const int lane = threadIdx.x & 31, sub = lane / G, gl = lane % G;
    const int nvec = cols >> 3;
    const long long warps_per_grid = (long long)gridDim.x * (blockDim.x >> 5);
    const long long warp_global = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const uint4 *in_v = reinterpret_cast<const uint4 *>(in);
    uint4 *out_v = reinterpret_cast<uint4 *>(out);
    grid_launch_dependents();  // launched with programmatic stream serialization: see common.h
    grid_dependency_wait();

    for (long long row0 = warp_global * kRowsPerStep; row0 < rows; row0 += warps_per_grid * kRowsPerStep) {
        // every load of the step is issued before the first use
        uint4 raw[kSlots][kVecs];
#pragma unroll
        for (int r = 0; r < kSlots; ++r) {
            const long long row = row0 + r * kRowsPerSlot + sub;
#pragma unroll
            for (int j = 0; j < kVecs; ++j) {
                const int v = gl + G * j;
                raw[r][j] = (row < rows && v < nvec) ? ld_stream(in_v + row * nvec + v) : make_uint4(0u, 0u, 0u, 0u);
            }
        }
#pragma unroll
        for (int r = 0; r < kSlots; ++r) {
            const long long row = row0 + r * kRowsPerSlot + sub;
            float x[kVecs][8];
            float m = kNegInf;
#pragma unroll
            for (int j = 0; j < kVecs; ++j) {
                Io::unpack(raw[r][j], x[j]);
                if (!(row < rows && gl + G * j < nvec)) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) x[j][e] = kNegInf;  // padding: contributes 2^(-inf) = 0
                }
                m = fmaxf(m, max8(x[j]));
            }
            m = group_allreduce_max<G>(m);
            const float neg = -m * kLog2e;
            float s = 0.f;
#pragma unroll
            for (int j = 0; j < kVecs; ++j) s += exp_shifted8(x[j], neg);
            s = group_allreduce_sum<G>(s);
            const float inv = rcp_approx(s);
#pragma unroll
            for (int j = 0; j < kVecs; ++j) {
                const int v = gl + G * j;
                if (row < rows && v < nvec) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) x[j][e] *= inv;
                    st_stream(out_v + row * nvec + v, Io::pack(x[j]));
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// block tier: one row per block, the row in registers (kThreads: the most threads a block may have; the block size is read
// at run time, so that a launch can bring exactly the threads the row needs)
// ---------------------------------------------------------------------------------------------
template <typename T, int kVecs, int kThreads>
__global__ void __launch_bounds__(kThreads) softmax16_block_kernel(const T *in, T *out, long long rows, int cols) {
    using Io = Half8<T>;
    __shared__ float s_exchange[33];
    const int nvec = cols >> 3;
    const uint4 *in_v = reinterpret_cast<const uint4 *>(in);
    uint4 *out_v = reinterpret_cast<uint4 *>(out);
    grid_launch_dependents();
    grid_dependency_wait();
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        float x[kVecs][8];
        float m = kNegInf;
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            const int v = threadIdx.x + blockDim.x * j;
            if (v < nvec) {
                Io::unpack(ld_stream(in_v + row * nvec + v), x[j]);
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) x[j][e] = kNegInf;
            }
            m = fmaxf(m, max8(x[j]));
        }
        m = block_allreduce<true>(m, s_exchange);
        const float neg = -m * kLog2e;
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < kVecs; ++j) s += exp_shifted8(x[j], neg);
        s = block_allreduce<false>(s, s_exchange);
        const float inv = rcp_approx(s);
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            const int v = threadIdx.x + blockDim.x * j;
            if (v < nvec) {
#pragma unroll
                for (int e = 0; e < 8; ++e) x[j][e] *= inv;
                st_stream(out_v + row * nvec + v, Io::pack(x[j]));
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// reread tier: one row per block in two passes, the second served by the L2 (see softmax_reread_tier)
// ---------------------------------------------------------------------------------------------
template <typename T, int kUnroll, int kThreads>
__global__ void __launch_bounds__(kThreads) softmax16_reread_kernel(const T *in, T *out, long long rows, int cols) {
    using Io = Half8<T>;
    __shared__ float s_exchange[33];
    const int nvec = cols >> 3;
    constexpr int kStep = kThreads * kUnroll;
    const uint64_t keep = l2_keep_policy();
    grid_launch_dependents();
    grid_dependency_wait();
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const uint4 *x_v = reinterpret_cast<const uint4 *>(in) + row * nvec;
        uint4 *y_v = reinterpret_cast<uint4 *>(out) + row * nvec;
        float m = kNegInf, s = 0.f;
        for (int base = 0; base < nvec; base += kStep) {
            uint4 raw[kUnroll];
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                const int v = base + (int)threadIdx.x + kThreads * j;
                raw[j] = v < nvec ? ld_keep(x_v + v, keep) : uint4{0u, 0u, 0u, 0u};
            }
            float x[kUnroll][8];
            float cm = kNegInf;
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                const int v = base + (int)threadIdx.x + kThreads * j;
                Io::unpack(raw[j], x[j]);
                if (v >= nvec) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) x[j][e] = kNegInf;
                }
                cm = fmaxf(cm, max8(x[j]));
            }
            const float grown = fmaxf(m, cm);
            if (grown != kNegInf) {  // a chunk of nothing but -inf adds nothing
                const float neg = -grown * kLog2e;
                float cs = 0.f;
#pragma unroll
                for (int j = 0; j < kUnroll; ++j) cs += exp_shifted8(x[j], neg);
                s = fmaf(s, exp2_approx(fmaf(m, kLog2e, neg)), cs);
                m = grown;
            }
        }
        const float row_max = block_allreduce<true>(m, s_exchange);
        const float neg = -row_max * kLog2e;
        s = m == kNegInf ? 0.f : s * exp2_approx(fmaf(m, kLog2e, neg));
        const float inv = rcp_approx(block_allreduce<false>(s, s_exchange));
        for (int base = 0; base < nvec; base += kStep) {
            uint4 raw[kUnroll];
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                const int v = base + (int)threadIdx.x + kThreads * j;
                if (v < nvec) raw[j] = ld_stream(x_v + v);
            }
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                const int v = base + (int)threadIdx.x + kThreads * j;
                if (v < nvec) {
                    float x[8];
                    Io::unpack(raw[j], x);
                    exp_shifted8(x, neg);
#pragma unroll
                    for (int e = 0; e < 8; ++e) x[e] *= inv;
                    st_stream(y_v + v, Io::pack(x));
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// stream tier: any cols, any alignment
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) softmax16_stream_kernel(const T *in, T *out, long long rows, int cols) {
    using Io = Half8<T>;
    __shared__ float s_exchange[33];
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const T *x = in + row * cols;
        T *y = out + row * cols;
        float m = kNegInf;
        for (int c = threadIdx.x; c < cols; c += blockDim.x) m = fmaxf(m, Io::widen(x[c]));
        m = block_allreduce<true>(m, s_exchange);
        const float neg = -m * kLog2e;
        float s = 0.f;
        for (int c = threadIdx.x; c < cols; c += blockDim.x) s += exp2_approx(fmaf(Io::widen(x[c]), kLog2e, neg));
        s = block_allreduce<false>(s, s_exchange);
        const float inv = rcp_approx(s);
        for (int c = threadIdx.x; c < cols; c += blockDim.x)
            y[c] = Io::narrow(exp2_approx(fmaf(Io::widen(x[c]), kLog2e, neg)) * inv);
        __syncthreads();
    }
}

}  // namespace ko
