// FP32 SGEMM kernel for problems that cannot fill the GPU with 128 x 128 tiles: 128 x 64 tile, 128
// threads (four warps stacked along M), 8 x 8 outputs per thread with scalar FFMA, cp.async
// multi-stage shared-memory ring, fragments double buffered in registers.
//
// At M = N = K = 1024 this gives 128 blocks -- one per SM on 128 of the 148 SMs -- with a single
// pass over K and no split, so every output is accumulated with one FMA per k in ascending k
// exactly like the reference (nn_operators/gemm/simt_gemm.h:202-222): bit-identical results.
// Same data path as the 128 x 128 kernel (simt_gemm_x2.h): A is copied 4 bytes at a time straight
// into a transposed, conflict-free shared tile, B in 16-byte pieces, out-of-range elements are
// zero-filled by cp.async's source size, so any M, N, K is legal.
#pragma once

#include "../../common/common.h"
#include "simt_gemm_x2.h"  // cp.async wrappers

namespace ko {
namespace sgemm8 {

constexpr int BM = 128, BN = 64, BK = 16;
constexpr int kThreads = 128;
constexpr int kStages = 4;
constexpr int kStrideA = BM + 4;
constexpr int kStrideB = BN;
constexpr int kStageFloats = BK * kStrideA + BK * kStrideB;
constexpr int kSmemBytes = kStages * kStageFloats * (int)sizeof(float);

struct Params {
    int M, N, K;
    const float *A, *B, *C;
    float *D;
};

template <bool kVecB>
__global__ void __launch_bounds__(kThreads) sgemm_a8_kernel(const Params p) {
    using sgemm2::cp_async_4;
    using sgemm2::cp_async_16;
    using sgemm2::cp_async_commit;
    extern __shared__ __align__(16) float smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int lane_m = lane >> 3, lane_n = lane & 7;
    const int tiles_n = (p.N + BN - 1) / BN;
    const int m_base = (blockIdx.x / tiles_n) * BM, n_base = (blockIdx.x % tiles_n) * BN;
    const int ktiles = (p.K + BK - 1) / BK;
    const uint32_t smem_base = smem_u32(smem);

    auto issue_tile = [&](int kt, int stage) {
        const int k0 = kt * BK;
        const uint32_t as = smem_base + (uint32_t)stage * kStageFloats * 4u;
        const uint32_t bs = as + BK * kStrideA * 4u;
#pragma unroll
        for (int i = 0; i < (BM * BK) / kThreads; ++i) {
            const int e = tid + i * kThreads;             // 0 .. 2047; a warp covers 4 rows x 8 consecutive k
            const int k = (e & 7) | ((e >> 9) & 1) << 3;
            const int m = (e >> 3) & 63 | ((e >> 10) & 1) << 6;
            const int gm = m_base + m, gk = k0 + k;
            const bool ok = gm < p.M && gk < p.K;
            cp_async_4(as + (uint32_t)(k * kStrideA + m) * 4u, p.A + (ok ? (size_t)gm * p.K + gk : 0), ok);
        }
        if (kVecB) {
#pragma unroll
            for (int i = 0; i < (BK * BN / 4) / kThreads; ++i) {
                const int e = tid + i * kThreads;  // 0 .. 255
                const int k = e >> 4, n = (e & 15) * 4;
                const int gk = k0 + k, gn = n_base + n;
                const bool ok = gk < p.K && gn < p.N;
                cp_async_16(bs + (uint32_t)(k * kStrideB + n) * 4u, p.B + (ok ? (size_t)gk * p.N + gn : 0), ok);
            }
        } else {
#pragma unroll
            for (int i = 0; i < (BK * BN) / kThreads; ++i) {
                const int e = tid + i * kThreads;  // 0 .. 1023
                const int k = e >> 6, n = e & 63;
                const int gk = k0 + k, gn = n_base + n;
                const bool ok = gk < p.K && gn < p.N;
                cp_async_4(bs + (uint32_t)(k * kStrideB + n) * 4u, p.B + (ok ? (size_t)gk * p.N + gn : 0), ok);
            }
        }
    };

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

#pragma unroll
    for (int s = 0; s < kStages - 1; ++s) {
        if (s < ktiles) issue_tile(s, s);
        cp_async_commit();
    }

    const int a_off = warp * 32 + lane_m * 4;  // + q * 16
    const int b_off = lane_n * 4;              // + q * 32
    float4 fa[2][2], fb[2][2];
    auto load_frag = [&](int buf, const float *as, const float *bs, int kk) {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            fa[buf][q] = *reinterpret_cast<const float4 *>(as + kk * kStrideA + q * 16);
            fb[buf][q] = *reinterpret_cast<const float4 *>(bs + kk * kStrideB + q * 32);
        }
    };

    for (int t = 0; t < ktiles; ++t) {
        sgemm2::cp_async_wait<kStages - 2>();
        __syncthreads();
        if (t + kStages - 1 < ktiles) issue_tile(t + kStages - 1, (t + kStages - 1) % kStages);
        cp_async_commit();

        const float *as = smem + (t % kStages) * kStageFloats + a_off;
        const float *bs = smem + (t % kStages) * kStageFloats + BK * kStrideA + b_off;
        load_frag(0, as, bs, 0);
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            const int cur = kk & 1;
            if (kk + 1 < BK) load_frag(cur ^ 1, as, bs, kk + 1);
            const float av[8] = {fa[cur][0].x, fa[cur][0].y, fa[cur][0].z, fa[cur][0].w,
                                 fa[cur][1].x, fa[cur][1].y, fa[cur][1].z, fa[cur][1].w};
            const float bv[8] = {fb[cur][0].x, fb[cur][0].y, fb[cur][0].z, fb[cur][0].w,
                                 fb[cur][1].x, fb[cur][1].y, fb[cur][1].z, fb[cur][1].w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
    }
    sgemm2::cp_async_wait<0>();

    const bool vec_out = (p.N % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.D) & 15u) == 0) &&
                         (p.C == nullptr || (reinterpret_cast<uintptr_t>(p.C) & 15u) == 0);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int m = m_base + a_off + (i >> 2) * 16 + (i & 3);
        if (m >= p.M) continue;
#pragma unroll
        for (int jq = 0; jq < 2; ++jq) {
            const int n = n_base + b_off + jq * 32;
            if (n >= p.N) continue;
            const size_t off = (size_t)m * p.N + n;
            float4 o = make_float4(acc[i][jq * 4], acc[i][jq * 4 + 1], acc[i][jq * 4 + 2], acc[i][jq * 4 + 3]);
            if (vec_out) {
                if (p.C) {
                    const float4 c = *reinterpret_cast<const float4 *>(p.C + off);
                    o.x += c.x; o.y += c.y; o.z += c.z; o.w += c.w;
                }
                *reinterpret_cast<float4 *>(p.D + off) = o;
            } else {
                const float v[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (n + j < p.N) p.D[off + j] = p.C ? v[j] + p.C[off + j] : v[j];
            }
        }
    }
}

}  // namespace sgemm8
}  // namespace ko
