// FP32 SGEMM main kernel for sm_100a: 128 x 128 tile, 128 threads, 16 x 8 outputs per thread,
// packed FFMA (fma.rn.f32x2), cp.async multi-stage shared-memory pipeline, optional split-K.
//
// Why this shape.  One FP32 FMA needs two operands from shared memory; with 128-bit shared loads a
// warp spends (TM + TN) shared-memory wavefronts per k for TM*TN FMA instructions, and the SM retires
// four FMA instructions per wavefront slot.  An 8 x 8 thread tile therefore saturates shared memory
// exactly when it saturates the FMA pipe; 16 x 8 leaves 25% slack.  fma.rn.f32x2 performs two
// IEEE-rounded FMAs per issue slot, which frees issue bandwidth for the shared loads and cp.async.
//
// Data path: A[M,K] row-major is copied 4 bytes at a time straight into a TRANSPOSED shared tile
// As[k][m] (cp.async with a source size of 0 zero-fills out-of-range elements, so every M, N, K is
// legal and nothing is read out of bounds -- the reference prefetches past the end,
// nn_operators/gemm/simt_gemm.h:287-292); B[K,N] goes in 16-byte pieces.  kStages tiles are in flight.
//
// Work distribution ("stream-K"): the (tile, K-tile) pairs form one linear sequence of units that is
// cut into `ctas` equal contiguous ranges, one per block.  With ctas == tiles every block owns one
// whole tile; with ctas == tiles * s every tile is cut into s K-slices (classic split-K); any other
// count (e.g. two blocks per SM) gives ranges that may end one tile and begin the next, so that a
// problem with few tiles still keeps every SM busy for the same time.
//
// Accumulation order: one FMA per k in ascending k per output, as in the reference
// (simt_gemm.h:202-222).  A tile computed by one block is bit-identical to that order; a tile shared
// by several blocks has each K-range accumulated that way and the ranges added in K order by the block
// that finishes last (deterministic; no atomics on data, no waiting between blocks).
#pragma once

#include "../../common/common.h"

namespace ko {
namespace sgemm2 {

constexpr int BM = 128, BN = 128, BK = 16;
constexpr int kThreads = 128;
constexpr int kStages = 4;
constexpr int kStrideA = BM + 4;   // 132: (4*k + m) mod 32 distinct for k < 8, m < 4 -> conflict-free transposed writes
constexpr int kStrideB = BN;
constexpr int kStageFloats = BK * kStrideA + BK * kStrideB;
constexpr int kSmemBytes = kStages * kStageFloats * (int)sizeof(float);
constexpr int kTileFloats = BM * BN;

using u64 = unsigned long long;

__device__ __forceinline__ u64 pack2(float lo, float hi) {
    u64 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(u64 v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
// c = a * b + c on both halves, round to nearest even
__device__ __forceinline__ void fma2(u64 &c, u64 a, u64 b) { asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(c) : "l"(a), "l"(b)); }

__device__ __forceinline__ void cp_async_4(uint32_t dst, const void *src, bool valid) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(valid ? 4 : 0) : "memory");
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void *src, bool valid) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(valid ? 16 : 0) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

struct Params {
    int M, N, K;
    const float *A, *B, *C;
    float *D;
    int ctas;           // blocks sharing the tiles * ktiles work units (== gridDim.x)
    int max_contrib;    // upper bound on the blocks that touch one tile (workspace slots per tile)
    float *workspace;   // [tiles][max_contrib][BM*BN] partial tiles (used when a tile is shared)
    unsigned *counters; // one arrival counter per tile, zero between launches
};

// the block whose unit range [b*U/G, (b+1)*U/G) contains unit u
__device__ __forceinline__ int block_of_unit(long long u, long long U, int G) {
    int b = (int)(u * G / U);
    while ((long long)(b + 1) * U / G <= u) ++b;
    while ((long long)b * U / G > u) --b;
    return b;
}

// kVecB: N % 4 == 0 and B 16-byte aligned (16-byte copies of B); otherwise 4-byte copies
template <bool kVecB>
__global__ void __launch_bounds__(kThreads) sgemm_x2_kernel(const Params p) {
    extern __shared__ __align__(16) float smem[];
    __shared__ int s_is_last;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int warp_m = warp >> 1, warp_n = warp & 1;   // 2 x 2 warps of 64 x 64
    const int lane_m = lane >> 3, lane_n = lane & 7;   // 4 x 8 lanes of 16 x 8
    const int tiles_n = (p.N + BN - 1) / BN;
    const int ktiles_total = (p.K + BK - 1) / BK;
    const long long units = (long long)((p.M + BM - 1) / BM) * tiles_n * ktiles_total;
    const long long unit_begin = units * blockIdx.x / p.ctas, unit_end = units * (blockIdx.x + 1) / p.ctas;

    const uint32_t smem_base = smem_u32(smem);
    int m_base = 0, n_base = 0;
    auto issue_tile = [&](int kt, int stage) {
        const int k0 = kt * BK;
        const uint32_t as = smem_base + (uint32_t)stage * kStageFloats * 4u;
        const uint32_t bs = as + BK * kStrideA * 4u;
        // A: a warp instruction covers 4 rows x 8 consecutive k (4 full 32-byte sectors)
#pragma unroll
        for (int i = 0; i < (BM * BK) / kThreads; ++i) {
            const int e = tid + i * kThreads;             // 0 .. 2047
            const int k = (e & 7) | ((e >> 9) & 1) << 3;  // low 3 bits, then bit 9 picks the k half
            const int m = (e >> 3) & 63 | ((e >> 10) & 1) << 6;
            const int gm = m_base + m, gk = k0 + k;
            const bool ok = gm < p.M && gk < p.K;
            cp_async_4(as + (uint32_t)(k * kStrideA + m) * 4u, p.A + (ok ? (size_t)gm * p.K + gk : 0), ok);
        }
        if (kVecB) {
#pragma unroll
            for (int i = 0; i < (BK * BN / 4) / kThreads; ++i) {
                const int e = tid + i * kThreads;  // 0 .. 511
                const int k = e >> 5, n = (e & 31) * 4;
                const int gk = k0 + k, gn = n_base + n;
                const bool ok = gk < p.K && gn < p.N;
                cp_async_16(bs + (uint32_t)(k * kStrideB + n) * 4u, p.B + (ok ? (size_t)gk * p.N + gn : 0), ok);
            }
        } else {
#pragma unroll
            for (int i = 0; i < (BK * BN) / kThreads; ++i) {
                const int e = tid + i * kThreads;  // 0 .. 2047
                const int k = e >> 7, n = e & 127;
                const int gk = k0 + k, gn = n_base + n;
                const bool ok = gk < p.K && gn < p.N;
                cp_async_4(bs + (uint32_t)(k * kStrideB + n) * 4u, p.B + (ok ? (size_t)gk * p.N + gn : 0), ok);
            }
        }
    };

    const int a_off = warp_m * 64 + lane_m * 4;  // + q * 16, q = 0..3
    const int b_off = warp_n * 64 + lane_n * 4;  // + q * 32, q = 0..1

    for (long long u = unit_begin; u < unit_end;) {
    // ---- one segment: K-tiles [kt_begin, kt_end) of one output tile
    const int tile = (int)(u / ktiles_total);
    const int kt_begin = (int)(u % ktiles_total);
    const int kt_end = (int)min((long long)ktiles_total, kt_begin + (unit_end - u));
    const int ktiles = kt_end - kt_begin;
    u += ktiles;
    const bool whole_tile = ktiles == ktiles_total;
    m_base = (tile / tiles_n) * BM;
    n_base = (tile % tiles_n) * BN;
    __syncthreads();  // the previous segment's shared-memory reads (and s_is_last) are done

    // acc[ip][j]: rows (2*ip, 2*ip+1) of the thread's 16, column j of its 8
    u64 acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0ull;

    // prologue: kStages - 1 tiles in flight
#pragma unroll
    for (int s = 0; s < kStages - 1; ++s) {
        if (s < ktiles) issue_tile(kt_begin + s, s);
        cp_async_commit();
    }

    for (int t = 0; t < ktiles; ++t) {
        cp_async_wait<kStages - 2>();
        __syncthreads();  // tile t has landed for every thread; the stage refilled below was consumed at t-1
        if (t + kStages - 1 < ktiles) issue_tile(kt_begin + t + kStages - 1, (t + kStages - 1) % kStages);
        cp_async_commit();

        const float *as = smem + (t % kStages) * kStageFloats + a_off;
        const float *bs = smem + (t % kStages) * kStageFloats + BK * kStrideA + b_off;
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            // A pairs (rows 2ip, 2ip+1) come out of shared memory as 64-bit values: no packing needed
            u64 a2[8], b2[8];
            float4 b4[2];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const ulonglong2 v = *reinterpret_cast<const ulonglong2 *>(as + kk * kStrideA + q * 16);
                a2[2 * q] = v.x;
                a2[2 * q + 1] = v.y;
            }
#pragma unroll
            for (int q = 0; q < 2; ++q) b4[q] = *reinterpret_cast<const float4 *>(bs + kk * kStrideB + q * 32);
            const float bv[8] = {b4[0].x, b4[0].y, b4[0].z, b4[0].w, b4[1].x, b4[1].y, b4[1].z, b4[1].w};
#pragma unroll
            for (int j = 0; j < 8; ++j) b2[j] = pack2(bv[j], bv[j]);
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) fma2(acc[i][j], a2[i], b2[j]);
        }
    }
    cp_async_wait<0>();

    // thread's outputs: row(ip, h) = m_base + a_off + (ip/2)*16 + (ip%2)*2 + h, col(j) = n_base + b_off + (j/4)*32 + j%4
    auto row_of = [&](int ip, int h) { return m_base + a_off + (ip >> 1) * 16 + (ip & 1) * 2 + h; };
    auto col_of = [&](int jq) { return n_base + b_off + jq * 32; };

    // final values of this thread's 32 float4 chunks (chunk c = (ip*2 + h)*2 + jq)
    float4 out[32];
#pragma unroll
    for (int ip = 0; ip < 8; ++ip)
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int jq = 0; jq < 2; ++jq) {
                float v[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float lo, hi;
                    unpack2(acc[ip][jq * 4 + j], lo, hi);
                    v[j] = h ? hi : lo;
                }
                out[(ip * 2 + h) * 2 + jq] = make_float4(v[0], v[1], v[2], v[3]);
            }
    int contributors = 1, slot = 0;
    if (!whole_tile) {
        const long long first_unit = (long long)tile * ktiles_total;
        const int first_block = block_of_unit(first_unit, units, p.ctas);
        contributors = block_of_unit(first_unit + ktiles_total - 1, units, p.ctas) - first_block + 1;
        slot = (int)blockIdx.x - first_block;
    }
    bool finish_tile = true;
    if (!whole_tile) {
        // publish this K-range's partial tile: [tile][slot][chunk][thread] float4, coalesced
        float4 *mine = reinterpret_cast<float4 *>(p.workspace + ((size_t)tile * p.max_contrib + slot) * kTileFloats);
#pragma unroll
        for (int c = 0; c < 32; ++c) mine[c * kThreads + tid] = out[c];
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const unsigned prev = atomicAdd(p.counters + tile, 1u);
            s_is_last = (prev == (unsigned)contributors - 1u);
        }
        __syncthreads();
        finish_tile = s_is_last != 0;
        if (finish_tile) __threadfence();
    }
    if (finish_tile) {

    if (!whole_tile) {
        // add the K-ranges in K order, whichever block arrived last (its own range comes from
        // registers, bit-identical to what it published); all loads of a range are independent
        // (two halves of 16 chunks keep the register count below the limit)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            float4 sum[16];
#pragma unroll
            for (int c = 0; c < 16; ++c) sum[c] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < contributors; ++s) {
                const float4 *part = reinterpret_cast<const float4 *>(p.workspace + ((size_t)tile * p.max_contrib + s) * kTileFloats) +
                                     (half * 16) * kThreads + tid;
                const bool own = s == slot;
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const float4 v = own ? out[half * 16 + c] : __ldcg(part + c * kThreads);
                    sum[c].x += v.x; sum[c].y += v.y; sum[c].z += v.z; sum[c].w += v.w;
                }
            }
#pragma unroll
            for (int c = 0; c < 16; ++c) out[half * 16 + c] = sum[c];
        }
    }

    const bool vec_out = (p.N % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.D) & 15u) == 0) &&
                         (p.C == nullptr || (reinterpret_cast<uintptr_t>(p.C) & 15u) == 0);
#pragma unroll
    for (int ip = 0; ip < 8; ++ip)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int m = row_of(ip, h);
#pragma unroll
            for (int jq = 0; jq < 2; ++jq) {
                const int n = col_of(jq);
                if (m >= p.M || n >= p.N) continue;
                const float4 o4 = out[(ip * 2 + h) * 2 + jq];
                const size_t off = (size_t)m * p.N + n;
                if (vec_out) {
                    float4 o = o4;
                    if (p.C) {
                        const float4 c = *reinterpret_cast<const float4 *>(p.C + off);
                        o.x += c.x; o.y += c.y; o.z += c.z; o.w += c.w;
                    }
                    *reinterpret_cast<float4 *>(p.D + off) = o;
                } else {
                    const float v[4] = {o4.x, o4.y, o4.z, o4.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (n + j < p.N) p.D[off + j] = p.C ? v[j] + p.C[off + j] : v[j];
                }
            }
        }
    if (!whole_tile && tid == 0) p.counters[tile] = 0u;  // ready for the next launch
    }  // finish_tile
    }  // segments
}

}  // namespace sgemm2
}  // namespace ko
