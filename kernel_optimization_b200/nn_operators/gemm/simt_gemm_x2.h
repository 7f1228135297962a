// FP32 SGEMM main kernel for sm_100a: 128 x 128 (or 64 x 128) tile, warps of 64 x 64 with 16 x 8 outputs per
// thread, packed FFMA (fma.rn.f32x2), cp.async multi-stage shared-memory pipeline, K split inside the
// block (warp groups) and across blocks (stream-K ranges).
//
// Why this shape.  One FP32 FMA needs two operands from shared memory; with 128-bit shared loads a
// warp spends (TM + TN) shared-memory wavefronts per k for TM*TN FMA instructions, and the SM retires
// four FMA instructions per wavefront slot.  An 8 x 8 thread tile therefore saturates shared memory
// exactly when it saturates the FMA pipe; 16 x 8 leaves 25% slack.  fma.rn.f32x2 performs two
// IEEE-rounded FMAs per instruction.  (Measured alternatives that lost: the same tile with scalar FFMA,
// 43 against 55 TFLOP/s at 4096^3; 16 x 4 per thread with twice the warps, shared-memory bound; A
// stored twice in shared memory so that no register moves are needed to build {b, b} pairs, 43 TFLOP/s;
// 32 x 4 per thread, which halves those moves at the price of three more shared loads per k, 54 TFLOP/s;
// pairing two consecutive k of one output instead of two rows -- even k in the low half, odd k in the high
// half, A as [m][k] and B transposed as [n][k] in shared memory so that both operands arrive as ready pairs
// and no moves are left -- which limits a thread to 8 x 8 outputs, a third more shared-memory data per FMA:
// shared-memory bound, 1024^3 in 68 us against 49.5 us and 4096^3 at 40 TFLOP/s.)
//
// Data path: A[M,K] row-major is copied 4 bytes at a time straight into a TRANSPOSED shared tile
// As[k][m] (cp.async with a source size of 0 zero-fills out-of-range elements, so every M, N, K is
// legal and nothing is read out of bounds -- the reference prefetches past the end,
// nn_operators/gemm/simt_gemm.h:287-292); B[K,N] goes in 16-byte pieces.  kStages tiles are in flight.
//
// Warp groups.  A block is kGroups independent groups of kWarpsM x kWarpsN warps.  Every group has its own
// shared-memory ring and its own named barrier and accumulates a contiguous part of the block's K range
// of the tile; at the end the groups exchange their partial tiles through the (then idle) rings, each
// group finishing the chunks c with c % kGroups == group, summed in K order.  One group of 4 warps
// leaves one warp per scheduler, which exposes every fixed-latency stall (1024 x 1024 output, time per
// 1024 of K on 128 SMs: 49.5 us with one group, 43.8 us with two; the FMA bound is 33.4 us).  Groups
// instead of more blocks per SM because the register file holds only two such blocks, and instead of
// smaller thread tiles because those are shared-memory bound.
//
// Work distribution ("stream-K"): the (tile, K-tile) pairs form one linear sequence of units that is
// cut into `ctas` equal contiguous ranges, one per block.  With ctas == tiles every block owns one
// whole tile; with ctas == tiles * s every tile is cut into s K-slices (classic split-K); any other
// count (e.g. two blocks per SM) gives ranges that may end one tile and begin the next, so that a
// problem with few tiles still keeps every SM busy for the same time.
//
// Accumulation order: one FMA per k in ascending k per output, as in the reference
// (simt_gemm.h:202-222).  A tile computed by one group of one block is bit-identical to that order;
// otherwise each K-range is accumulated that way and the ranges are added in K order -- the groups'
// through shared memory, the blocks' by the block that finishes last (deterministic; no atomics on
// data, no waiting between blocks).
#pragma once

#include "../../common/common.h"

namespace ko {
namespace sgemm2 {

constexpr int BK = 16;
constexpr int kStages = 4;

// A group is kWarpsM x kWarpsN warps of 64 x 64: tile size, threads per group, shared-memory ring of one group
template <int kWarpsM, int kWarpsN>
struct Shape {
    static constexpr int BM = 64 * kWarpsM, BN = 64 * kWarpsN;
    static constexpr int kGroupThreads = 32 * kWarpsM * kWarpsN;
    static constexpr int kStrideA = BM + 4;  // = 4 mod 32: (4*k + m) mod 32 distinct for k < 8, m < 4 -> conflict-free transposed writes
    static constexpr int kStageFloats = BK * kStrideA + BK * BN;
    static constexpr int kRingFloats = kStages * kStageFloats;
    static constexpr int kTileFloats = BM * BN;
    static constexpr int smem_bytes(int groups) { return groups * kRingFloats * (int)sizeof(float); }
};

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
// unconditional forms for tiles that lie inside the matrices
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
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
    int ws_per_block;   // 0: workspace is [tiles][max_contrib] partial tiles; 1: [ctas][2] (see partial_index)
    float *workspace;   // partial tiles of BM*BN floats (used when a tile is shared)
    unsigned *counters; // one arrival counter per tile, zero between launches
};

// the block whose unit range [b*U/G, (b+1)*U/G) contains unit u
__device__ __forceinline__ int block_of_unit(long long u, long long U, int G) {
    int b = (int)(u * G / U);
    while ((long long)(b + 1) * U / G <= u) ++b;
    while ((long long)b * U / G > u) --b;
    return b;
}

// Where contributor number `s` (block first_block + s) of `tile` keeps its partial tile.  Per tile:
// slot s of the tile.  Per block: a block shares at most two tiles with others -- the one its range
// begins in (it is not that tile's first contributor: slot 0) and the one its range ends in (it is
// that tile's first contributor: slot 1) -- so two slots per block suffice whatever the tile count.
__device__ __forceinline__ size_t partial_index(const Params &p, int tile, int first_block, int s) {
    return p.ws_per_block ? (size_t)(first_block + s) * 2 + (s == 0 ? 1 : 0) : (size_t)tile * p.max_contrib + s;
}

template <int kGroups, int kGroupThreads>
__device__ __forceinline__ void group_sync(int group) {
    if (kGroups == 1) __syncthreads();
    else asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "n"(kGroupThreads) : "memory");
}

// out[j * kGroups + group] with compile-time j: selects instead of a dynamically indexed register array
template <int kGroups>
__device__ __forceinline__ float4 own_chunk(const float4 (&out)[32], int j, int group) {
    float4 r = out[j * kGroups];
#pragma unroll
    for (int h = 1; h < kGroups; ++h)
        if (group == h) r = out[j * kGroups + h];
    return r;
}

// kVecB: N % 4 == 0 and B 16-byte aligned (16-byte copies of B); otherwise 4-byte copies.
// kWarpsM x kWarpsN: warps of a group (2 x 2 -> 128 x 128 tile; 1 x 2 -> 64 x 128).
// kGroups: warp groups per block (1, 2 or 4), each with a contiguous part of the block's K range.
template <bool kVecB, int kWarpsM, int kWarpsN, int kGroups>
__global__ void __launch_bounds__(32 * kWarpsM * kWarpsN * kGroups) sgemm_x2_kernel(const Params p) {
    using S = Shape<kWarpsM, kWarpsN>;
    constexpr int BM = S::BM, BN = S::BN, GT = S::kGroupThreads, kStageFloats = S::kStageFloats, kStrideA = S::kStrideA;
    static_assert(kGroups == 1 || kGroups == 2 || kGroups == 4, "chunks are dealt round-robin to the groups");
    static_assert(32 * GT * 4 <= S::kRingFloats, "a ring must hold the chunks a group hands over");
    extern __shared__ __align__(16) float smem_all[];
    __shared__ int s_is_last;
    const int group = kGroups == 1 ? 0 : (int)threadIdx.x / GT;
    const int tid = (int)threadIdx.x % GT, lane = tid & 31, warp = tid >> 5;
    float *smem = smem_all + group * S::kRingFloats;  // this group's ring
    const int warp_m = warp / kWarpsN, warp_n = warp % kWarpsN;  // kWarpsM x kWarpsN warps of 64 x 64
    const int lane_m = lane >> 3, lane_n = lane & 7;             // 4 x 8 lanes of 16 x 8
    const int tiles_n = (p.N + BN - 1) / BN;
    const int ktiles_total = (p.K + BK - 1) / BK;
    const long long units = (long long)((p.M + BM - 1) / BM) * tiles_n * ktiles_total;
    const long long unit_begin = units * blockIdx.x / p.ctas, unit_end = units * (blockIdx.x + 1) / p.ctas;

    // launched with programmatic stream serialization: this block may have been placed while the stream's
    // previous kernel was draining; nothing global is touched before that kernel's writes are visible
    grid_launch_dependents();
    grid_dependency_wait();
    const uint32_t smem_base = smem_u32(smem);
    int m_base = 0, n_base = 0;
    bool inner_mn = false;  // the tile lies inside M and N: K-tiles inside K need no bounds checks
    auto issue_tile = [&](int kt, int stage) {
        const int k0 = kt * BK;
        const uint32_t as = smem_base + (uint32_t)stage * kStageFloats * 4u;
        const uint32_t bs = as + BK * kStrideA * 4u;
        if (inner_mn && k0 + BK <= p.K) {
            // same element-to-thread mapping as below, addresses by pointer steps, no predicates
            constexpr int kRowsPerCopy = GT / 8, kCopiesPerHalf = BM / kRowsPerCopy;
            const int mt = tid >> 3, kl = tid & 7;
            const float *a_src = p.A + (size_t)(m_base + mt) * p.K + (k0 + kl);
            const size_t a_step = (size_t)kRowsPerCopy * p.K;
            const uint32_t a_dst = as + (uint32_t)(kl * kStrideA + mt) * 4u;
#pragma unroll
            for (int i = 0; i < kCopiesPerHalf; ++i) {
                cp_async_4(a_dst + (uint32_t)(i * kRowsPerCopy) * 4u, a_src + i * a_step);
                cp_async_4(a_dst + (uint32_t)(8 * kStrideA + i * kRowsPerCopy) * 4u, a_src + i * a_step + 8);
            }
            if (kVecB) {
                constexpr int kVecsPerRow = BN / 4, kRowsPerStep = GT / kVecsPerRow;
                const int kb = tid / kVecsPerRow, nb = (tid % kVecsPerRow) * 4;
                const float *b_src = p.B + (size_t)(k0 + kb) * p.N + (n_base + nb);
                const size_t b_step = (size_t)kRowsPerStep * p.N;
                const uint32_t b_dst = bs + (uint32_t)(kb * BN + nb) * 4u;
#pragma unroll
                for (int i = 0; i < BK / kRowsPerStep; ++i) cp_async_16(b_dst + (uint32_t)(i * kRowsPerStep * BN) * 4u, b_src + i * b_step);
                return;
            }
            // B by 4-byte copies: fall through to the checked loop for B only
#pragma unroll
            for (int i = 0; i < (BK * BN) / GT; ++i) {
                const int e = tid + i * GT;
                const int k = e / BN, n = e % BN;
                cp_async_4(bs + (uint32_t)(k * BN + n) * 4u, p.B + (size_t)(k0 + k) * p.N + (n_base + n));
            }
            return;
        }
        // A: a warp instruction covers 4 rows x 8 consecutive k (4 full 32-byte sectors)
#pragma unroll
        for (int i = 0; i < (BM * BK) / GT; ++i) {
            const int e = tid + i * GT;  // 0 .. BM*BK-1: 8 consecutive k, then the rows, then the k half
            const int k = (e & 7) + 8 * ((e >> 3) / BM);
            const int m = (e >> 3) % BM;
            const int gm = m_base + m, gk = k0 + k;
            const bool ok = gm < p.M && gk < p.K;
            cp_async_4(as + (uint32_t)(k * kStrideA + m) * 4u, p.A + (ok ? (size_t)gm * p.K + gk : 0), ok);
        }
        if (kVecB) {
#pragma unroll
            for (int i = 0; i < (BK * BN / 4) / GT; ++i) {
                const int e = tid + i * GT;
                const int k = e / (BN / 4), n = (e % (BN / 4)) * 4;
                const int gk = k0 + k, gn = n_base + n;
                const bool ok = gk < p.K && gn < p.N;
                cp_async_16(bs + (uint32_t)(k * BN + n) * 4u, p.B + (ok ? (size_t)gk * p.N + gn : 0), ok);
            }
        } else {
#pragma unroll
            for (int i = 0; i < (BK * BN) / GT; ++i) {
                const int e = tid + i * GT;
                const int k = e / BN, n = e % BN;
                const int gk = k0 + k, gn = n_base + n;
                const bool ok = gk < p.K && gn < p.N;
                cp_async_4(bs + (uint32_t)(k * BN + n) * 4u, p.B + (ok ? (size_t)gk * p.N + gn : 0), ok);
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
    const int seg_ktiles = kt_end - kt_begin;
    u += seg_ktiles;
    const bool whole_tile = seg_ktiles == ktiles_total;
    m_base = (tile / tiles_n) * BM;
    n_base = (tile % tiles_n) * BN;
    inner_mn = m_base + BM <= p.M && n_base + BN <= p.N;
    // this group's contiguous part of the segment
    const int kt_first = kt_begin + seg_ktiles * group / kGroups;
    const int ktiles = kt_begin + seg_ktiles * (group + 1) / kGroups - kt_first;
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
        if (s < ktiles) issue_tile(kt_first + s, s);
        cp_async_commit();
    }

    for (int t = 0; t < ktiles; ++t) {
        cp_async_wait<kStages - 2>();
        group_sync<kGroups, GT>(group);  // tile t has landed for the whole group; the stage refilled below was consumed at t-1
        if (t + kStages - 1 < ktiles) issue_tile(kt_first + t + kStages - 1, (t + kStages - 1) % kStages);
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
            for (int q = 0; q < 2; ++q) b4[q] = *reinterpret_cast<const float4 *>(bs + kk * BN + q * 32);
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

    // The thread's 32 float4 chunks: chunk c = row_index * 2 + jq with row_index = 2*ip + h,
    // row(c) = m_base + a_off + (row_index/4)*16 + row_index%4, columns n_base + b_off + jq*32 + 0..3.
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

    // Group g finishes the chunks c = j * kGroups + g (j < kFin): it hands the other chunks to their
    // owners through its own ring, and adds the K parts of its chunks in group (= K) order.  All threads
    // of the block then run the rest of the epilogue.  fin[j] is chunk j * kGroups + group.
    constexpr int kFin = 32 / kGroups;
    float4 fin[kFin];
    if (kGroups > 1) {
        float4 *ring = reinterpret_cast<float4 *>(smem);
        group_sync<kGroups, GT>(group);  // every warp of the group has finished reading the ring
#pragma unroll
        for (int c = 0; c < 32; ++c)
            if (c % kGroups != group) ring[c * GT + tid] = out[c];
        __syncthreads();
#pragma unroll
        for (int j = 0; j < kFin; ++j) {
            const float4 mine = own_chunk<kGroups>(out, j, group);
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int h = 0; h < kGroups; ++h) {
                const float4 *theirs = reinterpret_cast<const float4 *>(smem_all + h * S::kRingFloats);
                const float4 v = h == group ? mine : theirs[(j * kGroups + group) * GT + tid];
                if (h == 0) sum = v;
                else { sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w; }
            }
            fin[j] = sum;
        }
    } else {
#pragma unroll
        for (int j = 0; j < kFin; ++j) fin[j] = out[j];
    }

    int contributors = 1, slot = 0, first_block = 0;
    if (!whole_tile) {
        const long long first_unit = (long long)tile * ktiles_total;
        first_block = block_of_unit(first_unit, units, p.ctas);
        contributors = block_of_unit(first_unit + ktiles_total - 1, units, p.ctas) - first_block + 1;
        slot = (int)blockIdx.x - first_block;
    }
    bool finish_tile = true;
    if (!whole_tile) {
        // publish this K-range's partial tile: [chunk][thread of the group] float4, coalesced
        float4 *mine = reinterpret_cast<float4 *>(p.workspace + partial_index(p, tile, first_block, slot) * S::kTileFloats) +
                       group * GT + tid;
#pragma unroll
        for (int j = 0; j < kFin; ++j) mine[j * kGroups * GT] = fin[j];
        __syncthreads();
        if (threadIdx.x == 0) {
            // the barrier ordered the block's stores before this fence, which publishes them (fences are cumulative)
            __threadfence();
            const unsigned prev = atomicAdd(p.counters + tile, 1u);
            s_is_last = (prev == (unsigned)contributors - 1u);
            __threadfence();
        }
        __syncthreads();
        finish_tile = s_is_last != 0;
    }
    if (finish_tile) {
        if (!whole_tile) {
            // add the K-ranges in K order, whichever block arrived last (its own range comes from
            // registers, bit-identical to what it published); all loads of a range are independent
            // (at most 16 chunks at a time keep the register count below the limit)
            constexpr int kPart = kFin < 16 ? kFin : 16;
#pragma unroll
            for (int part = 0; part < kFin / kPart; ++part) {
                float4 sum[kPart];
#pragma unroll
                for (int c = 0; c < kPart; ++c) sum[c] = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int s = 0; s < contributors; ++s) {
                    const float4 *theirs =
                        reinterpret_cast<const float4 *>(p.workspace + partial_index(p, tile, first_block, s) * S::kTileFloats) +
                        (size_t)(part * kPart) * kGroups * GT + group * GT + tid;
                    const bool own = s == slot;
#pragma unroll
                    for (int c = 0; c < kPart; ++c) {
                        const float4 v = own ? fin[part * kPart + c] : __ldcg(theirs + c * kGroups * GT);
                        sum[c].x += v.x; sum[c].y += v.y; sum[c].z += v.z; sum[c].w += v.w;
                    }
                }
#pragma unroll
                for (int c = 0; c < kPart; ++c) fin[part * kPart + c] = sum[c];
            }
        }

        const bool vec_out = (p.N % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.D) & 15u) == 0) &&
                             (p.C == nullptr || (reinterpret_cast<uintptr_t>(p.C) & 15u) == 0);
#pragma unroll
        for (int j = 0; j < kFin; ++j) {
            const int c = j * kGroups + group;
            const int ri = c >> 1, jq = c & 1;
            const int m = m_base + a_off + (ri >> 2) * 16 + (ri & 3);
            const int n = n_base + b_off + jq * 32;
            if (m >= p.M || n >= p.N) continue;
            const float4 o4 = fin[j];
            const size_t off = (size_t)m * p.N + n;
            if (vec_out) {
                float4 o = o4;
                if (p.C) {
                    const float4 cv = *reinterpret_cast<const float4 *>(p.C + off);
                    o.x += cv.x; o.y += cv.y; o.z += cv.z; o.w += cv.w;
                }
                *reinterpret_cast<float4 *>(p.D + off) = o;
            } else {
                const float v[4] = {o4.x, o4.y, o4.z, o4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (n + e < p.N) p.D[off + e] = p.C ? v[e] + p.C[off + e] : v[e];
            }
        }
        if (!whole_tile && threadIdx.x == 0) p.counters[tile] = 0u;  // ready for the next launch
    }  // finish_tile
    }  // segments
}

}  // namespace sgemm2
}  // namespace ko
