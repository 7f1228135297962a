// Row softmax over the last dimension for sm_100a.
//
// Tiers, chosen by row length, row count and alignment (the reference's warp / block-cached /
// block-no-cache split, nn_operators/softmax/softmax.h:11-60, :62-113, :116-166, re-thought for B200):
//
//   staged tier persistent blocks; a producer warp streams chunks of whole rows into a shared-memory
//               ring with 1-D bulk copies (TMA) and consumer warps run the row math out of shared
//               memory (common/row_pipeline.h).  Bytes in flight are set by the ring, not by occupancy.
//   warp tier   one warp owns a few consecutive rows per step; a row sits in the registers of a group
//               of 8, 16 or 32 lanes as kVecs 128-bit vectors per lane (short rows share a warp);
//               every load of the step is issued before the first use.
//   block tier  one thread block per row, the row in registers (kVecs vectors per thread), warp
//               all-reduce + one shared-memory exchange per statistic.
//   prefetching block tier  the block tier with the block's next row landing in shared memory (bulk copy)
//               while the current one is reduced: 16385..32768 columns, one block per SM.
//   cluster tier one row per thread-block cluster (2, 4 or 8 blocks), each block a slice of the row in
//               registers, (max, sum) partials exchanged through distributed shared memory: few very long rows.
//   reread tier rows beyond one block's registers: one row per block in two passes (online max / sum, then the
//               row again from the L2); for rows up to 256 KB every load goes through a per-thread
//               shared-memory ring of (row, pass, chunk) items.
//   stream tier one thread block per row, three passes over global memory with scalar accesses; any
//               column count and any alignment (correctness path).
//
// All tiers compute exp(x - rowmax) / sum in FP32 as 2^(fma(x, log2 e, -fl(rowmax * log2 e))) on the
// special-function unit; a row's results do not depend on the tier's launch geometry.  The rounding of
// the shift is common to the whole row and cancels in the quotient; it is half an ulp of rowmax * log2 e,
// negligible against the exponent range for |x| < 1e9 (the stated input range).  (The reference's Subtract
// functor adds, common/functors.h:168, so it evaluates exp(x + rowmax); the two agree mathematically
// but the reference overflows once 2*rowmax > 88.7.)
//
// The reference's class templates SoftMaxWarpImpl / SoftMaxBlockImpl / SoftMaxBlockNoCacheImpl and
// the softmax<Kernel> __global__ wrapper keep their names, template parameters and static members,
// so `softmax<SoftMaxWarpImpl<float, 4, R, C>><<<grid, block, smem, stream>>>(in, out)` still
// compiles; those tiers are grid-stride loops and therefore correct for any launch geometry.
#pragma once

#include <cooperative_groups.h>

#include "../../common/common.h"
#include "../../common/functors.h"
#include "../../common/row_pipeline.h"

namespace ko {

constexpr float kNegInf = -__builtin_huge_valf();
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float max4(const float4 &v) { return fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)); }
__device__ __forceinline__ float4 neg_inf4() { return make_float4(kNegInf, kNegInf, kNegInf, kNegInf); }

// e^(x - m) for the four lanes of v, as 2^(x*log2e - m*log2e); returns their sum
__device__ __forceinline__ float exp_shifted4(float4 &v, float neg_m_log2e) {
    v.x = exp2_approx(fmaf(v.x, kLog2e, neg_m_log2e));
    v.y = exp2_approx(fmaf(v.y, kLog2e, neg_m_log2e));
    v.z = exp2_approx(fmaf(v.z, kLog2e, neg_m_log2e));
    v.w = exp2_approx(fmaf(v.w, kLog2e, neg_m_log2e));
    return (v.x + v.y) + (v.z + v.w);
}
__device__ __forceinline__ void scale4(float4 &v, float s) { v.x *= s; v.y *= s; v.z *= s; v.w *= s; }

// A row is spread over a group of G lanes (G = 8, 16 or 32), kVecs 128-bit vectors per lane, so a warp
// works on 32/G rows at once ("a slot") and short rows do not pay for 32-lane reductions.  G depends
// only on the column count, so a row's arithmetic is the same in every tier and launch geometry.
template <int G>
__device__ __forceinline__ float group_allreduce_max(float v) {
    if constexpr (G == 32) {
        return warp_redux_max(v);
    } else {
#pragma unroll
        for (int m = G / 2; m > 0; m >>= 1) v = fmaxf(v, __shfl_xor_sync(kFullMask, v, m));
        return v;
    }
}
template <int G>
__device__ __forceinline__ float group_allreduce_sum(float v) {
#pragma unroll
    for (int m = G / 2; m > 0; m >>= 1) v += __shfl_xor_sync(kFullMask, v, m);
    return v;
}

// kSlots independent slots, each holding one row per lane group (padding = -inf): in place to
// probabilities.  The independent chains are what hides the shuffle latency.
template <int kVecs, int kSlots, int G>
__device__ __forceinline__ void softmax_rows_in_registers(float4 (&x)[kSlots][kVecs]) {
    float mx[kSlots], sum[kSlots];
#pragma unroll
    for (int r = 0; r < kSlots; ++r) {
        float m = max4(x[r][0]);
#pragma unroll
        for (int j = 1; j < kVecs; ++j) m = fmaxf(m, max4(x[r][j]));
        mx[r] = m;
    }
#pragma unroll
    for (int r = 0; r < kSlots; ++r) mx[r] = group_allreduce_max<G>(mx[r]);
#pragma unroll
    for (int r = 0; r < kSlots; ++r) {
        const float neg = -mx[r] * kLog2e;
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < kVecs; ++j) s += exp_shifted4(x[r][j], neg);
        sum[r] = s;
    }
#pragma unroll
    for (int r = 0; r < kSlots; ++r) sum[r] = group_allreduce_sum<G>(sum[r]);
#pragma unroll
    for (int r = 0; r < kSlots; ++r) {
        const float inv = rcp_approx(sum[r]);
#pragma unroll
        for (int j = 0; j < kVecs; ++j) scale4(x[r][j], inv);
    }
}

// Loads/stores of a warp's kSlots * (32/G) consecutive rows starting at `base` (a row-major array of
// float4 with nvec vectors per row); rows >= nrows are padded / skipped.
template <int kVecs, int kSlots, int G, typename Load>
__device__ __forceinline__ void softmax_load_rows(float4 (&x)[kSlots][kVecs], int lane, int nvec, long long nrows,
                                                  Load &&load) {
    constexpr int kRowsPerSlot = 32 / G;
    const int sub = lane / G, gl = lane % G;
#pragma unroll
    for (int r = 0; r < kSlots; ++r) {
        const long long row = r * kRowsPerSlot + sub;
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            const int v = gl + G * j;
            x[r][j] = (row < nrows && v < nvec) ? load(row, v) : neg_inf4();
        }
    }
}
template <int kVecs, int kSlots, int G>
__device__ __forceinline__ void softmax_store_rows(const float4 (&x)[kSlots][kVecs], int lane, int nvec, long long nrows,
                                                   float4 *out_rows) {
    constexpr int kRowsPerSlot = 32 / G;
    const int sub = lane / G, gl = lane % G;
#pragma unroll
    for (int r = 0; r < kSlots; ++r) {
        const long long row = r * kRowsPerSlot + sub;
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            const int v = gl + G * j;
            if (row < nrows && v < nvec) st_stream(out_rows + row * nvec + v, x[r][j]);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// warp tier
// ---------------------------------------------------------------------------------------------
template <int kVecs, int kSlots, int G>
__device__ __forceinline__ void softmax_warp_tier(const float *in, float *out, long long rows, int cols) {
    constexpr int kRowsPerStep = kSlots * (32 / G);
    const int lane = threadIdx.x & 31;
    const int nvec = cols >> 2;  // 128-bit vectors per row
    const long long warps_per_grid = (long long)gridDim.x * (blockDim.x >> 5);
    const long long warp_global = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const float4 *in4 = reinterpret_cast<const float4 *>(in);
    float4 *out4 = reinterpret_cast<float4 *>(out);

    for (long long row0 = warp_global * kRowsPerStep; row0 < rows; row0 += warps_per_grid * kRowsPerStep) {
        float4 x[kSlots][kVecs];
        const float4 *src = in4 + row0 * nvec;
        softmax_load_rows<kVecs, kSlots, G>(x, lane, nvec, rows - row0,
                                            [&](long long row, int v) { return ld_stream(src + row * nvec + v); });
        softmax_rows_in_registers<kVecs, kSlots, G>(x);
        softmax_store_rows<kVecs, kSlots, G>(x, lane, nvec, rows - row0, out4 + row0 * nvec);
    }
}

// ---------------------------------------------------------------------------------------------
// staged tier: consumer side of the row pipeline
// ---------------------------------------------------------------------------------------------
template <int kVecs, int kSlots, int G, int kConsumerWarps>
__device__ __forceinline__ void softmax_staged_tier(const float *in, float *out, long long rows, int cols,
                                                    const RowPipeGeometry geo, uint8_t *smem, unsigned *status) {
    constexpr int kRowsPerStep = kSlots * (32 / G);
    const int nvec = cols >> 2;
    float4 *out4 = reinterpret_cast<float4 *>(out);
    row_pipeline<kConsumerWarps>(in, rows, geo, smem, status,
        [&](const uint8_t *stage, long long first_row, int n, int it, int cw, int lane) {
            const float4 *stage4 = reinterpret_cast<const float4 *>(stage);
            const int full_groups = (geo.rows_per_stage + kRowsPerStep - 1) / kRowsPerStep;
            const int groups = (n + kRowsPerStep - 1) / kRowsPerStep;
            for (int g = first_group_of_warp(it, full_groups, cw, kConsumerWarps); g < groups; g += kConsumerWarps) {
                const int r0 = g * kRowsPerStep;
                float4 x[kSlots][kVecs];
                const float4 *src = stage4 + (size_t)r0 * nvec;
                softmax_load_rows<kVecs, kSlots, G>(x, lane, nvec, n - r0,
                                                    [&](long long row, int v) { return src[row * nvec + v]; });
                softmax_rows_in_registers<kVecs, kSlots, G>(x);
                softmax_store_rows<kVecs, kSlots, G>(x, lane, nvec, n - r0, out4 + (first_row + r0) * nvec);
            }
        });
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
            x[j] = v < nvec ? ld_stream(in4 + row * nvec + v) : neg_inf4();
            m = fmaxf(m, max4(x[j]));
        }
        m = block_allreduce<true>(m, s_exchange);
        const float neg = -m * kLog2e;
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < kVecs; ++j) s += exp_shifted4(x[j], neg);
        s = block_allreduce<false>(s, s_exchange);
        const float inv = rcp_approx(s);
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            const int v = threadIdx.x + blockDim.x * j;
            if (v < nvec) {
                scale4(x[j], inv);
                st_stream(out4 + row * nvec + v, x[j]);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// prefetching block tier: one row per block in registers, the block's NEXT row landing in shared memory
// ---------------------------------------------------------------------------------------------
// A block that holds a long row in registers has nothing in flight while it reduces, and with 1024 threads
// there is one block per SM, so nobody else covers for it: the plain block tier moves 4.4 TB/s at 32768
// columns.  Here warp 0 starts a 1-D bulk copy (TMA) of the block's next row into a shared-memory row buffer as
// soon as the current row has been lifted from that buffer into registers; the copy runs under the reductions,
// the exponentials and the stores of the current row.  One mbarrier counts the bytes; the wait is bounded.
template <int kVecs, int kThreads>
__device__ __forceinline__ void softmax_block_prefetch_tier(const float *in, float *out, long long rows, int cols, float4 *row_buf,
                                                            uint64_t *bar_word, float *s_exchange, unsigned *status) {
    const int nvec = cols >> 2;
    const uint32_t row_bytes = (uint32_t)cols * 4u;
    const uint32_t buf = smem_u32(row_buf), bar = smem_u32(bar_word);
    float4 *out4 = reinterpret_cast<float4 *>(out);
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        fence_barrier_init();
        fence_proxy_async();
    }
    __syncthreads();
    long long row = blockIdx.x;
    if (row < rows && threadIdx.x < 32) prefetch_row(in + row * cols, row_bytes, buf, bar);
    volatile int never_aborted = 0;
    uint32_t parity = 0;
    for (; row < rows; row += gridDim.x, parity ^= 1u) {
        const bool landed = mbar_wait(bar, parity, &never_aborted);
        if (!__syncthreads_and(landed)) {  // the whole block leaves together
            if (threadIdx.x == 0) atomicCAS(status, 0u, kRowPrefetchTimeout);
            break;
        }
        float4 x[kVecs];
        float m = kNegInf;
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            const int v = threadIdx.x + kThreads * j;
            x[j] = v < nvec ? row_buf[v] : neg_inf4();
            m = fmaxf(m, max4(x[j]));
        }
        __syncthreads();  // the buffer has been read by everyone: it may be refilled
        const long long next = row + gridDim.x;
        if (next < rows && threadIdx.x < 32) prefetch_row(in + next * cols, row_bytes, buf, bar);
        m = block_allreduce<true>(m, s_exchange);
        const float neg = -m * kLog2e;
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < kVecs; ++j) s += exp_shifted4(x[j], neg);
        s = block_allreduce<false>(s, s_exchange);
        const float inv = rcp_approx(s);
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            const int v = threadIdx.x + kThreads * j;
            if (v < nvec) {
                scale4(x[j], inv);
                st_stream(out4 + row * nvec + v, x[j]);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// cluster tier: one row per thread-block CLUSTER, the row in the registers of all its blocks
// ---------------------------------------------------------------------------------------------
// For rows beyond one block's registers (more than 32768 columns) or few very long rows: each of the
// cluster's blocks holds a contiguous slice of the row, block-level (max, sum) partials are exchanged
// through distributed shared memory (every block reads its peers' partials with plain loads from
// their shared memory), so the row is still read from HBM exactly once.  One exchange per row: each block
// reduces its slice against its own maximum (online softmax) and the blocks trade (max, sum) pairs; the
// exchange slots are double buffered by row parity so no second synchronisation is needed.
// kPrefetch: the block's slice of the cluster's NEXT row is brought into a shared-memory buffer by a bulk copy while
// the current row is reduced, exchanged and stored (see the prefetching block tier); row_buf / bar_word / status are
// used only then.
// Partial (max, sum) exchange without cluster-wide barriers: every block pushes its value into each peer's mailbox
// (a plain store into the peer's shared memory) and arrives on that peer's mbarrier; a block waits only for its own
// mailbox to fill.  value[parity][kind][rank] (kind 0 = block maximum, 1 = block sum against that maximum), one
// mbarrier per parity expecting one arrival per block (bar[parity][0]; bar[parity][1] is unused); row parity
// double-buffers the slots -- a peer can be at most one exchange ahead, because every exchange needs
// everybody's arrival.  A cluster barrier costs about 1.3 us per row and use here, this about a third of it.
struct ClusterMailbox {
    uint64_t bar[2][2];
    float value[2][2][8];
};

template <int kVecs, bool kPrefetch>
__device__ __forceinline__ void softmax_cluster_tier(const float *in, float *out, long long rows, int cols,
                                                     float *s_exchange, float (*s_part)[2], float4 *row_buf = nullptr,
                                                     uint64_t *bar_word = nullptr, unsigned *status = nullptr,
                                                     ClusterMailbox *mail = nullptr) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned nblocks = cluster.num_blocks(), rank = cluster.block_rank();
    const int nvec = cols >> 2;
    const int slice = (nvec + (int)nblocks - 1) / (int)nblocks;
    const int v_begin = (int)rank * slice, v_end = min(nvec, v_begin + slice);
    const float4 *in4 = reinterpret_cast<const float4 *>(in);
    float4 *out4 = reinterpret_cast<float4 *>(out);
    const long long clusters = gridDim.x / nblocks, first = blockIdx.x / nblocks;
    const uint32_t slice_bytes = v_end > v_begin ? (uint32_t)(v_end - v_begin) * 16u : 0u;
    const uint32_t buf = kPrefetch ? smem_u32(row_buf) : 0u, bar = kPrefetch ? smem_u32(bar_word) : 0u;
    if (kPrefetch) {
        if (threadIdx.x == 0) {
            mbar_init(bar, 1);
            fence_barrier_init();
            fence_proxy_async();
        }
        __syncthreads();
        if (first < rows && slice_bytes && threadIdx.x < 32)
            prefetch_row(reinterpret_cast<const float *>(in4 + first * nvec + v_begin), slice_bytes, buf, bar);
    }
    if (mail) {
        if (threadIdx.x == 0) {
            for (int q = 0; q < 4; ++q) mbar_init(smem_u32(&mail->bar[q >> 1][q & 1]), nblocks);
            fence_barrier_init();
        }
        cluster.sync();  // every mailbox is ready before anybody pushes into it
    }
    // Every block pushes its (max, sum) pair into each peer's mailbox and arrives once on that peer's mbarrier;
    // returns once every block's pair has arrived here.  The result is made block-uniform (one thread of a block
    // could otherwise see the last poll succeed and another see it fail).
    auto exchange = [&](int par, float m_block, float s_block, uint32_t phase) -> bool {
        if (threadIdx.x < nblocks) {
            const uint32_t peer = threadIdx.x;
            st_cluster_f32(map_to_cluster_rank(smem_u32(&mail->value[par][0][rank]), peer), m_block);
            st_cluster_f32(map_to_cluster_rank(smem_u32(&mail->value[par][1][rank]), peer), s_block);
            mbar_arrive_cluster(map_to_cluster_rank(smem_u32(&mail->bar[par][0]), peer));
        }
        return __syncthreads_and(mbar_wait_cluster(smem_u32(&mail->bar[par][0]), phase)) != 0;
    };
    volatile int never_aborted = 0;
    uint32_t landed_parity = 0;
    bool gave_up = false;  // block-uniform by construction
    int parity = 0;
    uint32_t use = 0;  // rows done by this cluster: the mailbox of a parity is on its (use / 2)-th phase
    for (long long row = first; row < rows; row += clusters, parity ^= 1, ++use) {
        float4 x[kVecs];
        float m = kNegInf;
        if (kPrefetch) {
            // a block that gives up still takes part in every exchange below (its peers must not hang):
            // it works on padding from here on and the status word reports the call as failed
            if (slice_bytes && !gave_up) {
                const bool landed = mbar_wait(bar, landed_parity, &never_aborted);
                landed_parity ^= 1u;
                if (!__syncthreads_and(landed)) {
                    if (threadIdx.x == 0) atomicCAS(status, 0u, kRowPrefetchTimeout);
                    gave_up = true;
                }
            }
#pragma unroll
            for (int j = 0; j < kVecs; ++j) {
                const int v = v_begin + (int)threadIdx.x + (int)blockDim.x * j;
                x[j] = (v < v_end && !gave_up) ? row_buf[v - v_begin] : neg_inf4();
                m = fmaxf(m, max4(x[j]));
            }
            __syncthreads();  // the buffer has been read by everyone: it may be refilled
            const long long next = row + clusters;
            if (next < rows && slice_bytes && !gave_up && threadIdx.x < 32)
                prefetch_row(reinterpret_cast<const float *>(in4 + next * nvec + v_begin), slice_bytes, buf, bar);
        } else {
#pragma unroll
            for (int j = 0; j < kVecs; ++j) {
                const int v = v_begin + (int)threadIdx.x + (int)blockDim.x * j;
                x[j] = v < v_end ? ld_stream(in4 + row * nvec + v) : neg_inf4();
                m = fmaxf(m, max4(x[j]));
            }
        }
        // Online form: the block normalises its slice against its OWN maximum first, so that a single exchange of
        // (max, sum) pairs is enough; the row's sum is sum_r s_r * 2^((m_r - m) log2 e), added in rank order.
        m = block_allreduce<true>(m, s_exchange);
        const float neg_block = m == kNegInf ? 0.f : -m * kLog2e;  // an empty or fully masked slice contributes 2^(-inf) = 0
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < kVecs; ++j) s += exp_shifted4(x[j], neg_block);
        s = block_allreduce<false>(s, s_exchange);
        float row_max = kNegInf, total = 0.f;
        if (mail) {
            if (!exchange(parity, m, s, (use >> 1) & 1u) && !gave_up) {
                if (threadIdx.x == 0) atomicCAS(status, 0u, kRowPrefetchTimeout);
                gave_up = true;  // keeps pushing (the peers wait for it) but writes nothing
            }
            for (unsigned r = 0; r < nblocks; ++r) row_max = fmaxf(row_max, mail->value[parity][0][r]);
            for (unsigned r = 0; r < nblocks; ++r)
                total = fmaf(mail->value[parity][1][r], exp2_approx((mail->value[parity][0][r] - row_max) * kLog2e), total);
        } else {
            if (threadIdx.x == 0) {
                s_part[parity][0] = m;
                s_part[parity][1] = s;
            }
            cluster.sync();
            for (unsigned r = 0; r < nblocks; ++r) row_max = fmaxf(row_max, cluster.map_shared_rank(&s_part[parity][0], r)[0]);
            for (unsigned r = 0; r < nblocks; ++r) {
                const float *peer = cluster.map_shared_rank(&s_part[parity][0], r);
                total = fmaf(peer[1], exp2_approx((peer[0] - row_max) * kLog2e), total);
            }
        }
        const float scale = exp2_approx((m - row_max) * kLog2e) * rcp_approx(total);
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            const int v = v_begin + (int)threadIdx.x + (int)blockDim.x * j;
            if (v < v_end && !gave_up) {
                scale4(x[j], scale);
                st_stream(out4 + row * nvec + v, x[j]);
            }
        }
    }
    cluster.sync();  // no block may exit while a peer can still read its shared memory
}

// ---------------------------------------------------------------------------------------------
// reread tier: one row per thread block, two passes, the second one served by the L2
// ---------------------------------------------------------------------------------------------
// For rows longer than one block's registers when there are enough rows to fill every SM several times: pass 1
// streams the row once and keeps only a running (max, sum) pair per thread (online softmax: the sum is rescaled when the
// maximum grows), marking the lines evict-last; pass 2 reads the row again -- from the L2, as long as the rows in
// flight (one per block) fit there -- and writes the result.  HBM sees the row once in each direction, no block waits
// for another, and blocks drift apart so that some are in their read-only pass while others write.
template <int kUnroll>
__device__ __forceinline__ void softmax_reread_tier(const float *in, float *out, long long rows, int cols, float *s_exchange) {
    const int nvec = cols >> 2;
    const int step = (int)blockDim.x * kUnroll;
    const uint64_t keep = l2_keep_policy();
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const float4 *x4 = reinterpret_cast<const float4 *>(in) + row * nvec;
        float4 *y4 = reinterpret_cast<float4 *>(out) + row * nvec;
        float m = kNegInf, s = 0.f;
        for (int base = 0; base < nvec; base += step) {
            float4 x[kUnroll];
            float cm = kNegInf;
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                const int v = base + (int)threadIdx.x + (int)blockDim.x * j;
                x[j] = v < nvec ? ld_keep(x4 + v, keep) : neg_inf4();
                cm = fmaxf(cm, max4(x[j]));
            }
            const float grown = fmaxf(m, cm);
            if (grown != kNegInf) {  // a chunk of nothing but -inf adds nothing
                const float neg = -grown * kLog2e;
                float cs = 0.f;
#pragma unroll
                for (int j = 0; j < kUnroll; ++j) cs += exp_shifted4(x[j], neg);
                s = fmaf(s, exp2_approx(fmaf(m, kLog2e, neg)), cs);  // m = -inf: 2^(-inf) = 0 and s is still 0
                m = grown;
            }
        }
        const float row_max = block_allreduce<true>(m, s_exchange);
        const float neg = -row_max * kLog2e;
        s = m == kNegInf ? 0.f : s * exp2_approx(fmaf(m, kLog2e, neg));
        const float inv = rcp_approx(block_allreduce<false>(s, s_exchange));
        for (int base = 0; base < nvec; base += step) {
            float4 x[kUnroll];
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                const int v = base + (int)threadIdx.x + (int)blockDim.x * j;
                if (v < nvec) x[j] = ld_stream(x4 + v);
            }
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                const int v = base + (int)threadIdx.x + (int)blockDim.x * j;
                if (v < nvec) {
                    exp_shifted4(x[j], neg);
                    scale4(x[j], inv);
                    st_stream(y4 + v, x[j]);
                }
            }
        }
    }
}

// The same two passes with every load going through a per-thread shared-memory ring (cp.async): the block's work is
// a stream of items -- (row, pass, chunk of kUnroll vectors per thread) -- and the loads of the next kDepth - 1 items
// are always in flight, across the end of a pass and the end of a row, so the memory pipeline neither drains at the
// two block reductions of a row nor ramps up again at the start of the next.  A thread copies exactly the vectors it
// consumes, so the ring needs no block barrier.  ring: kDepth * kUnroll * kThreads vectors.
template <int kUnroll, int kThreads, int kDepth>
__device__ __forceinline__ void softmax_reread_ring_tier(const float *in, float *out, long long rows, int cols, float *s_exchange,
                                                         float4 *ring) {
    const int nvec = cols >> 2;
    constexpr int kStep = kThreads * kUnroll;
    const int chunks = (nvec + kStep - 1) / kStep;
    const float4 *in4 = reinterpret_cast<const float4 *>(in);
    const uint64_t keep = l2_keep_policy(), once = l2_stream_policy();
    // producer: the item kDepth - 1 ahead of the consumer
    long long p_row = blockIdx.x;
    int p_pass = 0, p_chunk = 0, p_slot = 0;
    auto produce = [&]() {
        if (p_row < rows) {
            const float4 *x4 = in4 + p_row * nvec;
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                const int v = p_chunk * kStep + (int)threadIdx.x + kThreads * j;
                if (v < nvec) cp_async16_policy(ring + (p_slot * kUnroll + j) * kThreads + threadIdx.x, x4 + v, p_pass == 0 ? keep : once);
            }
            if (++p_chunk == chunks) {
                p_chunk = 0;
                if (++p_pass == 2) {
                    p_pass = 0;
                    p_row += gridDim.x;
                }
            }
        }
        cp_async_commit_group();  // also when nothing was issued: the group count stays one per item
        p_slot = p_slot + 1 == kDepth ? 0 : p_slot + 1;
    };
#pragma unroll
    for (int i = 0; i < kDepth - 1; ++i) produce();
    int c_slot = 0;
    auto consume = [&](int chunk, float4 (&x)[kUnroll]) {
        produce();  // refills the slot read one item ago (by this same thread)
        cp_async_wait_group<kDepth - 1>();
#pragma unroll
        for (int j = 0; j < kUnroll; ++j) {
            const int v = chunk * kStep + (int)threadIdx.x + kThreads * j;
            x[j] = v < nvec ? ring[(c_slot * kUnroll + j) * kThreads + threadIdx.x] : neg_inf4();
        }
        c_slot = c_slot + 1 == kDepth ? 0 : c_slot + 1;
    };
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        float4 *y4 = reinterpret_cast<float4 *>(out) + row * nvec;
        float m = kNegInf, s = 0.f;
        for (int chunk = 0; chunk < chunks; ++chunk) {
            float4 x[kUnroll];
            consume(chunk, x);
            float cm = kNegInf;
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) cm = fmaxf(cm, max4(x[j]));
            const float grown = fmaxf(m, cm);
            if (grown != kNegInf) {  // a chunk of nothing but -inf adds nothing
                const float neg = -grown * kLog2e;
                float cs = 0.f;
#pragma unroll
                for (int j = 0; j < kUnroll; ++j) cs += exp_shifted4(x[j], neg);
                s = fmaf(s, exp2_approx(fmaf(m, kLog2e, neg)), cs);
                m = grown;
            }
        }
        const float row_max = block_allreduce<true>(m, s_exchange);
        const float neg = -row_max * kLog2e;
        s = m == kNegInf ? 0.f : s * exp2_approx(fmaf(m, kLog2e, neg));
        const float inv = rcp_approx(block_allreduce<false>(s, s_exchange));
        for (int chunk = 0; chunk < chunks; ++chunk) {
            float4 x[kUnroll];
            consume(chunk, x);
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                const int v = chunk * kStep + (int)threadIdx.x + kThreads * j;
                if (v < nvec) {
                    exp_shifted4(x[j], neg);
                    scale4(x[j], inv);
                    st_stream(y4 + v, x[j]);
                }
            }
        }
    }
    cp_async_wait_group<0>();
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
        const float neg = -m * kLog2e;
        float s = 0.f;
        for (int c = threadIdx.x; c < cols; c += blockDim.x) s += exp2_approx(fmaf(x[c], kLog2e, neg));
        s = block_allreduce<false>(s, s_exchange);
        const float inv = rcp_approx(s);
        for (int c = threadIdx.x; c < cols; c += blockDim.x) y[c] = exp2_approx(fmaf(x[c], kLog2e, neg)) * inv;
        __syncthreads();
    }
}

// runtime-shape kernels used by the C ABI
template <int kVecs, int kSlots, int G>
__global__ void __launch_bounds__(256) softmax_warp_kernel(const float *in, float *out, long long rows, int cols) {
    grid_launch_dependents();  // the next kernel of the stream may take SMs as this one's blocks retire
    grid_dependency_wait();    // nothing is read before the previous kernel's writes are visible
    softmax_warp_tier<kVecs, kSlots, G>(in, out, rows, cols);
}
template <int kVecs, int kSlots, int G, int kConsumerWarps>
__global__ void __launch_bounds__((kConsumerWarps + 1) * 32)
softmax_staged_kernel(const float *in, float *out, long long rows, int cols, const RowPipeGeometry geo, unsigned *status) {
    extern __shared__ __align__(128) uint8_t ko_row_stage_smem[];
    softmax_staged_tier<kVecs, kSlots, G, kConsumerWarps>(in, out, rows, cols, geo, ko_row_stage_smem, status);
}
template <int kVecs, int kThreads>
__global__ void __launch_bounds__(kThreads) softmax_block_kernel(const float *in, float *out, long long rows, int cols) {
    __shared__ float s_exchange[33];
    grid_launch_dependents();
    grid_dependency_wait();
    softmax_block_tier<kVecs>(in, out, rows, cols, s_exchange);
}
template <int kVecs, int kThreads>
__global__ void __launch_bounds__(kThreads) softmax_block_prefetch_kernel(const float *in, float *out, long long rows, int cols,
                                                                         unsigned *status) {
    extern __shared__ __align__(128) uint8_t ko_row_buffer[];  // one row
    __shared__ float s_exchange[33];
    __shared__ __align__(8) uint64_t s_bar;
    grid_launch_dependents();
    grid_dependency_wait();
    softmax_block_prefetch_tier<kVecs, kThreads>(in, out, rows, cols, reinterpret_cast<float4 *>(ko_row_buffer), &s_bar, s_exchange,
                                                 status);
}
template <int kVecs, int kThreads>
__global__ void __launch_bounds__(kThreads) softmax_cluster_kernel(const float *in, float *out, long long rows, int cols) {
    __shared__ float s_exchange[33];
    __shared__ float s_part[2][2];
    softmax_cluster_tier<kVecs, false>(in, out, rows, cols, s_exchange, s_part);
}
template <int kVecs, int kThreads>
__global__ void __launch_bounds__(kThreads) softmax_cluster_prefetch_kernel(const float *in, float *out, long long rows, int cols,
                                                                           unsigned *status, int use_mailbox) {
    extern __shared__ __align__(128) uint8_t ko_row_buffer[];  // this block's slice of one row
    __shared__ float s_exchange[33];
    __shared__ float s_part[2][2];
    __shared__ __align__(8) uint64_t s_bar;
    __shared__ __align__(8) ClusterMailbox s_mail;
    softmax_cluster_tier<kVecs, true>(in, out, rows, cols, s_exchange, s_part, reinterpret_cast<float4 *>(ko_row_buffer), &s_bar, status,
                                      use_mailbox ? &s_mail : nullptr);
}
template <int kUnroll, int kThreads>
__global__ void __launch_bounds__(kThreads) softmax_reread_kernel(const float *in, float *out, long long rows, int cols) {
    grid_launch_dependents();
    grid_dependency_wait();
    __shared__ float s_exchange[33];
    softmax_reread_tier<kUnroll>(in, out, rows, cols, s_exchange);
}
template <int kUnroll, int kThreads, int kDepth>
__global__ void __launch_bounds__(kThreads) softmax_reread_ring_kernel(const float *in, float *out, long long rows, int cols) {
    grid_launch_dependents();
    grid_dependency_wait();
    __shared__ float s_exchange[33];
    extern __shared__ __align__(16) float4 ko_softmax_item_ring[];
    softmax_reread_ring_tier<kUnroll, kThreads, kDepth>(in, out, rows, cols, s_exchange, ko_softmax_item_ring);
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
    static constexpr int kNvec = num_column / 4;
    static constexpr int kGroup = kNvec <= 32 ? 8 : (kNvec <= 64 ? 16 : 32);   // lanes per row
    static constexpr int kVecs = (kNvec + kGroup - 1) / kGroup;
    static_assert(kVecs <= 16, "row too long for the warp tier; use SoftMaxBlockImpl");
    static constexpr int kSlots = kVecs >= 8 ? 1 : 2;
    __device__ __forceinline__ static void run(T *in_data, T *out_data) {
        ko::softmax_warp_tier<kVecs, kSlots, kGroup>(in_data, out_data, num_row, num_column);
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
