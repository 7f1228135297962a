// Persistent, TMA-staged streaming of whole rows through shared memory (the "staged tier" of the
// row operators).
//
// A thread block owns a contiguous range of rows.  Warp 0 is the producer: one lane issues 1-D bulk
// copies (cp.async.bulk, this block's shared memory only) of `rows_per_stage` consecutive rows --
// one contiguous chunk of global memory -- into a ring of stages and signals a `full` mbarrier with
// the byte count.  The other warps consume: they wait for a stage, process its rows out of shared
// memory, write results straight to global memory, and release the stage through an `empty`
// mbarrier.  The producer runs up to `stages` chunks ahead, so the bytes in flight per SM are set by
// the ring (tens of KB), not by occupancy or by how many registers the row math needs.
//
// Every mbarrier wait is bounded; when one runs out the block records a code in the device status
// word, raises its abort flag, waits (bounded) for the copies it already issued and returns.
#pragma once

#include "common.h"

namespace ko {

enum : unsigned { kRowPipeOk = 0, kRowPipeTimeoutProducer = 1, kRowPipeTimeoutConsumer = 2 };

struct RowPipeGeometry {
    int rows_per_stage;  // rows per bulk copy
    int stages;          // ring depth
    unsigned row_bytes;  // bytes per row (multiple of 16)
};

// bytes of dynamic shared memory the pipeline needs
__host__ __device__ inline size_t row_pipe_smem_bytes(const RowPipeGeometry &g) {
    return (size_t)g.stages * g.rows_per_stage * g.row_bytes + 128 /*alignment*/ + 2 * 8 * (size_t)g.stages + 16;
}

// kConsumerWarps + 1 warps per block.  consume(stage_base, first_row, nrows, stage_index, consumer_warp,
// lane) is called by every consumer warp for every stage; the rows of the stage are
// [first_row, first_row+nrows) and stage_index counts this block's stages from 0.
template <int kConsumerWarps, typename Consume>
__device__ __forceinline__ void row_pipeline(const void *in, long long rows, const RowPipeGeometry geo, uint8_t *smem_raw,
                                             unsigned *status, Consume &&consume) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t ring = (raw + 127u) & ~127u;
    uint8_t *ring_ptr = smem_raw + (ring - raw);
    const uint32_t stage_bytes = (uint32_t)geo.rows_per_stage * geo.row_bytes;
    const uint32_t bar_base = ring + (uint32_t)geo.stages * stage_bytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (geo.stages + s); };
    volatile int *abort_flag = reinterpret_cast<volatile int *>(ring_ptr + (size_t)geo.stages * stage_bytes + 16 * geo.stages);

    // this block's rows
    const long long row_begin = rows * blockIdx.x / gridDim.x;
    const long long row_end = rows * (blockIdx.x + 1) / gridDim.x;
    const int my_stages = (int)((row_end - row_begin + geo.rows_per_stage - 1) / geo.rows_per_stage);

    if (threadIdx.x == 0) {
        for (int s = 0; s < geo.stages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), kConsumerWarps);
        }
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    __syncthreads();

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (; it < my_stages; ++it) {
                const int s = it % geo.stages;
                const uint32_t phase = (uint32_t)(it / geo.stages) & 1u;
                if (!mbar_wait(empty_bar(s), phase ^ 1u, abort_flag)) {
                    if (!*abort_flag) atomicCAS(status, kRowPipeOk, kRowPipeTimeoutProducer);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                const long long first = row_begin + (long long)it * geo.rows_per_stage;
                const long long n = min((long long)geo.rows_per_stage, row_end - first);
                const uint32_t bytes = (uint32_t)n * geo.row_bytes;
                mbar_expect_tx(full_bar(s), bytes);
                bulk_load_1d(ring + s * stage_bytes, static_cast<const uint8_t *>(in) + first * geo.row_bytes, bytes, full_bar(s));
            }
            if (!ok || *abort_flag) {
                // copies already issued still land in shared memory: wait (bounded) for the latest
                // fill of every stage before the block retires
                for (int back = 0; back < geo.stages && back < it; ++back) {
                    const int j = it - 1 - back;
                    const uint32_t bar = full_bar(j % geo.stages), parity = (uint32_t)(j / geo.stages) & 1u;
                    for (uint32_t spin = 0; spin < kSpinLimit && !mbar_try_wait(bar, parity); ++spin) {}
                }
            }
        }
        __syncwarp();
    } else {
        const int cw = warp - 1;
        for (int it = 0; it < my_stages; ++it) {
            const int s = it % geo.stages;
            const uint32_t phase = (uint32_t)(it / geo.stages) & 1u;
            if (!mbar_wait(full_bar(s), phase, abort_flag)) {
                if (lane == 0 && !*abort_flag) atomicCAS(status, kRowPipeOk, kRowPipeTimeoutConsumer);
                *abort_flag = 1;
                break;
            }
            const long long first = row_begin + (long long)it * geo.rows_per_stage;
            const int n = (int)min((long long)geo.rows_per_stage, row_end - first);
            consume(ring_ptr + (size_t)s * stage_bytes, first, n, it, cw, lane);
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar(s));
        }
    }
    // keep shared memory alive until every role is done with it
    __syncthreads();
}

// ---------------------------------------------------------------------------------------------
// one-row prefetch used by the block- and cluster-per-row tiers: warp 0 copies a block's next row (or its
// slice of it) into a shared-memory buffer with 1-D bulk copies while the current row is processed from
// registers; one mbarrier counts the bytes, the consumers' wait is bounded (mbar_wait)
// ---------------------------------------------------------------------------------------------
constexpr unsigned kRowPrefetchTimeout = 3;  // status code (row-operator status word)
constexpr uint32_t kBulkPiece = 16384;       // bytes per bulk copy: the lanes of warp 0 issue the pieces of a row in parallel

__device__ __forceinline__ void prefetch_row(const void *row_ptr, uint32_t row_bytes, uint32_t buf, uint32_t bar) {
    // warp 0 only; row_bytes is a multiple of 16
    const int lane = threadIdx.x & 31;
    fence_proxy_async();  // the buffer's previous contents were read through the generic proxy (ordered by the block barrier)
    if (lane == 0) mbar_expect_tx(bar, row_bytes);
    __syncwarp();
    for (uint32_t off = (uint32_t)lane * kBulkPiece; off < row_bytes; off += 32u * kBulkPiece) {
        const uint32_t n = min(kBulkPiece, row_bytes - off);
        bulk_load_1d(buf + off, reinterpret_cast<const uint8_t *>(row_ptr) + off, n, bar);
    }
}


// Work split inside a stage: the stage's rows form groups of `rows_per_group` (what one warp takes
// at a time); groups are dealt round-robin over the consumer warps, continuing across stages so that
// stages smaller than one group per warp still keep every warp busy.
__device__ __forceinline__ int first_group_of_warp(int stage_index, int groups_per_full_stage, int consumer_warp,
                                                   int consumer_warps) {
    const int dealt = (int)(((long long)stage_index * groups_per_full_stage) % consumer_warps);
    return (consumer_warp - dealt + consumer_warps) % consumer_warps;
}

}  // namespace ko
