// Two-SM form of the tensor-core GEMM (tcgen05 cta_group::2): a cluster of two CTAs computes one 256 x BN tile.
//
// Each CTA of the pair brings in ITS OWN 128 rows of A and ITS OWN half of the B tile (BN/2 columns) with plain
// per-CTA TMA loads from this GPU's memory -- no multicast anywhere -- and one thread of the pair's leader (cluster
// rank 0) issues tcgen05.mma.cta_group::2 (M = 256, N = BN, K = 16): the hardware reads both CTAs' shared memory,
// each SM accumulating its 128 rows x BN columns in its own tensor memory.  Per CTA that is 16 KB of A + 16 KB of B
// per K-block for a 128 x 256 accumulator -- the operand traffic of the single-CTA 256 x 256 tile -- while the
// accumulator still fits tensor memory twice (2 x 256 columns), so the epilogue of one tile overlaps the MMAs of the
// next, which the single-CTA 256 x 256 tile cannot do.
//
// Synchronisation (all mbarriers; every wait is bounded and reports through the device status word):
//   full[s]      leader only.  The leader's producer posts the byte count of BOTH CTAs' loads of stage s; both CTAs'
//                TMA loads complete on it (the peer passes the leader's barrier, cp.async.bulk.tensor ... cta_group::2).
//   empty[s]     one per CTA.  The leader's MMA thread commits (tcgen05.commit.cta_group::2, which tracks both SMs) to
//                the leader's barrier only -- a commit costs the MMA issue stream about 50 ns, a second one per stage
//                measured 14 % -- and the leader's producer, once it has seen that release, passes it on to the
//                peer's barrier with a relaxed remote arrive; each producer waits on its own barrier.
//   acc_ready[a] one per CTA, two plain commits (shared::cluster addresses) once a tile's MMAs are issued; each CTA's
//                epilogue warps wait on their own.
//   acc_free[a]  leader only, 8 arrivals: the four epilogue warps of both CTAs (the peer's arrive remotely).
// Before tensor memory is released and before either CTA exits, the leader drains its MMAs and the pair meets at a
// cluster barrier: the leader's MMAs read the peer's shared memory and write its tensor memory until then.
//
// Column-major B only; K a multiple of 8; any M, N (TMA zero-fills, stores are clipped / predicated).  Uneven column
// tiles (GemmParams::tiles_n) work as in the single-CTA kernel with widths that are multiples of 32.
#pragma once

#include "tensor_core_gemm.h"

namespace ko {
namespace tc {

struct PairConfig {
    static constexpr int kBN = 256;                          // widest tile; TMEM holds two accumulators of it
    static constexpr int kBytesA = kBM * kBK * 2;            // this CTA's 128 rows
    static constexpr int kBytesB = (kBN / 2) * kBK * 2;      // this CTA's half of the B tile, at most
    static constexpr int kStageBytes = kBytesA + kBytesB;    // 32 KB
    static constexpr int kStages = 6;
    static constexpr int kTmemCols = 2 * kBN;
    static constexpr int kStoreBoxes = 2;
    static constexpr int kStoreBoxBytes = 32 * 32 * 4;
    static constexpr int kStoreBytes = 4 * kStoreBoxes * kStoreBoxBytes;
    static constexpr int kBarrierBytes = 256;
    static constexpr int kSmemBytes = kStages * kStageBytes + kStoreBytes + kBarrierBytes + 1024;
    static_assert(kSmemBytes <= 232448, "stage ring exceeds the shared memory of an SM");
};

// ---- cta_group::2 forms of the PTX wrappers ----
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// whole warp, in both CTAs of the pair, same shared-memory offset for the result
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_result, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// D[tmem of both SMs] (+)= A[both CTAs' smem] * B[both CTAs' smem]; issued by one thread of the leader CTA; the
// descriptors as (low, high) words (see umma_f16_words)
__device__ __forceinline__ void umma_f16_pair_words(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                                    uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrives on the mbarrier at shared::cluster address `bar` once every tcgen05.mma issued so far by this thread has
// completed in both SMs
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}
// TMA 2-D tile load into THIS CTA's shared memory, completion counted on an mbarrier that may live in the other CTA
// of the pair (shared::cluster address); no multicast: the tile is delivered to this CTA only
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(cluster_bar)
        : "memory");
}
// Arrive on an mbarrier of another CTA of the cluster as a pure token (no data of this thread is handed over, so no
// release: a releasing arrive from the producer thread measured twice the kernel time, it waits for the thread's
// copies in flight).
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_bar_addr) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar_addr) : "memory");
}
// bounded wait with cluster-scope acquire (for barriers another CTA arrives on)
__device__ __forceinline__ bool mbar_wait_remote(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if ((spin & 1023u) == 1023u && *abort_flag) return false;
    }
    return false;
}

// map_b / map_b_narrow: boxes of bn_wide / 2 and bn_narrow / 2 rows (128 rows when the tiles are uniform)
template <bool kTmaStore>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const __grid_constant__ CUtensorMap map_b_narrow, const __grid_constant__ CUtensorMap map_d,
                         const GemmParams p) {
    using Cfg = PairConfig;
    constexpr int BN = Cfg::kBN, kTileM = 2 * kBM;
    extern __shared__ uint8_t ko_tc_pair_smem_raw[];
    const uint32_t raw = smem_u32(ko_tc_pair_smem_raw);
    const uint32_t ring = (raw + 1023u) & ~1023u;  // the same offset in both CTAs
    uint8_t *ring_ptr = ko_tc_pair_smem_raw + (ring - raw);
    const uint32_t store_base = ring + Cfg::kStages * Cfg::kStageBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(ring_ptr + Cfg::kStages * Cfg::kStageBytes + Cfg::kStoreBytes);
    const uint32_t bar_base = store_base + Cfg::kStoreBytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (Cfg::kStages + s); };
    auto acc_ready_bar = [&](int a) { return bar_base + 8u * (2 * Cfg::kStages + a); };
    auto acc_free_bar = [&](int a) { return bar_base + 8u * (2 * Cfg::kStages + 2 + a); };
    const uint32_t drain_bar = bar_base + 8u * (2 * Cfg::kStages + 4);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * Cfg::kStages + 5);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();  // 0 = leader
    const bool leader = rank == 0;
    const int tiles_m = (p.M + kTileM - 1) / kTileM, tiles_n = p.tiles_n ? p.tiles_n : (p.N + BN - 1) / BN;
    const long long num_tiles = (long long)tiles_m * tiles_n;
    const int k_blocks = (p.K + kBK - 1) / kBK;
    const long long pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_ready_bar(a), 1);
            mbar_init(acc_free_bar(a), 8);  // four epilogue warps of each CTA
        }
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        if (p.tiles_n) prefetch_tensormap(&map_b_narrow);
        if (kTmaStore) prefetch_tensormap(&map_d);
    }
    grid_launch_dependents();
    if (warp == 1) tmem_alloc_pair(smem_u32(tmem_slot), Cfg::kTmemCols);
    tc_fence_before();
    __syncthreads();
    cluster_barrier();  // both CTAs' barriers are initialised before either signals the other's
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    grid_dependency_wait();

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (long long t = pair; t < num_tiles && ok; t += pairs) {
                int tm, tn, col0, bn;
                tile_of(p, t, tiles_m, tiles_n, tm, tn);
                column_tile<BN>(p, tn, col0, bn);
                const int half = bn >> 1;  // this CTA's share of the tile's columns
                const CUtensorMap *b_map = (p.tiles_n && bn != p.bn_wide) ? &map_b_narrow : &map_b;  // box of bn / 2 rows
                const uint32_t cta_bytes = (uint32_t)Cfg::kBytesA + (uint32_t)half * (kBK * 2);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % Cfg::kStages;
                    const uint32_t phase = (it / Cfg::kStages) & 1u;
                    if (!mbar_wait(empty_bar(s), phase ^ 1u, abort_flag)) {
                        if (!*abort_flag) atomicCAS(p.status, kStatusOk, kTimeoutProducer);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    if (leader) {
                        // the MMAs that read this stage -- in both CTAs -- have completed: tell the peer's producer (a plain
                        // remote arrive; a second tcgen05.commit per stage would cost the MMA issue stream ~50 ns each)
                        if (it >= (uint32_t)Cfg::kStages) mbar_arrive_cluster_relaxed(map_to_cluster_rank(empty_bar(s), 1));
                        mbar_expect_tx(full_bar(s), 2u * cta_bytes);  // both CTAs' loads land on this barrier
                    }
                    const uint32_t leader_full = map_to_cluster_rank(full_bar(s), 0);
                    const uint32_t dst = ring + s * Cfg::kStageBytes;
                    tma_load_2d_pair(dst, &map_a, kb * kBK, tm * kTileM + (int)rank * kBM, leader_full);
                    if (!p.b_row_major) {
                        tma_load_2d_pair(dst + Cfg::kBytesA, b_map, kb * kBK, col0 + (int)rank * half, leader_full);
                    } else {
                        // row-major B: this CTA's 128 columns as two boxes of 64 K-rows x 64 columns (MN-major operand)
#pragma unroll
                        for (int nb = 0; nb < BN / 128; ++nb)
                            tma_load_2d_pair(dst + Cfg::kBytesA + nb * 8192, &map_b, col0 + (int)rank * (BN / 2) + nb * 64, kb * kBK,
                                             leader_full);
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && leader) {
            uint32_t it = 0, local_tile = 0;
            uint32_t stage = 0, phase = 0;  // ring position of K-block `it` and the parity of its fill
            // descriptor words of the ring's first stage, stepped by 32-bit adds (see the single-CTA kernel)
            const uint32_t desc_hi = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);
            const uint32_t a_lo0 = ((ring & 0x3ffffu) >> 4) | (1u << 16);
            const uint32_t b_lo0 = (((ring + Cfg::kBytesA) & 0x3ffffu) >> 4) | (p.b_row_major ? (uint32_t)(8192 >> 4) << 16 : 1u << 16);
            const uint32_t b_kstep = p.b_row_major ? 2048u >> 4 : (uint32_t)(kUmmaK * 2) >> 4;
            bool ok = true;
            const uint32_t own_empty0 = map_to_cluster_rank(empty_bar(0), 0);
            const uint32_t peer_ready0 = map_to_cluster_rank(acc_ready_bar(0), 1), own_ready0 = map_to_cluster_rank(acc_ready_bar(0), 0);
            for (long long t = pair; t < num_tiles && ok; t += pairs, ++local_tile) {
                int tm, tn, col0, bn;
                tile_of(p, t, tiles_m, tiles_n, tm, tn);
                column_tile<BN>(p, tn, col0, bn);
                const uint32_t idesc = make_idesc(p.fmt, kTileM, bn) | (p.b_row_major ? 1u << 16 : 0u);  // bit 16: B is MN-major
                const uint32_t acc = local_tile & 1u, acc_phase = (local_tile >> 1) & 1u;
                if (!mbar_wait_remote(acc_free_bar(acc), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_lo = a_lo0 + stage * (uint32_t)(Cfg::kStageBytes >> 4), b_lo = b_lo0 + stage * (uint32_t)(Cfg::kStageBytes >> 4);
                    uint32_t accumulate = kb != 0 ? 1u : 0u;
#pragma unroll
                    for (int k = 0; k < kBK / kUmmaK; ++k) {
                        umma_f16_pair_words(d_tmem, a_lo + k * 2, desc_hi, b_lo + k * b_kstep, desc_hi, idesc, accumulate);
                        accumulate = 1u;
                    }
                    // the stage is reusable once these MMAs have read it (in both CTAs: the commit tracks both SMs); the
                    // leader's producer passes the release on to the peer
                    umma_commit_pair(own_empty0 + 8u * stage);
                    if (++stage == (uint32_t)Cfg::kStages) { stage = 0; phase ^= 1u; }
                }
                if (ok) {
                    umma_commit_pair(own_ready0 + 8u * acc);
                    umma_commit_pair(peer_ready0 + 8u * acc);
                }
            }
            if (!ok) {
                if (!*abort_flag) atomicCAS(p.status, kStatusOk, kTimeoutMma);
                *abort_flag = 1;
            }
            // nothing may still be reading the peer's shared memory or writing tensor memory when the pair parts
            umma_commit_pair(map_to_cluster_rank(drain_bar, 0));
            bool drained = false;
            for (uint32_t spin = 0; spin < kSpinLimit && !(drained = mbar_try_wait(drain_bar, 0)); ++spin) {}
            if (!drained) atomicCAS(p.status, kStatusOk, kTimeoutDrain);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
        const int quad = warp & 3;
        uint32_t local_tile = 0, store_seq = 0;
        bool ok = true;
        for (long long t = pair; t < num_tiles && ok; t += pairs, ++local_tile) {
            int tm, tn, col0, bn;
            tile_of(p, t, tiles_m, tiles_n, tm, tn);
            column_tile<BN>(p, tn, col0, bn);
            const uint32_t acc = local_tile & 1u, acc_phase = (local_tile >> 1) & 1u;
            if (!mbar_wait(acc_ready_bar(acc), acc_phase, abort_flag)) {
                if (lane == 0 && !*abort_flag) atomicCAS(p.status, kStatusOk, kTimeoutEpilogue);
                *abort_flag = 1;
                ok = false;
                break;
            }
            tc_fence_after();
            const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN;
            epilogue_block<kTmaStore, Cfg::kStoreBoxes>(&map_d, p, t_row, tm * kTileM + (int)rank * kBM + quad * 32, col0, bn, lane,
                                                        store_base + (uint32_t)((warp - 2) * Cfg::kStoreBoxes) * Cfg::kStoreBoxBytes,
                                                        (uint32_t)Cfg::kStoreBoxBytes, store_seq);
            // the accumulator may be overwritten once all eight epilogue warps of the pair have read theirs
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cluster_rank(acc_free_bar(acc), 0));
        }
        if (kTmaStore && lane == 0) bulk_wait_group_read<0>();
        __syncwarp();
    }

    tc_fence_before();
    __syncthreads();
    cluster_barrier();  // the leader has drained its MMAs; nobody touches the other CTA's memory after this
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
    }
}

}  // namespace tc
}  // namespace ko
