// C-ABI launchers of the LayerNorm forward: tier and launch geometry from the runtime shape.
#include "row_launch.h"

#include <algorithm>

#include "../nn_operators/layernorm/layernorm.h"

namespace {

using ko::DeviceInfo;

template <typename T>
struct Args {
    const T *in;
    T *out;
    long long rows;
    int cols;
    float eps;
    const T *gamma, *beta;
    int ddof;
};

template <typename T, int kVecs, int kRows>
int launch_warp(const Args<T> &a, const ko_row_knobs_t &k, cudaStream_t s) {
    const int block = (k.block > 0 && k.block <= 256) ? k.block : 128;
    const long long groups = (a.rows + kRows - 1) / kRows;
    const unsigned grid = ko::clamp_grid((groups + block / 32 - 1) / (block / 32), k.grid_cap);
    return ko::launch_overlapped(ko::layernorm_warp_kernel<T, kVecs, kRows>, grid, (unsigned)block, 0, s, a.in, a.out,
                                 (long long)a.rows, a.cols, a.eps, a.gamma, a.beta, a.ddof);
}

template <typename T, int kVecs, int kRows>
int launch_staged(const Args<T> &a, const ko_row_knobs_t &k, const DeviceInfo &info, cudaStream_t s, bool *used) {
    constexpr int W = ko::kStagedConsumerWarps;
    const ko::StagedPlan plan = ko::plan_staged(a.rows, (unsigned)a.cols * (unsigned)sizeof(T), kRows, k, info);
    *used = plan.ok;
    if (!plan.ok) return KO_OK;
    unsigned *status = nullptr;
    if (int st = ko::device_status_word(1, &status)) return st;
    auto kernel = ko::layernorm_staged_kernel<T, kVecs, kRows, W>;
    if (int st = ko::ensure_dynamic_smem(reinterpret_cast<const void *>(kernel), plan.smem_bytes)) return st;
    kernel<<<plan.grid, ko::kStagedThreads, plan.smem_bytes, s>>>(a.in, a.out, a.rows, a.cols, a.eps, a.gamma, a.beta, a.ddof,
                                                                  plan.geo, status);
    KO_CHECK_LAUNCH("layernorm_staged_kernel");
    return KO_OK;
}

template <typename T, int kVecs, int kThreads>
int launch_block(const Args<T> &a, long long grid_cap, cudaStream_t s) {
    return ko::launch_overlapped(ko::layernorm_block_kernel<T, kVecs, kThreads>, ko::clamp_grid(a.rows, grid_cap), kThreads, 0, s,
                                 a.in, a.out, (long long)a.rows, a.cols, a.eps, a.gamma, a.beta, a.ddof);
}

template <typename T, int kThreads>
int launch_block_vecs(int vecs, const Args<T> &a, long long grid_cap, cudaStream_t s) {
    if (vecs <= 1) return launch_block<T, 1, kThreads>(a, grid_cap, s);
    if (vecs <= 2) return launch_block<T, 2, kThreads>(a, grid_cap, s);
    if (vecs <= 4) return launch_block<T, 4, kThreads>(a, grid_cap, s);
    return launch_block<T, 8, kThreads>(a, grid_cap, s);
}

template <typename T, int kVecs, int kThreads, int kRing>
int launch_resident(const Args<T> &a, long long grid_cap, int sm_count, cudaStream_t s) {
    // persistent blocks: exactly as many as the device holds at once, so that no block waits for a slot and the
    // rows are dealt evenly (more blocks than that would run as a partly filled second wave)
    const bool affine = a.gamma || a.beta;
    auto with_affine = ko::layernorm_resident_kernel<T, kVecs, kThreads, true, kRing>;
    auto without = ko::layernorm_resident_kernel<T, kVecs, kThreads, false, kRing>;
    constexpr size_t kRingBytes = (size_t)kRing * kThreads * kVecs * 16;
    const void *fn = affine ? reinterpret_cast<const void *>(with_affine) : reinterpret_cast<const void *>(without);
    if (kRingBytes + 1024 > (48u << 10))  // the kernel's static shared memory counts against the 48 KB a launch gets unasked
        if (int st = ko::ensure_dynamic_smem(fn, kRingBytes)) return st;
    int per_sm = 0;
    if (affine) KO_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, with_affine, kThreads, kRingBytes));
    else KO_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, without, kThreads, kRingBytes));
    const long long cap = grid_cap > 0 ? grid_cap : (long long)sm_count * (per_sm > 0 ? per_sm : 1);
    const unsigned grid = ko::clamp_grid(a.rows, cap);
    if (affine)
        return ko::launch_overlapped(with_affine, grid, kThreads, kRingBytes, s, a.in, a.out, (long long)a.rows, a.cols, a.eps, a.gamma,
                                     a.beta, a.ddof);
    return ko::launch_overlapped(without, grid, kThreads, kRingBytes, s, a.in, a.out, (long long)a.rows, a.cols, a.eps, a.gamma, a.beta,
                                 a.ddof);
}

// ring: rows in flight into shared memory per block (cp.async) instead of one row into registers: three rows while a
// row is at most 8 KB, two beyond (up to 2 x 64 KB)
template <typename T, int kVecs, int kThreads>
int launch_resident_ring(bool ring, const Args<T> &a, long long grid_cap, int sm_count, cudaStream_t s) {
    constexpr int kDepth = kThreads * kVecs <= 512 ? 3 : 2;
    if (ring) return launch_resident<T, kVecs, kThreads, kDepth>(a, grid_cap, sm_count, s);
    return launch_resident<T, kVecs, kThreads, 0>(a, grid_cap, sm_count, s);
}

template <typename T, int kThreads>
int launch_resident_vecs(int vecs, bool ring, const Args<T> &a, long long grid_cap, int sm_count, cudaStream_t s) {
    if (vecs <= 1) return launch_resident_ring<T, 1, kThreads>(ring, a, grid_cap, sm_count, s);
    if (vecs <= 2) return launch_resident_ring<T, 2, kThreads>(ring, a, grid_cap, sm_count, s);
    return launch_resident_ring<T, 4, kThreads>(ring, a, grid_cap, sm_count, s);
}

// one row per cluster of `c` blocks of 1024 threads, up to 8 vectors per thread
template <typename T>
int launch_cluster(const Args<T> &a, int c, bool mailbox, long long grid_cap, int sm_count, cudaStream_t s) {
    const int slice = (a.cols / ko::RowIo<T>::kPerVec + c - 1) / c;
    const int threads = slice <= 256 * 4 ? 256 : 1024;
    // clusters that can be resident at once (a cluster lives inside one GPC: fewer than SMs / c); more than that
    // would run as a second wave behind grid-stride loops that already cover every row
    const void *probe = threads == 256 ? reinterpret_cast<const void *>(ko::layernorm_cluster_kernel<T, 4, 256>)
                                       : reinterpret_cast<const void *>(ko::layernorm_cluster_kernel<T, 8, 1024>);
    int resident = 0;
    if (int st = ko::max_resident_clusters(probe, (unsigned)threads, (unsigned)c, 0, &resident)) return st;
    (void)sm_count;
    long long clusters = a.rows;
    const long long cap = grid_cap > 0 ? grid_cap / c : (long long)resident;
    if (clusters > cap) clusters = cap > 0 ? cap : 1;
    const unsigned grid = (unsigned)(clusters * c);
    unsigned *status = nullptr;
    if (int st = ko::device_status_word(1, &status)) return st;
    const int mail = mailbox ? 1 : 0;
    if (slice <= 256 * 4)
        return ko::launch_clustered(ko::layernorm_cluster_kernel<T, 4, 256>, grid, 256, c, s, a.in, a.out, a.rows, a.cols, a.eps, a.gamma,
                                    a.beta, a.ddof, status, mail);
    if (slice <= 1024 * 4)
        return ko::launch_clustered(ko::layernorm_cluster_kernel<T, 4, 1024>, grid, 1024, c, s, a.in, a.out, a.rows, a.cols, a.eps, a.gamma,
                                    a.beta, a.ddof, status, mail);
    return ko::launch_clustered(ko::layernorm_cluster_kernel<T, 8, 1024>, grid, 1024, c, s, a.in, a.out, a.rows, a.cols, a.eps, a.gamma,
                                a.beta, a.ddof, status, mail);
}

template <typename T, bool kStaged>
int dispatch_rows(int vecs, int rpw, const Args<T> &a, const ko_row_knobs_t &k, const DeviceInfo &info, cudaStream_t s,
                  bool *used) {
#define KO_GO(V, R)                                                                  \
    do {                                                                             \
        if constexpr (kStaged) return launch_staged<T, V, R>(a, k, info, s, used);   \
        else { *used = true; return launch_warp<T, V, R>(a, k, s); }                 \
    } while (0)
    if (vecs == 1) { if (rpw == 1) KO_GO(1, 1); if (rpw == 2) KO_GO(1, 2); KO_GO(1, 4); }
    if (vecs == 2) { if (rpw == 1) KO_GO(2, 1); if (rpw == 4) KO_GO(2, 4); KO_GO(2, 2); }
    // 768 columns of 16-bit data: one row per warp (BF16 [16384,768] 11.7 us, 12.9 with two rows or with a padded fourth vector)
    if (vecs == 3) { if (rpw == 2) KO_GO(3, 2); if (rpw == 4) KO_GO(3, 4); KO_GO(3, 1); }
    if (vecs <= 4) { if (rpw == 1) KO_GO(4, 1); KO_GO(4, 2); }
    if (vecs <= 6) { if (rpw == 2) KO_GO(6, 2); KO_GO(6, 1); }
    if (vecs <= 8) { if (rpw == 2) KO_GO(8, 2); KO_GO(8, 1); }
    if (vecs <= 12) KO_GO(12, 1);
    KO_GO(16, 1);
#undef KO_GO
}

// short rows: G lanes per row, kVecs vectors per lane, kSlots x 32/G rows per warp step; persistent warps
template <typename T, int kVecs, int kSlots, int G>
int launch_group(const Args<T> &a, long long grid_cap, int sm_count, cudaStream_t s) {
    auto kernel = ko::layernorm_group_kernel<T, kVecs, kSlots, G>;
    int per_sm = 0;
    KO_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, 256, 0));
    constexpr int kRowsPerBlock = 8 * kSlots * (32 / G);
    const long long blocks = (a.rows + kRowsPerBlock - 1) / kRowsPerBlock;
    const long long cap = grid_cap > 0 ? grid_cap : (long long)sm_count * (per_sm > 0 ? per_sm : 1);
    return ko::launch_overlapped(kernel, ko::clamp_grid(blocks, cap), 256u, 0, s, a.in, a.out, (long long)a.rows, a.cols, a.eps, a.gamma,
                                 a.beta, a.ddof);
}

template <typename T, int G>
int launch_group_g(int nvec, int slots, const Args<T> &a, long long grid_cap, int sm_count, cudaStream_t s) {
    const int per_lane = (nvec + G - 1) / G;
    if (per_lane <= 1) {
        if (slots == 1) return launch_group<T, 1, 1, G>(a, grid_cap, sm_count, s);
        if (slots == 4) return launch_group<T, 1, 4, G>(a, grid_cap, sm_count, s);
        return launch_group<T, 1, 2, G>(a, grid_cap, sm_count, s);
    }
    if (per_lane <= 2) {
        if (slots == 1) return launch_group<T, 2, 1, G>(a, grid_cap, sm_count, s);
        if (slots == 4) return launch_group<T, 2, 4, G>(a, grid_cap, sm_count, s);
        return launch_group<T, 2, 2, G>(a, grid_cap, sm_count, s);
    }
    if (per_lane <= 3) {  // 24 or 48 vectors fill 8 or 16 lanes exactly with three each (padded vectors cost as much as real ones)
        // two row slots by default for FP32 ([349525,96] 5.8 -> 6.0 TB/s), one for 16-bit data
        if (slots == 2 || (slots == 0 && sizeof(T) == 4)) return launch_group<T, 3, 2, G>(a, grid_cap, sm_count, s);
        return launch_group<T, 3, 1, G>(a, grid_cap, sm_count, s);
    }
    if (per_lane <= 4) {
        if (slots == 2) return launch_group<T, 4, 2, G>(a, grid_cap, sm_count, s);
        return launch_group<T, 4, 1, G>(a, grid_cap, sm_count, s);
    }
    return ko::fail(KO_ERR_SHAPE, "layernorm: %d lanes hold at most %d vectors per row", G, G * 4);
}

// one row per block, read twice (the second time from the L2); blocks per SM: as many as fit, fewer when the rows in
// flight would not fit in `l2_budget` bytes
template <typename T, int kThreads, bool kPair>
int launch_reread(const Args<T> &a, long long grid_cap, int sm_count, cudaStream_t s) {
    // registers: 16-bit vectors unpack to 8 floats each, and a pair of rows doubles what the second pass holds
    constexpr int kStatUnroll = (sizeof(T) == 2 && kThreads == 1024) ? 2 : 4;
    constexpr int kUnroll = ((sizeof(T) == 2 || kPair) && kThreads == 1024) ? 2 : 4;
    auto kernel = ko::layernorm_reread_kernel<T, kStatUnroll, kUnroll, kThreads, kPair>;
    long long cap = grid_cap;
    if (cap <= 0) {
        int per_sm = 0;
        KO_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, 0));
        const long long l2_budget = 80ll << 20;
        const long long fit = l2_budget / ((long long)a.cols * (long long)sizeof(T) * sm_count * (kPair ? 2 : 1));
        cap = (long long)sm_count * std::max(1ll, std::min<long long>(per_sm, fit));
    }
    const long long units = kPair ? (a.rows + 1) / 2 : a.rows;
    return ko::launch_overlapped(kernel, ko::clamp_grid(units, cap), (unsigned)kThreads, 0, s, a.in, a.out, a.rows, a.cols, a.eps,
                                 a.gamma, a.beta, a.ddof);
}

// the single-row reread tier with every row load through a per-thread shared-memory ring of kDepth items
template <typename T, int kThreads, int kUnroll, int kDepth>
int launch_reread_ring(const Args<T> &a, long long grid_cap, int sm_count, cudaStream_t s) {
    auto kernel = ko::layernorm_reread_ring_kernel<T, kUnroll, kThreads, kDepth>;
    constexpr size_t kBytes = (size_t)kDepth * kUnroll * kThreads * 16;
    if (int st = ko::ensure_dynamic_smem(reinterpret_cast<const void *>(kernel), kBytes)) return st;
    long long cap = grid_cap;
    if (cap <= 0) {
        int per_sm = 0;
        KO_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, kBytes));
        const long long fit = (80ll << 20) / ((long long)a.cols * (long long)sizeof(T) * sm_count);
        cap = (long long)sm_count * std::max(1ll, std::min<long long>(per_sm, fit));
    }
    return ko::launch_overlapped(kernel, ko::clamp_grid(a.rows, cap), (unsigned)kThreads, kBytes, s, a.in, a.out, a.rows, a.cols, a.eps,
                                 a.gamma, a.beta, a.ddof);
}

template <typename T>
int layernorm_dispatch(const Args<T> &a, const ko_row_knobs_t *knobs, cudaStream_t s) {
    KO_REQUIRE(a.rows >= 0 && a.cols >= 0, KO_ERR_INVALID_ARG, "layernorm: negative shape [%lld, %d]", a.rows, a.cols);
    KO_REQUIRE(a.ddof == 0 || a.ddof == 1, KO_ERR_INVALID_ARG, "layernorm: ddof must be 0 or 1, got %d", a.ddof);
    if (a.rows == 0 || a.cols == 0) return KO_OK;
    KO_REQUIRE(a.in != nullptr && a.out != nullptr, KO_ERR_INVALID_ARG, "layernorm: NULL pointer");
    const ko_row_knobs_t k = knobs ? *knobs : ko_row_knobs_t{};
    KO_REQUIRE((k.tier >= 0 && k.tier <= 6) || k.tier == 8 || k.tier == 9, KO_ERR_INVALID_ARG, "layernorm: unknown tier %d", k.tier);
    KO_REQUIRE(k.cluster == 0 || k.cluster == 2 || k.cluster == 4 || k.cluster == 8, KO_ERR_INVALID_ARG,
               "layernorm: cluster size %d not in {2,4,8}", k.cluster);
    KO_REQUIRE(k.block >= 0 && k.block % 32 == 0 && k.block <= 1024, KO_ERR_INVALID_ARG,
               "layernorm: block %d must be a multiple of 32, <= 1024", k.block);
    DeviceInfo info;
    if (int st = ko::current_device_info(&info)) return st;

    constexpr int kPer = ko::RowIo<T>::kPerVec;
    constexpr int kMaxVecsPerThread = 8;  // block tier: 8 raw vectors per thread
    const bool vec_ok = a.cols % kPer == 0 && ko::aligned16(a.in) && ko::aligned16(a.out) && ko::aligned16(a.gamma) &&
                        ko::aligned16(a.beta);
    const int nvec = a.cols / kPer;
    const int vecs = (nvec + 31) / 32;
    const bool warp_ok = vec_ok && nvec <= 32 * 16;

    int tier = k.tier;
    if (tier == 0) {
        if (!vec_ok) tier = 3;
        // measured on B200: the warp tier wins while a lane holds at most 8 vectors of 16-bit data
        // (16 of FP32); beyond that the resident tier (row unpacked once, packed FP32 math) is faster
        // (BF16 [32768,2048]: resident tier with 128-thread blocks 46.0 us, warp tier 51.8 us; at 1024 columns they tie)
        // short rows: a row does not fill a warp's lanes, or fills them with so little data that per-row costs dominate
        // (BF16 64 columns 1.3 -> 5.5 TB/s, 128: 2.4 -> 5.4, 256: 4.1 -> 5.5, 512: 4.7 -> 5.3; FP32 32 columns 1.9 -> 5.9,
        // 64: 3.5 -> 5.9, 128: 5.5 -> 5.9)
        else if (vec_ok && nvec <= (sizeof(T) == 2 ? 64 : 48)) tier = 9;
        else if (warp_ok && (sizeof(T) == 4 || nvec <= 128)) tier = 1;
        // (16-bit rows of more than 16384 columns would need 1024 threads with 32 unpacked values each and spill:
        // two passes per row with 256-thread blocks instead, BF16 [3276,20480] 2.4 -> 3.6 TB/s)
        else if (nvec <= 1024 * 4 && !(sizeof(T) == 2 && nvec > 512 * 4)) tier = 5;
        // FP32 rows of more than 16384 columns: two passes per row, the second from the L2, measured faster than the
        // row in registers (5.1 against 4.4 TB/s at [4096,20480], 5.1 against 4.8 at [8192,32768]); 16-bit rows of
        // 49153..65536 columns stay in registers (3.9 TB/s either way at [4096,65536])
        else if (nvec > 1024 * 6 && nvec <= 1024 * kMaxVecsPerThread && sizeof(T) == 2) tier = 2;
        // beyond one block's registers: with fewer rows than SMs a cluster spreads each row over several SMs
        else if (nvec > 1024 * kMaxVecsPerThread && a.rows < info.sm_count && nvec <= 8 * 1024 * kMaxVecsPerThread) tier = 6;
        else tier = 8;
    }
    if (tier == 9) {
        KO_REQUIRE(vec_ok && nvec <= 128, KO_ERR_SHAPE, "layernorm: the group tier needs 16-byte aligned rows of at most 128 vectors");
        int g = k.stage_rows;  // lanes per row
        if (g == 0) {
            // few lanes with several vectors each: up to four 16-bit vectors per lane, two FP32 vectors
            const int per_lane = sizeof(T) == 2 ? 4 : 2;
            g = 4;
            while (g < 32 && g * per_lane < nvec) g *= 2;
            // FP32: half the lanes with three vectors each when that holds the row (40 vectors: 16 x 3 instead of 32 x 2,
            // [209715,160] 5.7 -> 6.0 TB/s)
            if (sizeof(T) == 4 && g >= 8 && (g / 2) * 3 >= nvec) g /= 2;
        }
        switch (g) {
            case 4: return launch_group_g<T, 4>(nvec, k.rows_per_warp, a, k.grid_cap, info.sm_count, s);
            case 8: return launch_group_g<T, 8>(nvec, k.rows_per_warp, a, k.grid_cap, info.sm_count, s);
            case 16: return launch_group_g<T, 16>(nvec, k.rows_per_warp, a, k.grid_cap, info.sm_count, s);
            case 32: return launch_group_g<T, 32>(nvec, k.rows_per_warp, a, k.grid_cap, info.sm_count, s);
            default: return ko::fail(KO_ERR_INVALID_ARG, "layernorm: the group tier takes 4, 8, 16 or 32 lanes per row, got %d", g);
        }
    }
    if (tier == 8) {
        KO_REQUIRE(vec_ok, KO_ERR_SHAPE, "layernorm: the reread tier needs 16-byte aligned rows");
        // two rows per block at a time, gamma / beta loaded once for both: measured faster from 512 KB per row
        // (FP32 [512,131072]: 4.1 against 3.6 TB/s; [1024,65536]: 4.2 against 4.5)
        const bool pair = k.rows_per_warp == 2 || (k.rows_per_warp == 0 && (long long)a.cols * (long long)sizeof(T) >= (512ll << 10));
        int block = k.block;
        if (block == 0) {
            if (sizeof(T) == 2) block = nvec <= 1024 * 6 ? 256 : 1024;  // BF16 [1365,49152]: 3.8 TB/s with 256, 3.3 with 1024
            else block = nvec <= 1024 * 5 ? 256 : (nvec <= 1024 * kMaxVecsPerThread ? 512 : 1024);
        }
        // row loads through a shared-memory ring of items (stages: 3 = on, 1 = off, 0 = where it measured faster: rows of
        // 128..256 KB with 1024 threads -- FP32 [1024,65536] 4.3 -> 4.8 TB/s, [4096,65536] 4.6 -> 5.3, BF16 [2048,131072]
        // 4.0 -> 4.2 -- and FP32 rows of 80..128 KB with 512 threads: [1365,24576] 4.4 -> 4.7, [8192,32768] 5.2 -> 5.3)
        const long long row_bytes = (long long)a.cols * (long long)sizeof(T);
        bool ring = k.stages == 3;
        if (k.stages == 0 && k.block == 0 && k.rows_per_warp == 0 && !pair) {
            if (row_bytes > (128ll << 10) && row_bytes <= (256ll << 10)) {
                ring = true;
                block = 1024;
            } else if (sizeof(T) == 4 && row_bytes > (80ll << 10) && row_bytes <= (128ll << 10)) {
                ring = true;
                block = 512;
            }
        }
        if (ring && !pair) {
            constexpr int kU = sizeof(T) == 2 ? 2 : 4;
            if (block == 256) return launch_reread_ring<T, 256, 4, 4>(a, k.grid_cap, info.sm_count, s);
            if (block == 512) return launch_reread_ring<T, 512, kU, 3>(a, k.grid_cap, info.sm_count, s);
            return launch_reread_ring<T, 1024, kU, 3>(a, k.grid_cap, info.sm_count, s);
        }
        if (block == 256) return pair ? launch_reread<T, 256, true>(a, k.grid_cap, info.sm_count, s) : launch_reread<T, 256, false>(a, k.grid_cap, info.sm_count, s);
        if (block == 512) return pair ? launch_reread<T, 512, true>(a, k.grid_cap, info.sm_count, s) : launch_reread<T, 512, false>(a, k.grid_cap, info.sm_count, s);
        return pair ? launch_reread<T, 1024, true>(a, k.grid_cap, info.sm_count, s) : launch_reread<T, 1024, false>(a, k.grid_cap, info.sm_count, s);
    }
    if (tier == 6) {
        KO_REQUIRE(vec_ok, KO_ERR_SHAPE, "layernorm: the cluster tier needs 16-byte aligned rows");
        const int c = ko::cluster_size_for(nvec, 1024 * kMaxVecsPerThread, k.cluster);
        KO_REQUIRE(c > 0, KO_ERR_SHAPE, "layernorm: %d columns exceed what a cluster of 8 blocks holds", a.cols);
        return launch_cluster<T>(a, c, k.stages != 2, k.grid_cap, info.sm_count, s);  // stages = 2: cluster barriers instead of mailboxes
    }
    if (tier == 5) {
        // resident tier: at most 4 vectors per thread
        KO_REQUIRE(vec_ok && nvec <= 1024 * 4, KO_ERR_SHAPE, "layernorm: the resident tier needs 16-byte aligned rows of at most 4096 vectors");
        int threads = k.block;
        if (threads == 0) {
            threads = nvec <= 256 ? 128 : 256;  // two vectors per thread at 2048 and 4096 columns of 16-bit data
            // FP32 rows of 3072..4096 columns: 512 threads with at most two vectors each ([10922,3072] 5.2 -> 5.8 TB/s)
            if (sizeof(T) == 4 && nvec >= 768) threads = 512;
            while (threads < 1024 && nvec > threads * 4) threads *= 2;
            // 2049..3072 vectors: 768 threads with four each instead of 1024 of which a quarter or more hold padding
            // (padded vectors cost as much as real ones) -- FP32 [3472,9216] 4.0 -> 6.0 TB/s, [3125,10240] 4.3 -> 5.7,
            // [2840,11264] 4.4 -> 5.5, [2604,12288] 4.6 -> 5.4; 3073..3584 vectors: 896 threads ([2232,14336] 4.9 -> 5.2)
            if (nvec > 2048 && nvec <= 768 * 4) threads = 768;
            else if (nvec > 768 * 4 && nvec <= 896 * 4) threads = 896;
        }
        KO_REQUIRE(nvec <= threads * 4, KO_ERR_SHAPE, "layernorm: %d threads hold at most %d vectors per row", threads, threads * 4);
        const int per_thread = (nvec + threads - 1) / threads;
        // The next rows of a block in flight into shared memory (cp.async) instead of one row into registers: measured
        // faster whenever the threads are not exactly filled with two vectors each (BF16 [32768,5120] 191 -> 108 us,
        // [32768,3072] 81 -> 66, [32768,8192] 231 -> 187; FP32 [16384,2560] 68 -> 61,
        // [5461,6144] 5.1 -> 5.8 TB/s); with exactly two vectors per thread it measured slower (BF16 [32768,4096] 96 -> 100
        // us, FP32 [16384,4096] 91 -> 95), as it did with four FP32 vectors in 256 threads.  stages: 0 = that rule,
        // 1 = registers, 3 = ring.
        const int held = per_thread <= 1 ? 1 : (per_thread <= 2 ? 2 : 4);  // vectors per thread of the instantiation
        const bool full = nvec == threads * held;
        const bool ring = k.stages == 3 ||
                          (k.stages == 0 && (!full || (held == 4 && (sizeof(T) == 2 || threads >= 512))));
        switch (threads) {
            case 128: return launch_resident_vecs<T, 128>(per_thread, ring, a, k.grid_cap, info.sm_count, s);
            case 256: return launch_resident_vecs<T, 256>(per_thread, ring, a, k.grid_cap, info.sm_count, s);
            case 512: return launch_resident_vecs<T, 512>(per_thread, ring, a, k.grid_cap, info.sm_count, s);
            case 1024: return launch_resident_vecs<T, 1024>(per_thread, ring, a, k.grid_cap, info.sm_count, s);
            // between the powers of two: four vectors per thread, rows through the shared-memory ring
            case 768: return launch_resident_ring<T, 4, 768>(true, a, k.grid_cap, info.sm_count, s);
            case 896: return launch_resident_ring<T, 4, 896>(true, a, k.grid_cap, info.sm_count, s);
            default: return ko::fail(KO_ERR_INVALID_ARG, "layernorm: resident tier needs 128/256/512/768/896/1024 threads, got %d", threads);
        }
    }
    if (tier == 4) {
        KO_REQUIRE(warp_ok, KO_ERR_SHAPE, "layernorm: the staged tier needs 16-byte aligned rows of at most 512 vectors");
        bool used = false;
        if (int st = dispatch_rows<T, true>(vecs, k.rows_per_warp, a, k, info, s, &used)) return st;
        if (used) return KO_OK;
        KO_REQUIRE(k.tier == 0, KO_ERR_SHAPE, "layernorm: the requested staged geometry does not fit in shared memory");
        tier = 1;
    }
    if (tier == 1) {
        KO_REQUIRE(warp_ok, KO_ERR_SHAPE, "layernorm: the warp tier needs 16-byte aligned rows of at most 512 vectors");
        bool used = false;
        return dispatch_rows<T, false>(vecs, k.rows_per_warp, a, k, info, s, &used);
    }
    if (tier == 2) {
        KO_REQUIRE(vec_ok && nvec <= 1024 * kMaxVecsPerThread, KO_ERR_SHAPE,
                   "layernorm: the block tier needs 16-byte aligned rows of at most 8192 vectors");
        // threads per row: aim at 2 vectors per thread unless the caller picks the block size
        int threads = k.block;
        if (threads == 0) {
            threads = 128;
            while (threads < 1024 && nvec > threads * 2) threads *= 2;
        }
        while (threads < 1024 && nvec > threads * kMaxVecsPerThread) threads *= 2;
        const int per_thread = (nvec + threads - 1) / threads;
        // The next rows of a block in flight into shared memory (cp.async) instead of one row into registers: measured
        // faster whenever the threads are not exactly filled with two vectors each (BF16 [32768,5120] 191 -> 108 us,
        // [32768,3072] 81 -> 66, [32768,8192] 231 -> 187; FP32 [16384,2560] 68 -> 61,
        // [5461,6144] 5.1 -> 5.8 TB/s); with exactly two vectors per thread it measured slower (BF16 [32768,4096] 96 -> 100
        // us, FP32 [16384,4096] 91 -> 95), as it did with four FP32 vectors in 256 threads.  stages: 0 = that rule,
        // 1 = registers, 3 = ring.
        const int held = per_thread <= 1 ? 1 : (per_thread <= 2 ? 2 : 4);  // vectors per thread of the instantiation
        const bool full = nvec == threads * held;
        const bool ring = k.stages == 3 ||
                          (k.stages == 0 && (!full || (held == 4 && (sizeof(T) == 2 || threads >= 512))));
        switch (threads) {
            case 128: return launch_block_vecs<T, 128>(per_thread, a, k.grid_cap, s);
            case 256: return launch_block_vecs<T, 256>(per_thread, a, k.grid_cap, s);
            case 512: return launch_block_vecs<T, 512>(per_thread, a, k.grid_cap, s);
            case 1024: return launch_block_vecs<T, 1024>(per_thread, a, k.grid_cap, s);
            default: return ko::fail(KO_ERR_INVALID_ARG, "layernorm: block tier needs 128/256/512/1024 threads, got %d", threads);
        }
    }
    const long long cap = k.grid_cap > 0 ? k.grid_cap : (long long)info.sm_count * 8;
    ko::layernorm_stream_kernel<T><<<ko::clamp_grid(a.rows, cap), 256, 0, s>>>(a.in, a.out, a.rows, a.cols, a.eps, a.gamma,
                                                                             a.beta, a.ddof);
    KO_CHECK_LAUNCH("layernorm_stream_kernel");
    return KO_OK;
}

}  // namespace

extern "C" {

int ko_layernorm_f32_tuned(const float *in, float *out, int64_t rows, int32_t cols, float eps, const float *gamma,
                           const float *beta, int ddof, const ko_row_knobs_t *knobs, void *stream) {
    const Args<float> a{in, out, rows, cols, eps, gamma, beta, ddof};
    return layernorm_dispatch<float>(a, knobs, static_cast<cudaStream_t>(stream));
}

int ko_layernorm_bf16_tuned(const uint16_t *in, uint16_t *out, int64_t rows, int32_t cols, float eps,
                            const uint16_t *gamma, const uint16_t *beta, int ddof, const ko_row_knobs_t *knobs,
                            void *stream) {
    using B = __nv_bfloat16;
    const Args<B> a{reinterpret_cast<const B *>(in), reinterpret_cast<B *>(out), rows, cols, eps,
                    reinterpret_cast<const B *>(gamma), reinterpret_cast<const B *>(beta), ddof};
    return layernorm_dispatch<B>(a, knobs, static_cast<cudaStream_t>(stream));
}

int ko_layernorm_f16_tuned(const uint16_t *in, uint16_t *out, int64_t rows, int32_t cols, float eps,
                           const uint16_t *gamma, const uint16_t *beta, int ddof, const ko_row_knobs_t *knobs,
                           void *stream) {
    using H = __half;
    const Args<H> a{reinterpret_cast<const H *>(in), reinterpret_cast<H *>(out), rows, cols, eps,
                    reinterpret_cast<const H *>(gamma), reinterpret_cast<const H *>(beta), ddof};
    return layernorm_dispatch<H>(a, knobs, static_cast<cudaStream_t>(stream));
}

int ko_layernorm_f32(const float *in, float *out, int64_t rows, int32_t cols, float eps, const float *gamma,
                     const float *beta, int ddof, void *stream) {
    return ko_layernorm_f32_tuned(in, out, rows, cols, eps, gamma, beta, ddof, nullptr, stream);
}

int ko_layernorm_bf16(const uint16_t *in, uint16_t *out, int64_t rows, int32_t cols, float eps, const uint16_t *gamma,
                      const uint16_t *beta, int ddof, void *stream) {
    return ko_layernorm_bf16_tuned(in, out, rows, cols, eps, gamma, beta, ddof, nullptr, stream);
}

int ko_layernorm_f16(const uint16_t *in, uint16_t *out, int64_t rows, int32_t cols, float eps, const uint16_t *gamma,
                     const uint16_t *beta, int ddof, void *stream) {
    return ko_layernorm_f16_tuned(in, out, rows, cols, eps, gamma, beta, ddof, nullptr, stream);
}

}  // extern "C"
