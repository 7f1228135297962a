// C-ABI launcher of the row softmax: picks the tier and the launch geometry from the runtime shape.
#include "row_launch.h"

#include <algorithm>

#include "../nn_operators/softmax/softmax.h"
#include "../nn_operators/softmax/softmax_16bit.h"

namespace {

using ko::DeviceInfo;

template <int kVecs, int kSlots, int G>
int launch_warp(const float *in, float *out, long long rows, int cols, const ko_row_knobs_t &k, cudaStream_t s) {
    constexpr int kRowsPerStep = kSlots * (32 / G);
    const int block = (k.block > 0 && k.block <= 256) ? k.block : 256;
    const long long groups = (rows + kRowsPerStep - 1) / kRowsPerStep;
    const unsigned grid = ko::clamp_grid((groups + block / 32 - 1) / (block / 32), k.grid_cap);
    return ko::launch_overlapped(ko::softmax_warp_kernel<kVecs, kSlots, G>, grid, (unsigned)block, 0, s, in, out, rows, cols);
}

template <int kVecs, int kSlots, int G>
int launch_staged(const float *in, float *out, long long rows, int cols, const ko_row_knobs_t &k,
                  const DeviceInfo &info, cudaStream_t s, bool *used) {
    constexpr int W = ko::kStagedConsumerWarps;
    const ko::StagedPlan plan = ko::plan_staged(rows, (unsigned)cols * 4u, kSlots * (32 / G), k, info);
    *used = plan.ok;
    if (!plan.ok) return KO_OK;
    unsigned *status = nullptr;
    if (int st = ko::device_status_word(1, &status)) return st;
    auto kernel = ko::softmax_staged_kernel<kVecs, kSlots, G, W>;
    if (int st = ko::ensure_dynamic_smem(reinterpret_cast<const void *>(kernel), plan.smem_bytes)) return st;
    kernel<<<plan.grid, ko::kStagedThreads, plan.smem_bytes, s>>>(in, out, rows, cols, plan.geo, status);
    KO_CHECK_LAUNCH("softmax_staged_kernel");
    return KO_OK;
}

template <int kVecs, int kThreads>
int launch_block(const float *in, float *out, long long rows, int cols, long long grid_cap, cudaStream_t s) {
    return ko::launch_overlapped(ko::softmax_block_kernel<kVecs, kThreads>, ko::clamp_grid(rows, grid_cap), kThreads, 0, s, in, out,
                                 rows, cols);
}
// the same kernel (compiled for up to kBound threads; it reads its block size at run time) with `threads` per block
template <int kVecs, int kBound>
int launch_block_threads(int threads, const float *in, float *out, long long rows, int cols, long long grid_cap, cudaStream_t s) {
    return ko::launch_overlapped(ko::softmax_block_kernel<kVecs, kBound>, ko::clamp_grid(rows, grid_cap), (unsigned)threads, 0, s, in, out,
                                 rows, cols);
}

// one row per block in registers, the next row prefetched into shared memory by a bulk copy; one block per SM
template <int kVecs, int kThreads>
int launch_block_prefetch(const float *in, float *out, long long rows, int cols, long long grid_cap, int sm_count, cudaStream_t s) {
    unsigned *status = nullptr;
    if (int st = ko::device_status_word(1, &status)) return st;
    auto kernel = ko::softmax_block_prefetch_kernel<kVecs, kThreads>;
    const size_t smem = (size_t)cols * 4;
    if (int st = ko::ensure_dynamic_smem(reinterpret_cast<const void *>(kernel), smem)) return st;
    const int per_sm = smem <= 100 * 1024 && kThreads <= 512 ? 2 : 1;
    const long long cap = grid_cap > 0 ? grid_cap : (long long)sm_count * per_sm;
    return ko::launch_overlapped(kernel, ko::clamp_grid(rows, cap), (unsigned)kThreads, smem, s, in, out, rows, cols, status);
}

// one row per block, read twice (the second time from the L2); blocks per SM: as many as fit, fewer when the rows in
// flight would not fit in `l2_budget` bytes
template <int kThreads>
int launch_reread(const float *in, float *out, long long rows, int cols, long long grid_cap, int sm_count, cudaStream_t s) {
    auto kernel = ko::softmax_reread_kernel<4, kThreads>;
    long long cap = grid_cap;
    if (cap <= 0) {
        int per_sm = 0;
        KO_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, 0));
        const long long l2_budget = 80ll << 20;
        const long long fit = l2_budget / ((long long)cols * 4 * sm_count);
        cap = (long long)sm_count * std::max(1ll, std::min<long long>(per_sm, fit));
    }
    return ko::launch_overlapped(kernel, ko::clamp_grid(rows, cap), (unsigned)kThreads, 0, s, in, out, rows, cols);
}

// the reread tier with every load through a per-thread shared-memory ring of kDepth items
template <int kThreads, int kUnroll, int kDepth>
int launch_reread_ring(const float *in, float *out, long long rows, int cols, long long grid_cap, int sm_count, cudaStream_t s) {
    auto kernel = ko::softmax_reread_ring_kernel<kUnroll, kThreads, kDepth>;
    constexpr size_t kBytes = (size_t)kDepth * kUnroll * kThreads * 16;
    if (int st = ko::ensure_dynamic_smem(reinterpret_cast<const void *>(kernel), kBytes)) return st;
    long long cap = grid_cap;
    if (cap <= 0) {
        int per_sm = 0;
        KO_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, kBytes));
        const long long fit = (80ll << 20) / ((long long)cols * 4 * sm_count);
        cap = (long long)sm_count * std::max(1ll, std::min<long long>(per_sm, fit));
    }
    return ko::launch_overlapped(kernel, ko::clamp_grid(rows, cap), (unsigned)kThreads, kBytes, s, in, out, rows, cols);
}

// one row per cluster of `c` blocks; a block holds up to 8 vectors per thread.  256-thread blocks when the slice
// allows: several clusters (rows) then share an SM and one row's reductions and cluster barriers overlap another's
// loads, which a single 1024-thread block per SM cannot do.  threads: 0 = choose, 256 or 1024.
int launch_cluster(const float *in, float *out, long long rows, int cols, int c, int threads, bool prefetch, bool mailbox,
                   long long grid_cap, int sm_count, cudaStream_t s) {
    const int slice = (cols / 4 + c - 1) / c;
    if (threads == 0) threads = slice <= 256 * 8 ? 256 : (slice <= 512 * 8 ? 512 : 1024);
    KO_REQUIRE((threads == 256 || threads == 512 || threads == 1024) && slice <= threads * 8, KO_ERR_SHAPE,
               "softmax: a cluster of %d blocks of %d threads holds at most %d columns", c, threads, c * threads * 32);
    const bool use_prefetch = prefetch && threads == 1024 && slice > 1024 * 4;
    const size_t smem = use_prefetch ? (size_t)slice * 16 : 0;
    // clusters that can be resident at once: a cluster lives inside one GPC, so this can be fewer than SMs / c;
    // more clusters than that would run as a second wave behind grid-stride loops that already cover every row
    const void *probe = use_prefetch ? reinterpret_cast<const void *>(ko::softmax_cluster_prefetch_kernel<8, 1024>)
                        : threads == 1024 ? reinterpret_cast<const void *>(ko::softmax_cluster_kernel<8, 1024>)
                        : threads == 512  ? reinterpret_cast<const void *>(ko::softmax_cluster_kernel<8, 512>)
                                          : reinterpret_cast<const void *>(ko::softmax_cluster_kernel<8, 256>);
    if (smem) {
        if (int st = ko::ensure_dynamic_smem(probe, smem)) return st;
    }
    int resident = 0;
    if (int st = ko::max_resident_clusters(probe, (unsigned)threads, (unsigned)c, smem, &resident)) return st;
    long long clusters = rows;
    const long long cap = grid_cap > 0 ? grid_cap / c : (long long)resident;
    if (clusters > cap) clusters = cap > 0 ? cap : 1;
    const unsigned grid = (unsigned)(clusters * c);
    if (threads == 256) {
        if (slice <= 256 * 4) return ko::launch_clustered(ko::softmax_cluster_kernel<4, 256>, grid, 256, c, s, in, out, rows, cols);
        return ko::launch_clustered(ko::softmax_cluster_kernel<8, 256>, grid, 256, c, s, in, out, rows, cols);
    }
    if (threads == 512) return ko::launch_clustered(ko::softmax_cluster_kernel<8, 512>, grid, 512, c, s, in, out, rows, cols);
    if (slice <= 1024 * 4) return ko::launch_clustered(ko::softmax_cluster_kernel<4, 1024>, grid, 1024, c, s, in, out, rows, cols);
    if (use_prefetch) {
        // one 1024-thread block per SM: the slice of the next row is prefetched into shared memory meanwhile
        unsigned *status = nullptr;
        if (int st = ko::device_status_word(1, &status)) return st;
        return ko::launch_clustered_smem(ko::softmax_cluster_prefetch_kernel<8, 1024>, grid, 1024, c, smem, s, in, out, rows, cols, status,
                                         mailbox ? 1 : 0);
    }
    return ko::launch_clustered(ko::softmax_cluster_kernel<8, 1024>, grid, 1024, c, s, in, out, rows, cols);
}

// lanes per row and vectors per lane depend on the column count only; `slots` (rows a warp handles
// together = slots * 32/G) is the tunable
template <bool kStaged>
int dispatch_rows(int nvec, int slots, const float *in, float *out, long long rows, int cols, const ko_row_knobs_t &k,
                  const DeviceInfo &info, cudaStream_t s, bool *used) {
#define KO_GO(V, R, G)                                                                       \
    do {                                                                                     \
        if constexpr (kStaged) return launch_staged<V, R, G>(in, out, rows, cols, k, info, s, used); \
        else { *used = true; return launch_warp<V, R, G>(in, out, rows, cols, k, s); }       \
    } while (0)
#define KO_SLOTS(V, G, DEF)                          \
    do {                                             \
        const int want = slots > 0 ? slots : (DEF);  \
        if (want <= 1) KO_GO(V, 1, G);               \
        if (want == 2) KO_GO(V, 2, G);               \
        KO_GO(V, 4, G);                              \
    } while (0)
    if (nvec <= 8) KO_SLOTS(1, 8, 4);
    if (nvec <= 16) KO_SLOTS(2, 8, 2);
    if (nvec <= 32) KO_SLOTS(4, 8, 2);
    if (nvec <= 64) KO_SLOTS(4, 16, 2);
    if (nvec <= 128) KO_SLOTS(4, 32, 2);
    if (nvec <= 192) { if (slots == 2) KO_GO(6, 2, 32); KO_GO(6, 1, 32); }
    if (nvec <= 256) { if (slots == 2) KO_GO(8, 2, 32); KO_GO(8, 1, 32); }
    if (nvec <= 384) KO_GO(12, 1, 32);
    KO_GO(16, 1, 32);
#undef KO_SLOTS
#undef KO_GO
}

// FP16 / BF16 rows: warp tier up to 1536 columns, block tier up to 24576, two passes per row beyond; scalar
// stream tier for rows that cannot be moved in 16-byte vectors
template <typename T>
int softmax16_dispatch(const T *in, T *out, int64_t rows, int32_t cols, cudaStream_t s) {
    KO_REQUIRE(rows >= 0 && cols >= 0, KO_ERR_INVALID_ARG, "softmax: negative shape [%lld, %d]", (long long)rows, cols);
    if (rows == 0 || cols == 0) return KO_OK;
    KO_REQUIRE(in != nullptr && out != nullptr, KO_ERR_INVALID_ARG, "softmax: NULL pointer");
    DeviceInfo info;
    if (int st = ko::current_device_info(&info)) return st;
    const bool vec_ok = (cols % 8 == 0) && ko::aligned16(in) && ko::aligned16(out);
    const int nvec = cols / 8;
    if (vec_ok && nvec <= 32 * 8) {
        auto warp = [&](auto kernel, int rows_per_step) -> int {
            const long long groups = (rows + rows_per_step - 1) / rows_per_step;
            return ko::launch_overlapped(kernel, ko::clamp_grid((groups + 7) / 8, 0), 256, 0, s, in, out, (long long)rows, (int)cols);
        };
        // the smallest lane group x vectors per lane that holds the row: padded vectors cost as much as real ones
        // (BF16 768 columns: 4 vectors per lane 4.8 TB/s, 3 vectors per lane 5.5; 1280 columns: 8 vectors 4.5, 5 vectors 6.4)
        if (nvec <= 8) return warp(ko::softmax16_warp_kernel<T, 1, 2, 8>, 8);
        if (nvec <= 16) return warp(ko::softmax16_warp_kernel<T, 2, 1, 8>, 4);   // one row slot per lane group: FP16 [196608,128] 5.3 -> 5.6 TB/s
        if (nvec <= 24) return warp(ko::softmax16_warp_kernel<T, 3, 1, 8>, 4);
        if (nvec <= 32) return warp(ko::softmax16_warp_kernel<T, 2, 1, 16>, 2);  // [196608,256] 5.7 -> 6.0
        if (nvec <= 48) return warp(ko::softmax16_warp_kernel<T, 3, 1, 16>, 2);
        if (nvec <= 64) return warp(ko::softmax16_warp_kernel<T, 2, 1, 32>, 1);
        if (nvec <= 96) return warp(ko::softmax16_warp_kernel<T, 3, 1, 32>, 1);
        if (nvec <= 128) return warp(ko::softmax16_warp_kernel<T, 4, 1, 32>, 1);
        if (nvec <= 160) return warp(ko::softmax16_warp_kernel<T, 5, 1, 32>, 1);
        if (nvec <= 192) return warp(ko::softmax16_warp_kernel<T, 6, 1, 32>, 1);
    }
    if (vec_ok && nvec <= 128 * 2)
        return ko::launch_overlapped(ko::softmax16_block_kernel<T, 2, 128>, ko::clamp_grid(rows, 0), 128u, 0, s, in, out, (long long)rows,
                                     (int)cols);
    if (vec_ok && nvec <= 512 * 6) {
        // Block tier up to 24576 columns: six vectors per thread (three up to 3072 columns) and exactly the threads the
        // row needs, a multiple of 32 -- padded vectors cost as much as real ones, and six vectors in few threads beat
        // four in many.  BF16, TB/s, against the former power-of-two blocks of 4..6 vectors: 2304 columns 5.5 -> 6.6,
        // 7168 5.6 -> 6.4, 9216 5.3 -> 6.5, 11264 5.6 -> 6.4, 13312 4.5 -> 5.8, 15360 4.9 -> 6.1; and instead of the
        // two-pass tier: 18432 4.5 -> 5.5, 24576 5.0 -> 5.9.
        const int per = nvec <= 384 ? 3 : 6;
        const unsigned threads = (unsigned)(((nvec + per - 1) / per + 31) / 32 * 32);
        if (per == 3)
            return ko::launch_overlapped(ko::softmax16_block_kernel<T, 3, 512>, ko::clamp_grid(rows, 0), threads, 0, s, in, out, (long long)rows, (int)cols);
        return ko::launch_overlapped(ko::softmax16_block_kernel<T, 6, 512>, ko::clamp_grid(rows, 0), threads, 0, s, in, out, (long long)rows, (int)cols);
    }
    if (vec_ok) {
        // beyond 24576 columns: two passes per row, the second from the L2, in 256-thread blocks so that several rows
        // per SM are in flight ([2048,32768] 3.8 -> 4.8 TB/s against a 1024-thread block
        // holding the row; [1024,65536] 4.2 -> 4.5 against one 1024-thread reread block per SM)
        // while at least four rows per SM fit in the L2 besides the output stream; longer rows: one 1024-thread block per
        // SM (BF16 [2048,131072]: 4.6 TB/s; 3.3 with two 256-thread blocks per SM, 4.2 with eight that overflow the L2)
        const long long fit = (80ll << 20) / ((long long)cols * 2);
        if (fit >= 4ll * info.sm_count) {
            auto kernel = ko::softmax16_reread_kernel<T, 4, 256>;
            int per_sm = 1;
            KO_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, 256, 0));
            const long long cap = std::min<long long>((long long)info.sm_count * (per_sm > 0 ? per_sm : 1), fit);
            return ko::launch_overlapped(kernel, ko::clamp_grid(rows, cap), 256u, 0, s, in, out, (long long)rows, (int)cols);
        }
        auto kernel = ko::softmax16_reread_kernel<T, 2, 1024>;
        return ko::launch_overlapped(kernel, ko::clamp_grid(rows, info.sm_count), 1024u, 0, s, in, out, (long long)rows, (int)cols);
    }
    ko::softmax16_stream_kernel<T><<<ko::clamp_grid(rows, (long long)info.sm_count * 8), 256, 0, s>>>(in, out, rows, cols);
    KO_CHECK_LAUNCH("softmax16_stream_kernel");
    return KO_OK;
}

}  // namespace

extern "C" {

int ko_softmax_f16(const uint16_t *in, uint16_t *out, int64_t rows, int32_t cols, void *stream) {
    return softmax16_dispatch(reinterpret_cast<const __half *>(in), reinterpret_cast<__half *>(out), rows, cols,
                              static_cast<cudaStream_t>(stream));
}

int ko_softmax_bf16(const uint16_t *in, uint16_t *out, int64_t rows, int32_t cols, void *stream) {
    return softmax16_dispatch(reinterpret_cast<const __nv_bfloat16 *>(in), reinterpret_cast<__nv_bfloat16 *>(out), rows, cols,
                              static_cast<cudaStream_t>(stream));
}

int ko_softmax_f32_tuned(const float *in, float *out, int64_t rows, int32_t cols, const ko_row_knobs_t *knobs,
                         void *stream) {
    KO_REQUIRE(rows >= 0 && cols >= 0, KO_ERR_INVALID_ARG, "softmax: negative shape [%lld, %d]", (long long)rows, cols);
    if (rows == 0 || cols == 0) return KO_OK;
    KO_REQUIRE(in != nullptr && out != nullptr, KO_ERR_INVALID_ARG, "softmax: NULL pointer");
    const ko_row_knobs_t k = knobs ? *knobs : ko_row_knobs_t{};
    KO_REQUIRE((k.tier >= 0 && k.tier <= 4) || (k.tier >= 6 && k.tier <= 8), KO_ERR_INVALID_ARG, "softmax: unknown tier %d", k.tier);
    KO_REQUIRE(k.cluster == 0 || k.cluster == 2 || k.cluster == 4 || k.cluster == 8, KO_ERR_INVALID_ARG,
               "softmax: cluster size %d not in {2,4,8}", k.cluster);
    KO_REQUIRE(k.block >= 0 && (k.block % 32 == 0 || k.block == 1) && k.block <= 1024, KO_ERR_INVALID_ARG,
               "softmax: block %d must be a multiple of 32, <= 1024", k.block);
    DeviceInfo info;
    if (int st = ko::current_device_info(&info)) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool vec_ok = (cols % 4 == 0) && ko::aligned16(in) && ko::aligned16(out);
    const int nvec = cols / 4;

    int tier = k.tier;
    if (tier == 0) {
        if (!vec_ok) tier = 3;
        else if (nvec <= 32 * 16) tier = 1;  // measured faster than the staged tier at every benchmark shape
        else if (nvec <= 1024 * 4) tier = 2;
        else if (nvec <= 1024 * 8) tier = 7;  // beyond 16384 columns one block per SM: prefetch the next row (5.8 vs 4.4 TB/s at 32768)
        // beyond one block's registers: with fewer rows than SMs a cluster spreads each row over several SMs; otherwise
        // one block per row in two passes, the second from the L2 (5.2 against 4.2 TB/s at [1024,65536], 4.5 against
        // 3.5 TB/s at [256,262144]; rows of any length)
        else if (rows < info.sm_count && nvec <= 8 * 1024 * 8) tier = 6;
        else tier = 8;
    }
    if (tier == 8) {
        KO_REQUIRE(vec_ok, KO_ERR_SHAPE, "softmax: the reread tier needs cols %% 4 == 0 and 16-byte aligned pointers");
        // loads through a shared-memory ring of items (stages: 3 = on, 1 = off, 0 = on for rows of at most 256 KB, where it
        // measured faster: [1024,65536] 5.3 -> 5.7 TB/s, [4096,65536] 5.5 -> 6.1; beyond, the items fetched ahead across
        // the end of a row compete for the L2 with the rows being re-read: [2048,131072] 5.2 either way)
        if (k.stages == 3 || (k.stages == 0 && k.block == 0 && (long long)cols * 4 <= (256ll << 10))) {
            if (k.block == 256) return launch_reread_ring<256, 4, 4>(in, out, rows, cols, k.grid_cap, info.sm_count, s);
            if (k.block == 512) return launch_reread_ring<512, 4, 3>(in, out, rows, cols, k.grid_cap, info.sm_count, s);
            if (k.rows_per_warp == 2) return launch_reread_ring<1024, 2, 4>(in, out, rows, cols, k.grid_cap, info.sm_count, s);
            return launch_reread_ring<1024, 4, 3>(in, out, rows, cols, k.grid_cap, info.sm_count, s);
        }
        if (k.block == 256) return launch_reread<256>(in, out, rows, cols, k.grid_cap, info.sm_count, s);
        if (k.block == 512) return launch_reread<512>(in, out, rows, cols, k.grid_cap, info.sm_count, s);
        return launch_reread<1024>(in, out, rows, cols, k.grid_cap, info.sm_count, s);
    }
    if (tier == 6) {
        KO_REQUIRE(vec_ok, KO_ERR_SHAPE, "softmax: the cluster tier needs cols %% 4 == 0 and 16-byte aligned pointers");
        // the smallest cluster that holds the row (larger clusters measured slower: every row costs two cluster barriers)
        const int c = ko::cluster_size_for(nvec, 1024 * 8, k.cluster);  // k.cluster: where the search starts
        KO_REQUIRE(c > 0 && (nvec + c - 1) / c <= 1024 * 8, KO_ERR_SHAPE, "softmax: %d columns exceed what a cluster of %d blocks holds", cols, c ? c : 8);
        const int threads = (k.block == 256 || k.block == 512 || k.block == 1024) ? k.block : 0;
        // stages = 1: no prefetch; stages = 2: prefetch, partials exchanged with cluster barriers instead of mailboxes
        return launch_cluster(in, out, rows, cols, c, threads, k.stages != 1, k.stages != 2, k.grid_cap, info.sm_count, s);
    }
    if (tier == 4) {
        KO_REQUIRE(vec_ok && nvec <= 32 * 16, KO_ERR_SHAPE, "softmax: the staged tier needs cols %% 4 == 0, cols <= 2048 and 16-byte aligned pointers");
        bool used = false;
        if (int st = dispatch_rows<true>(nvec, k.rows_per_warp, in, out, rows, cols, k, info, s, &used)) return st;
        if (used) return KO_OK;
        KO_REQUIRE(k.tier == 0, KO_ERR_SHAPE, "softmax: the requested staged geometry does not fit in shared memory");
        tier = 1;
    }
    if (tier == 1) {
        KO_REQUIRE(vec_ok && nvec <= 32 * 16, KO_ERR_SHAPE, "softmax: the warp tier needs cols %% 4 == 0, cols <= 2048 and 16-byte aligned pointers");
        bool used = false;
        return dispatch_rows<false>(nvec, k.rows_per_warp, in, out, rows, cols, k, info, s, &used);
    }
    if (tier == 7) {
        KO_REQUIRE(vec_ok && nvec > 0 && nvec <= 1024 * 8, KO_ERR_SHAPE,
                   "softmax: the prefetching block tier needs cols %% 4 == 0, cols <= 32768 and 16-byte aligned pointers");
        if (nvec <= 512 * 4) return launch_block_prefetch<4, 512>(in, out, rows, cols, k.grid_cap, info.sm_count, s);
        if (nvec <= 1024 * 4) return launch_block_prefetch<4, 1024>(in, out, rows, cols, k.grid_cap, info.sm_count, s);
        if (nvec <= 1024 * 5) return launch_block_prefetch<5, 1024>(in, out, rows, cols, k.grid_cap, info.sm_count, s);
        if (nvec <= 1024 * 6) return launch_block_prefetch<6, 1024>(in, out, rows, cols, k.grid_cap, info.sm_count, s);
        return launch_block_prefetch<8, 1024>(in, out, rows, cols, k.grid_cap, info.sm_count, s);
    }
    if (tier == 2) {
        KO_REQUIRE(vec_ok && nvec <= 1024 * 8, KO_ERR_SHAPE, "softmax: the block tier needs cols %% 4 == 0, cols <= 32768 and 16-byte aligned pointers");
        // three vectors per thread for 2049..3072 columns ([13107,2560] 5.7 -> 6.2 TB/s); five or six vectors in 256 or
        // 512 threads measured slower than four in twice the threads ([6553,5120] 5.4 against 5.6, [3276,10240] 4.7 / 5.4)
        // The block has as many threads as the row needs with four vectors each, a multiple of 32:
        // padded vectors cost as much as real ones ([8184,4100] 5.0 -> 6.0 TB/s, [6553,5120] 5.7 -> 6.6, [3640,9216]
        // 5.2 -> 5.7, [3276,10240] 5.5 -> 6.0; k.block = 1: powers of two only, for comparison)
        // (up to 4096 columns the 256-thread blocks of three or four vectors stay where they are filled to 88 % or more:
        // [10922,3072] 6.63 against 6.51 TB/s, [8192,4096] 6.61 / 6.51; [16352,2052] 5.7 -> 6.5 with 160 threads)
        const int pow2_slots = nvec <= 256 * 3 ? 256 * 3 : 256 * 4;
        const bool exact = k.block != 1 && (nvec > 256 * 4 || nvec * 100 < pow2_slots * 88);
        if (exact && nvec <= 1024 * 4) return launch_block_threads<4, 1024>(((nvec + 3) / 4 + 31) / 32 * 32, in, out, rows, cols, k.grid_cap, s);
        if (nvec <= 256 * 3) return launch_block<3, 256>(in, out, rows, cols, k.grid_cap, s);
        if (nvec <= 256 * 4) return launch_block<4, 256>(in, out, rows, cols, k.grid_cap, s);
        if (nvec <= 512 * 4) return launch_block<4, 512>(in, out, rows, cols, k.grid_cap, s);
        if (nvec <= 1024 * 4) return launch_block<4, 1024>(in, out, rows, cols, k.grid_cap, s);
        return launch_block<8, 1024>(in, out, rows, cols, k.grid_cap, s);
    }
    const long long cap = k.grid_cap > 0 ? k.grid_cap : (long long)info.sm_count * 8;
    ko::softmax_stream_kernel<<<ko::clamp_grid(rows, cap), 256, 0, s>>>(in, out, rows, cols);
    KO_CHECK_LAUNCH("softmax_stream_kernel");
    return KO_OK;
}

int ko_softmax_f32(const float *in, float *out, int64_t rows, int32_t cols, void *stream) {
    return ko_softmax_f32_tuned(in, out, rows, cols, nullptr, stream);
}

}  // extern "C"
