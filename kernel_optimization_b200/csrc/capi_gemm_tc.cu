// C-ABI launchers of the tcgen05 tensor-core GEMM: build the TMA descriptors, pick the tile width,
// launch one persistent CTA per SM.
#include "ko_context.h"
#include "ko_internal.h"
#include "../../include/ko_b200_tuning.h"
#include "row_launch.h"

#include <algorithm>
#include <mutex>

#include <cudaTypedefs.h>

#include "../nn_operators/gemm/tensor_core_gemm.h"
#include "../nn_operators/gemm/tensor_core_gemm_pair.h"

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int get_encode_fn(EncodeTiledFn *out) {
    static std::mutex mu;
    static EncodeTiledFn cached = nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!cached) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        KO_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        KO_REQUIRE(qres == cudaDriverEntryPointSuccess && fn != nullptr, KO_ERR_CUDA,
                   "cuTensorMapEncodeTiled is not available from this driver");
        cached = reinterpret_cast<EncodeTiledFn>(fn);
    }
    *out = cached;
    return KO_OK;
}

// 2-D map over a K-contiguous 16-bit matrix [rows, K]; box = 64 (K) x box_rows, 128-byte swizzle,
// out-of-range elements read as zero
int make_map(EncodeTiledFn encode, CUtensorMap *map, int fmt, const void *base, int64_t rows, int64_t K, int box_rows) {
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)ko::tc::kBK, (cuuint32_t)box_rows};
    const cuuint32_t elem_strides[2] = {1, 1};
    const CUtensorMapDataType dt = fmt == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const CUresult r = encode(map, dt, 2, const_cast<void *>(base), dims, strides, box, elem_strides,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    KO_REQUIRE(r == CUDA_SUCCESS, KO_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return KO_OK;
}

// 2-D map over a row-major 16-bit B[K, N] (N contiguous); box = 64 columns x 64 K-rows, 128-byte swizzle
int make_map_b_row_major(EncodeTiledFn encode, CUtensorMap *map, int fmt, const void *base, int64_t K, int64_t N) {
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)K};
    const cuuint64_t strides[1] = {(cuuint64_t)N * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)ko::tc::kBK};
    const cuuint32_t elem_strides[2] = {1, 1};
    const CUtensorMapDataType dt = fmt == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const CUresult r = encode(map, dt, 2, const_cast<void *>(base), dims, strides, box, elem_strides,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    KO_REQUIRE(r == CUDA_SUCCESS, KO_ERR_CUDA, "cuTensorMapEncodeTiled (row-major B) failed with CUresult %d", (int)r);
    return KO_OK;
}

template <int BN, bool kTmaStore, int MT = 1, int kBoxes = 2>
int launch(const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &mb_narrow, const CUtensorMap &md,
           const ko::tc::GemmParams &p, int sm_count, cudaStream_t s) {
    using Cfg = ko::tc::TileConfig<BN, MT, kBoxes>;
    auto kernel = ko::tc::gemm_tcgen05_kernel<BN, kTmaStore, MT, kBoxes>;
    if (int st = ko::ensure_dynamic_smem(reinterpret_cast<const void *>(kernel), Cfg::kSmemBytes)) return st;
    const long long tiles_n = p.tiles_n ? p.tiles_n : (p.N + BN - 1) / BN;
    const long long units = (long long)((p.M + MT * ko::tc::kBM - 1) / (MT * ko::tc::kBM)) * tiles_n * (p.split_k > 1 ? p.split_k : 1);
    const unsigned grid = (unsigned)(units < sm_count ? units : sm_count);
    return ko::launch_overlapped(kernel, grid, (unsigned)ko::tc::kThreads, (size_t)Cfg::kSmemBytes, s, ma, mb, mb_narrow, md, p);
}

// The two-SM kernel: clusters of two CTAs, one 256 x BN tile per cluster at a time, as many clusters as the device
// holds at once (a cluster lives inside one GPC, so that can be fewer than SMs / 2).
template <bool kTmaStore>
int launch_pair(const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &mb_narrow, const CUtensorMap &md,
                const ko::tc::GemmParams &p, int resident_pairs, cudaStream_t s) {
    using Cfg = ko::tc::PairConfig;
    auto kernel = ko::tc::gemm_tcgen05_pair_kernel<kTmaStore>;
    const long long tiles_n = p.tiles_n ? p.tiles_n : (p.N + Cfg::kBN - 1) / Cfg::kBN;
    const long long tiles = (long long)((p.M + 2 * ko::tc::kBM - 1) / (2 * ko::tc::kBM)) * tiles_n;
    const unsigned pairs = (unsigned)(tiles < resident_pairs ? tiles : resident_pairs);
    return ko::launch_clustered_overlapped(kernel, 2 * pairs, (unsigned)ko::tc::kThreads, 2, (size_t)Cfg::kSmemBytes, s, ma, mb,
                                           mb_narrow, md, p);
}

// clusters of two CTAs of the pair kernel the current device holds at once (cached per device)
int resident_pairs(int *out) {
    static std::mutex mu;
    static int cached[64] = {};
    int dev = 0;
    KO_CUDA(cudaGetDevice(&dev));
    KO_REQUIRE(dev >= 0 && dev < 64, KO_ERR_NO_DEVICE, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == 0) {
        using Cfg = ko::tc::PairConfig;
        for (const void *k : {reinterpret_cast<const void *>(ko::tc::gemm_tcgen05_pair_kernel<true>),
                              reinterpret_cast<const void *>(ko::tc::gemm_tcgen05_pair_kernel<false>)})
            if (int st = ko::ensure_dynamic_smem(k, Cfg::kSmemBytes)) return st;
        int n = 0;
        if (int st = ko::max_resident_clusters(reinterpret_cast<const void *>(ko::tc::gemm_tcgen05_pair_kernel<true>), ko::tc::kThreads, 2,
                                               Cfg::kSmemBytes, &n))
            return st;
        cached[dev] = n;
    }
    *out = cached[dev];
    return KO_OK;
}

// Uneven column tiles.  With every tile bn_max columns wide, tiles_m * ceil(N / bn_max) tiles run as whole rounds of
// `slots` CTAs and the last round may be mostly empty (4096^3 with 256 x 256 tiles: 256 tiles on 148 CTAs, the second
// round 73 % full).  Cutting N into a few more, slightly narrower tiles (widths multiples of 32, the first
// `wide_tiles_n` one step wider than the rest) fills the rounds: 17 column tiles (9 of 256, 8 of 224) make 272 tiles
// whose second round holds only 224-wide ones -- 480 tile-columns per CTA instead of 512 (measured 98.9 against
// 102.3 us).  Cost model: a round takes as long as its widest tile (wide tiles are dealt first, ko::tc::tile_of); a
// tile takes the longer of its MMAs (rows x width) and of bringing its operands into shared memory (rows + width,
// scaled so that the 128 x 256 tile is operand-bound at 0.87 of the MMA rate, as measured on long K) -- narrower
// tiles move more operand bytes per MMA, which is why the FFN shape keeps its 12 equal column tiles (15 uneven
// ones measured 85.2 against 78.8 us).
struct ColumnPlan {
    int tiles_n = 0, wide_tiles_n = 0, bn_wide = 0, bn_narrow = 0;  // tiles_n == 0: uniform
};
// pair: the tile is computed by two CTAs, each with half the rows and half the B columns to load
// The 256-row tiles (one CTA or a pair) run at the rate their operands arrive even at full width -- measured: a tile
// of 256 x 168 columns takes 0.83 of the time of 256 x 256, i.e. (256 + 168) / (256 + 256) and not 168 / 256 -- so their
// cost is rows + width; a narrower tile saves less than its width suggests (8192 x 3072 x 4096: 18 column tiles of
// 192 / 160 columns took 173 us against 157 us for 12 of 256).
double tile_cost(int rows, int width, bool pair) {
    const double mma = (double)(pair ? rows / 2 : rows) * width;
    const double per_unit = rows >= 256 ? 128.0 : 128.0 * 256.0 / 0.87 / 384.0;
    const double operands = per_unit * (pair ? rows / 2 + width / 2 : rows + width);
    return mma > operands ? mma : operands;
}
// force: the cheapest uneven plan even when the uniform one is modelled cheaper (the tuning codes that ask for one)
ColumnPlan plan_columns(long long M, long long N, int tile_m, int bn_max, int slots, bool pair, bool force) {
    ColumnPlan best;
    const long long tiles_m = (M + tile_m - 1) / tile_m;
    const long long uniform_n = (N + bn_max - 1) / bn_max;
    const long long uniform_rounds = (tiles_m * uniform_n + slots - 1) / slots;
    double best_cost = force ? 1e300 : (double)uniform_rounds * tile_cost(tile_m, bn_max, pair);
    if (tiles_m * uniform_n <= slots) return best;  // a single, partly filled round: nothing to even out
    const long long units = (N + 31) / 32;
    for (long long tn = uniform_n + 1; tn <= 2 * uniform_n; ++tn) {
        const long long narrow_u = units / tn, extra = units % tn;
        if (narrow_u * 32 < bn_max / 2) break;
        const int narrow = (int)narrow_u * 32, wide = extra ? narrow + 32 : narrow;
        if (wide > bn_max) continue;
        const long long total = tiles_m * tn, wide_total = tiles_m * extra;
        double cost = 0.0;
        for (long long r = 0; r * slots < total; ++r) cost += tile_cost(tile_m, (r * slots < wide_total) ? wide : narrow, pair);
        if (cost < 0.97 * best_cost) {  // worth a new shape only for a clear gain
            best_cost = cost;
            best.tiles_n = (int)tn;
            best.wide_tiles_n = (int)extra;
            best.bn_wide = wide;
            best.bn_narrow = narrow;
        }
    }
    return best;
}

// [M, N] row-major output, boxes of 32 rows x 32 columns: FP32 rows of 128 bytes with the 128-byte swizzle,
// 16-bit rows of 64 bytes with the 64-byte swizzle
int make_store_map(EncodeTiledFn encode, CUtensorMap *map, int out_fmt, void *D, int64_t M, int64_t N) {
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)N * (out_fmt == 0 ? 4 : 2)};
    const cuuint32_t box[2] = {32, 32};
    const cuuint32_t elem_strides[2] = {1, 1};
    const CUtensorMapDataType dt = out_fmt == 0   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                   : out_fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                  : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const CUresult r = encode(map, dt, 2, D, dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              out_fmt == 0 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    KO_REQUIRE(r == CUDA_SUCCESS, KO_ERR_CUDA, "cuTensorMapEncodeTiled (D) failed with CUresult %d", (int)r);
    return KO_OK;
}

double wave_efficiency(long long M, long long N, int bn, int sm_count, int bm = 128) {
    const long long tiles = ((M + bm - 1) / bm) * ((N + bn - 1) / bn);
    const long long waves = (tiles + sm_count - 1) / sm_count;
    return (double)(M * N) / (double)(waves * sm_count * (long long)bm * bn);
}

// fmt: A and B, 0 = F16, 1 = BF16; out_fmt: D and C, 0 = FP32, 1 = F16, 2 = BF16; b_row_major: 0 = B[K,N]
// column-major (K contiguous), 1 = row-major (N contiguous);
// bn: 0 = choose; 64 / 128 / 256 = columns per 128-row tile; 512 = the 256 x 256 tile of one CTA (two 128-row halves
// share every B tile); 1024 / 1280 = the 128- / 256-row tile with uneven column tiles forced; 2048 / 2304 = the
// two-SM kernel (256 x 256 tile per pair of CTAs) with equal / uneven column tiles;
// store_mode: 0 = choose, 1 = TMA-store epilogue (error if not possible), 2 = direct stores.
// The TMA descriptors of a call are looked up in the context's cache by (base, shape, box, type) and encoded only
// when that combination is new.
int gemm_tc_dispatch(ko_context_t *handle, int fmt, int out_fmt, int b_row_major, int64_t M, int64_t N, int64_t K, const void *A,
                     const void *B, const void *C, void *D, int bn, int store_mode, void *stream) {
    KO_REQUIRE(fmt == 0 || fmt == 1, KO_ERR_INVALID_ARG, "gemm: fmt must be 0 (f16) or 1 (bf16)");
    KO_REQUIRE(out_fmt >= 0 && out_fmt <= 2, KO_ERR_INVALID_ARG, "gemm: out_fmt must be 0 (f32), 1 (f16) or 2 (bf16)");
    KO_REQUIRE(b_row_major == 0 || b_row_major == 1, KO_ERR_INVALID_ARG, "gemm: b_row_major must be 0 or 1");
    KO_REQUIRE(M >= 0 && N >= 0 && K >= 0, KO_ERR_INVALID_ARG, "gemm: negative shape {%lld,%lld,%lld}", (long long)M,
               (long long)N, (long long)K);
    if (M == 0 || N == 0) return KO_OK;
    KO_REQUIRE(M <= 0x7fffffff && N <= 0x7fffffff && K <= 0x7fffffff, KO_ERR_SHAPE, "gemm: dimension exceeds 2^31-1");
    KO_REQUIRE(K >= 8 && K % 8 == 0, KO_ERR_SHAPE, "gemm: K = %lld must be a positive multiple of 8 (16-byte row pitch)",
               (long long)K);
    KO_REQUIRE(!b_row_major || N % 8 == 0, KO_ERR_SHAPE, "gemm: row-major B needs N = %lld to be a multiple of 8 (16-byte row pitch)",
               (long long)N);
    KO_REQUIRE(A != nullptr && B != nullptr && D != nullptr, KO_ERR_INVALID_ARG, "gemm: NULL pointer");
    KO_REQUIRE(ko::aligned16(A) && ko::aligned16(B), KO_ERR_ALIGN, "gemm: A and B must be 16-byte aligned");
    KO_REQUIRE((const void *)D != A && (const void *)D != B, KO_ERR_INVALID_ARG, "gemm: D must not alias A or B");
    ko::DeviceInfo info;
    if (int st = ko::current_device_info(&info)) return st;
    EncodeTiledFn encode = nullptr;
    if (int st = get_encode_fn(&encode)) return st;
    ko::Context *ctx = nullptr;
    if (int st = ko::resolve_context(handle, &ctx)) return st;

    // bits 16-23 of the tile code: K slices per tile (0 = choose, 1 = none, n = n slices; single-CTA kernels)
    int split_request = (bn >> 16) & 0xff;
    bn &= 0xffff;
    const int bn_request = bn;
    // The two-SM kernel when the caller asks for it, and by default where it measured fastest: medium K, where the
    // single-CTA tiles are limited by bringing operands in (128 x 256) or by their exposed epilogue (256 x 256) --
    // 16384 x 3072 x 768: 72.7 against 77.6 us; 16384 x 768 x 3072: 65.8 / 70.8; 4096 x 4096 x 1024: 35.1 / 36.7.
    // Longer K goes to the single-CTA 256 x 256 tile with uneven columns (4096^3: 97.6 against 101.9 us), K <= 512 and
    // small problems to the 128-row tile (8192 x 8192 x 512: 79.5 / 82.4; 32768 x 1024 x 256: 31.8 / 37.6).
    // (row-major B, same rule: 16384 x 3072 x 768 71.0 against 76.9 us, with BF16 output 62.4 / 65.1)
    // Long K with many tiles too (at least three per SM as 256 x 256 tiles, so that the pairs' coarser rounds cost little):
    // the pair's double-buffered accumulator hides the epilogue that the single-CTA 256 x 256 tile exposes -- 8192^3 762
    // against 795 us, 8192 x 8192 x 4096 383 / 411, 16384 x 8192 x 8192 1573 / 1655, 6144^3 346 / 362 (medians of interleaved
    // runs); 4096^3 (256 tiles) stays with the single-CTA tile and its uneven columns.
    const long long tiles256 = ((M + 255) / 256) * ((N + 255) / 256);
    const bool pair = bn == 2048 || bn == 2304 ||
                      (bn == 0 && K > 512 && M >= 4096 && N >= 512 && (K <= 3072 || tiles256 >= 3LL * info.sm_count));
    KO_REQUIRE(bn != 2304 || !b_row_major, KO_ERR_SHAPE, "gemm: uneven column tiles need column-major B");
    if (bn == 1024) bn = 256;  // 128 x 256 tiles, uneven column tiles forced
    if (bn == 1280) bn = 512;  // 256 x 256 tiles, uneven column tiles forced
    if (pair) bn = 256;
    // K slices chosen by default (see below where they are set up): few tiles and a long K.  Modelled time in
    // microseconds of the 128-row tile in 128 or 256 columns with 1 .. SMs / tiles slices: 3.3 (ramp, first loads,
    // epilogue) + rounds x K-blocks per slice x time per K-block (unsliced 0.31 us; sliced 0.29 us for 128 x 256,
    // 0.25 us for 128 x 128) and, when sliced, 3.0 for the second kernel plus the partial tiles' way through the L2
    // (every slice written once and read once, D written once, about 5 TB/s).  Fits the measurements within 10 %:
    // 1024 x 384 x 4096 21.8 us unsliced, 12.5 sliced; 1024 x 1536 x 4096 23.8 / 21.0 (48 tiles x 3);
    // 256 x 256 x 16384 74.3 / 12.4 (2 x 32).
    int auto_split = 1;
    if (bn == 0 && split_request == 0 && !pair) {
        const long long k_blocks = (K + ko::tc::kBK - 1) / ko::tc::kBK;
        const long long tiles_m = (M + ko::tc::kBM - 1) / ko::tc::kBM;
        double best = 1e300, unsliced = 1e300;
        int best_bn = 0, best_split = 1;
        for (int width : {128, 256}) {
            if (width == 256 && N <= 128) continue;
            const long long tiles = tiles_m * ((N + width - 1) / width);
            const double t_kb = width == 256 ? 0.29 : 0.25;
            const long long max_split = std::min<long long>(std::max<long long>(info.sm_count / tiles, 1), std::max<long long>(k_blocks / 4, 1));
            for (long long sp = 1; sp <= max_split && sp <= 64; ++sp) {
                const long long rounds = (tiles * sp + info.sm_count - 1) / info.sm_count;
                double cost = 3.3 + (double)rounds * (double)((k_blocks + sp - 1) / sp) * (sp == 1 ? 0.31 : t_kb);
                if (sp > 1) cost += 3.0 + (2.0 * sp + 1.0) * (double)M * (double)N * 4.0 / 5e6;
                if (sp == 1 && cost < unsliced) unsliced = cost;
                if (cost < best) { best = cost; best_bn = width; best_split = (int)sp; }
            }
        }
        if (best_split > 1 && best < 0.95 * unsliced && k_blocks >= 16) {
            bn = best_bn;
            auto_split = best_split;
        }
    }
    if (bn == 0) {
        const double e256 = wave_efficiency(M, N, 256, info.sm_count);
        // a 128 x 128 tile brings twice the operand bytes per MMA of a 128 x 256 tile: on long K it runs at little more
        // than half the rate per SM (8192 x 768 x 4096: 72.9 us in 128-wide tiles, 54.6 in 256-wide, 51.1 in 256 x 256);
        // on short K the epilogue dominates and the two are level
        const double e128 = (K <= 512 ? 0.80 : 0.58) * wave_efficiency(M, N, 128, info.sm_count);
        bn = (N > 128 && e256 >= e128) ? 256 : 128;
        if (N <= 64) bn = 64;
        if (bn == 256 && M > 128) {
            // 256 x 256 tiles (two halves share each B tile) against 128 x 256: the 128-row tile is limited by operand
            // delivery (measured 0.87 of the 256-row tile's rate on long K), the 256-row tile pays its epilogue
            // un-overlapped (about 2.5 K-blocks' worth of time per tile) and has half as many tiles to fill the waves.
            // 4096^3: 0.83 vs 0.75 (measured 101 vs 109 us); 16384 x 3072 x 768: 0.72 vs 0.82 (114 vs 97 us).
            const double k_blocks = (double)((K + ko::tc::kBK - 1) / ko::tc::kBK);
            const double tall = wave_efficiency(M, N, 256, info.sm_count, 256) / (1.0 + 2.5 / k_blocks);
            if (tall > 0.87 * e256) bn = 512;
        }
    }
    KO_REQUIRE(bn == 64 || bn == 128 || bn == 256 || bn == 512, KO_ERR_INVALID_ARG,
               "gemm: tile code %d not in {64,128,256,512,1024,1280,2048,2304}", bn_request);
    KO_REQUIRE(split_request <= 64, KO_ERR_INVALID_ARG, "gemm: %d K slices out of range (at most 64)", split_request);
    const int mt = bn == 512 ? 2 : 1;
    if (bn == 512) bn = 256;

    int pair_slots = 0;
    if (pair)
        if (int st = resident_pairs(&pair_slots)) return st;

    // uneven column tiles for the wide tile shapes (column-major B)
    ColumnPlan cols;
    const bool may_split = !b_row_major && bn == 256 && N > 256 &&
                           ((bn_request == 0 && !pair) || bn_request == 1024 || bn_request == 1280 || bn_request == 2304);
    const bool forced = bn_request == 1024 || bn_request == 1280 || bn_request == 2304;
    if (may_split)
        cols = pair ? plan_columns(M, N, 256, 256, pair_slots, true, forced) : plan_columns(M, N, mt * ko::tc::kBM, 256, info.sm_count, false, forced);
    KO_REQUIRE((bn_request != 1024 && bn_request != 1280 && bn_request != 2304) || cols.tiles_n != 0, KO_ERR_SHAPE,
               "gemm: uneven column tiles bring nothing for this shape");

    alignas(64) CUtensorMap map_a, map_b, map_b_narrow, map_d;
    // key.kind: bits 0-1 input / output type, bits 4-7 which of the map layouts
    const int a_box_rows = pair ? ko::tc::kBM : mt * ko::tc::kBM;  // a CTA of a pair loads its own 128 rows
    const ko::TensorMapKey key_a{A, (uint64_t)K, (uint64_t)M, (uint32_t)ko::tc::kBK, (uint32_t)a_box_rows, (uint32_t)fmt | 0x10u};
    if (int st = ctx->tensor_map(key_a, &map_a, [&](CUtensorMap *m) { return make_map(encode, m, fmt, A, M, K, a_box_rows); })) return st;
    if (b_row_major) {
        const ko::TensorMapKey key_b{B, (uint64_t)N, (uint64_t)K, 64u, (uint32_t)ko::tc::kBK, (uint32_t)fmt | 0x20u};
        if (int st = ctx->tensor_map(key_b, &map_b, [&](CUtensorMap *m) { return make_map_b_row_major(encode, m, fmt, B, K, N); })) return st;
    } else {
        // a CTA of a pair loads half of the tile's columns
        const int box_rows = (cols.tiles_n ? cols.bn_wide : bn) / (pair ? 2 : 1);
        const ko::TensorMapKey key_b{B, (uint64_t)K, (uint64_t)N, (uint32_t)ko::tc::kBK, (uint32_t)box_rows, (uint32_t)fmt | 0x10u};
        if (int st = ctx->tensor_map(key_b, &map_b, [&](CUtensorMap *m) { return make_map(encode, m, fmt, B, N, K, box_rows); })) return st;
    }
    map_b_narrow = map_b;
    if (cols.tiles_n && cols.bn_narrow != cols.bn_wide) {
        const int box_rows = cols.bn_narrow / (pair ? 2 : 1);
        const ko::TensorMapKey key_n{B, (uint64_t)K, (uint64_t)N, (uint32_t)ko::tc::kBK, (uint32_t)box_rows, (uint32_t)fmt | 0x10u};
        if (int st = ctx->tensor_map(key_n, &map_b_narrow, [&](CUtensorMap *m) { return make_map(encode, m, fmt, B, N, K, box_rows); }))
            return st;
    }
    // TMA-store epilogue when D has a 16-byte pitch and nothing is added to it
    const bool tma_store = store_mode != 2 && C == nullptr && N % (out_fmt == 0 ? 4 : 8) == 0 && ko::aligned16(D);
    KO_REQUIRE(store_mode != 1 || tma_store, KO_ERR_SHAPE,
               "gemm: the TMA-store epilogue needs C == NULL and a 16-byte row pitch and base for D");
    if (tma_store) {
        const ko::TensorMapKey key_d{D, (uint64_t)N, (uint64_t)M, 32u, 32u, (uint32_t)out_fmt | 0x40u};
        if (int st = ctx->tensor_map(key_d, &map_d, [&](CUtensorMap *m) { return make_store_map(encode, m, out_fmt, D, M, N); })) return st;
    } else {
        map_d = map_a;  // unused by the direct-store epilogue
    }

    ko::tc::GemmParams p;
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.C = C; p.D = D; p.fmt = fmt; p.out_fmt = out_fmt; p.b_row_major = b_row_major;
    p.tiles_n = cols.tiles_n; p.wide_tiles_n = cols.wide_tiles_n; p.bn_wide = cols.bn_wide; p.bn_narrow = cols.bn_narrow;
    p.split_k = 1; p.partials = nullptr;
    if (int st = ko::device_status_word(0, &p.status)) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    // K slices.  A tile's main loop is a serial chain of K / 64 K-blocks (about 0.34 us each), so a problem with fewer
    // tiles than SMs and a long K leaves most of the device idle for the whole chain: 1024 x 384 x 4096 took 24.5 us
    // whatever the tile shape.  Cut into slices, every SM gets a part of the chain; the price is one FP32 partial tile
    // per slice, written by the GEMM kernel and summed into D by a second, small kernel (both L2-resident).
    KO_REQUIRE(split_request <= 1 || !pair, KO_ERR_INVALID_ARG, "gemm: K slices are not available in the two-SM kernel");
    long long sum_blocks = 0;  // blocks of the kernel that adds the slices (one per 32 x 32 chunk of every tile)
    if (!pair) {
        const long long tile_m = (long long)mt * ko::tc::kBM;
        const long long tiles = ((M + tile_m - 1) / tile_m) * (cols.tiles_n ? cols.tiles_n : (N + bn - 1) / bn);
        const long long k_blocks = (K + ko::tc::kBK - 1) / ko::tc::kBK;
        long long split = split_request ? split_request : auto_split;
        if (split > k_blocks) split = k_blocks;
        if (split > 1) {
            // the scratch lane of this stream in the context, shared with the SGEMM's K split (launches of one stream
            // run one after the other); sized once for the largest default request: one slot per SM
            const size_t slot_floats = (size_t)tile_m * bn;
            const size_t floor_tiles = (size_t)4 * info.sm_count;
            ko::SgemmScratch sc;
            const int st = ctx->sgemm_scratch(s, (size_t)(tiles * split) * slot_floats, 0, floor_tiles * 128 * 128, floor_tiles, &sc);
            if (st == KO_OK) {
                p.split_k = (int)split;
                p.partials = sc.partials;
                sum_blocks = tiles * (tile_m / 32) * (bn / 32);
            } else if (split_request > 1) {
                return st;
            }  // chosen by default but no scratch to be had (a stream being captured): one slice
        }
    }
    if (pair)
        return tma_store ? launch_pair<true>(map_a, map_b, map_b_narrow, map_d, p, pair_slots, s)
                         : launch_pair<false>(map_a, map_b, map_b_narrow, map_d, p, pair_slots, s);
    int st;
    if (mt == 2) {
        st = tma_store ? launch<256, true, 2>(map_a, map_b, map_b_narrow, map_d, p, info.sm_count, s)
                       : launch<256, false, 2>(map_a, map_b, map_b_narrow, map_d, p, info.sm_count, s);
    } else {
        switch (bn) {
            case 64: st = tma_store ? launch<64, true>(map_a, map_b, map_b_narrow, map_d, p, info.sm_count, s) : launch<64, false>(map_a, map_b, map_b_narrow, map_d, p, info.sm_count, s); break;
            case 128: st = tma_store ? launch<128, true>(map_a, map_b, map_b_narrow, map_d, p, info.sm_count, s) : launch<128, false>(map_a, map_b, map_b_narrow, map_d, p, info.sm_count, s); break;
            default: st = tma_store ? launch<256, true>(map_a, map_b, map_b_narrow, map_d, p, info.sm_count, s) : launch<256, false>(map_a, map_b, map_b_narrow, map_d, p, info.sm_count, s); break;
        }
    }
    if (st != KO_OK || p.split_k <= 1) return st;
    KO_REQUIRE(sum_blocks <= 0x7fffffffLL, KO_ERR_SHAPE, "gemm: %lld chunks exceed the grid limit", sum_blocks);
    return ko::launch_overlapped(ko::tc::gemm_slice_sum_kernel<256>, (unsigned)sum_blocks, 256u, (size_t)0, s, p, mt * ko::tc::kBM, bn);
}

}  // namespace

extern "C" {

int ko_gemm_tc_tuned(int fmt, int out_fmt, int b_row_major, int64_t M, int64_t N, int64_t K, const void *A, const void *B,
                     const void *C, void *D, int bn, int store_mode, void *stream) {
    return gemm_tc_dispatch(nullptr, fmt, out_fmt, b_row_major, M, N, K, A, B, C, D, bn, store_mode, stream);
}

int ko_gemm_tc(int in_fmt, int out_fmt, int b_row_major, int64_t M, int64_t N, int64_t K, const void *A, const void *B,
               const void *C, void *D, void *stream) {
    return gemm_tc_dispatch(nullptr, in_fmt, out_fmt, b_row_major, M, N, K, A, B, C, D, 0, 0, stream);
}

int ko_gemm_tc_ctx(ko_context_t *ctx, int in_fmt, int out_fmt, int b_row_major, int64_t M, int64_t N, int64_t K, const void *A,
                   const void *B, const void *C, void *D, void *stream) {
    return gemm_tc_dispatch(ctx, in_fmt, out_fmt, b_row_major, M, N, K, A, B, C, D, 0, 0, stream);
}

int ko_gemm_f16_f32(int64_t M, int64_t N, int64_t K, const uint16_t *A, const uint16_t *B, const float *C, float *D,
                    void *stream) {
    return ko_gemm_tc_tuned(0, 0, 0, M, N, K, A, B, C, D, 0, 0, stream);
}

int ko_gemm_bf16_f32(int64_t M, int64_t N, int64_t K, const uint16_t *A, const uint16_t *B, const float *C, float *D,
                     void *stream) {
    return ko_gemm_tc_tuned(1, 0, 0, M, N, K, A, B, C, D, 0, 0, stream);
}

int ko_gemm_f16_f16(int64_t M, int64_t N, int64_t K, const uint16_t *A, const uint16_t *B, const uint16_t *C, uint16_t *D,
                    void *stream) {
    return ko_gemm_tc_tuned(0, 1, 0, M, N, K, A, B, C, D, 0, 0, stream);
}

int ko_gemm_bf16_bf16(int64_t M, int64_t N, int64_t K, const uint16_t *A, const uint16_t *B, const uint16_t *C, uint16_t *D,
                      void *stream) {
    return ko_gemm_tc_tuned(1, 2, 0, M, N, K, A, B, C, D, 0, 0, stream);
}

}  // extern "C"
