// C-ABI launcher of the FFMA SGEMM: picks the tile configuration from the problem shape.
#include "ko_context.h"
#include "ko_internal.h"
#include "../../include/ko_b200_tuning.h"

#include "../nn_operators/gemm/simt_gemm.h"
#include "../nn_operators/gemm/simt_gemm_x2.h"
#include "row_launch.h"

namespace {

//                              BM   BN  BK  WM  WN LM
using CfgBig = ko::SgemmConfig<128, 128, 16, 32, 64, 4>;   // 256 threads, 8x8 per lane
using CfgWide = ko::SgemmConfig<128, 64, 16, 32, 32, 4>;   // 256 threads, 8x4 per lane
using CfgSmall = ko::SgemmConfig<64, 64, 16, 32, 32, 4>;   // 128 threads, 8x4 per lane

template <typename Cfg>
int launch(int M, int N, int K, const float *A, const float *B, const float *C, float *D, bool aligned,
           cudaStream_t s) {
    const long long tiles = (long long)((M + Cfg::BM - 1) / Cfg::BM) * ((N + Cfg::BN - 1) / Cfg::BN);
    KO_REQUIRE(tiles <= 0x7fffffffLL, KO_ERR_SHAPE, "sgemm: %lld tiles exceed the grid limit", tiles);
    if (aligned)
        ko::sgemm_kernel<Cfg, true><<<(unsigned)tiles, Cfg::kThreads, Cfg::kSmemBytes, s>>>(M, N, K, A, B, C, D);
    else
        ko::sgemm_kernel<Cfg, false><<<(unsigned)tiles, Cfg::kThreads, Cfg::kSmemBytes, s>>>(M, N, K, A, B, C, D);
    KO_CHECK_LAUNCH("sgemm_kernel");
    return KO_OK;
}

// Split-K scratch (partial tiles plus one arrival counter per tile) comes from the context: one lane per
// stream, so that launches on different streams never share partials; allocated the first time a stream needs
// one, at the largest size the shape rules below can ask for (ranges: 2 partial tiles for each of 2 x SMs blocks,
// tiles < 4 x SMs), never freed or moved before the context dies.  Counters are zero whenever no launch is in
// flight (the last block of a tile resets its counter).
// One launch of sgemm_x2_kernel<kVecB, kWarpsM, kWarpsN, kGroups>.
// split_k: 0 = choose the block count, 1 = one block per tile, n > 1 = n K-slices per tile.
template <int kWarpsM, int kWarpsN, int kGroups>
int launch_x2_shape(ko::Context *ctx, int M, int N, int K, const float *A, const float *B, const float *C, float *D, int split_k,
                    int sm_count, cudaStream_t s) {
    namespace x2 = ko::sgemm2;
    using S = x2::Shape<kWarpsM, kWarpsN>;
    const long long tiles = (long long)((M + S::BM - 1) / S::BM) * ((N + S::BN - 1) / S::BN);
    const int ktiles = (K + x2::BK - 1) / x2::BK;
    const long long units = tiles * ktiles;
    const long long slots = (kGroups == 1 ? 2LL : 1LL) * sm_count;  // blocks resident at a time
    long long ctas = tiles;
    int max_contrib = 1;
    bool ranges = false;  // blocks own contiguous unit ranges that may straddle tiles
    if (split_k > 1) {
        if (split_k > ktiles) split_k = ktiles;
        ctas = tiles * split_k;
        max_contrib = split_k;  // slices of a uniform split never straddle a tile
    } else if (split_k == 0 && tiles * 2 <= sm_count) {
        // few tiles: a uniform split that gives about one block per SM measured faster than finer ranges,
        // whose partial-tile traffic and short K loops cost more than the idle SMs
        // (at least 4 K-tiles per block: 256^3 runs 10.7 us as 8 tiles x 4 slices against 15.2 us unsplit)
        int split = (int)(sm_count / tiles);
        while (split > 1 && ktiles / split < 4) --split;
        if (split > 1) {
            ctas = tiles * split;
            max_contrib = split;
        }
    } else if (split_k == 0 && kGroups == 1 && tiles < 2 * slots && tiles % slots != 0) {
        // up to two waves of whole tiles, the last one partly empty: hand every slot the same number of
        // (tile, K-tile) units instead, as long as a block still gets at least 8 K-tiles to amortise its
        // pipeline fill and the partial-tile traffic.  (With more waves the tail costs less than the
        // partial tiles: 4096^3, 3.46 waves, measured 2510 us as whole tiles and 2584 us as ranges.)
        ctas = slots;
        if (units / ctas < 8) ctas = units / 8 > tiles ? units / 8 : tiles;
        ranges = ctas != tiles;
    }
    KO_REQUIRE(ctas <= 0x7fffffffLL, KO_ERR_SHAPE, "sgemm: %lld blocks exceed the grid limit", ctas);
    x2::Params p{M, N, K, A, B, C, D, (int)ctas, max_contrib, ranges ? 1 : 0, nullptr, nullptr};
    if (ctas != tiles) {
        if (ranges) {
            const long long per_block = units / ctas;  // floor: the shortest range
            const long long most = (ktiles + per_block - 1) / per_block + 1;
            p.max_contrib = (int)(most > ctas ? ctas : most);
        }
        ko::SgemmScratch sc;
        const size_t partials = ranges ? (size_t)ctas * 2 : (size_t)tiles * max_contrib;
        const size_t floor_tiles = (size_t)4 * sm_count;
        if (int st = ctx->sgemm_scratch(s, partials * S::kTileFloats, (size_t)tiles, floor_tiles * 128 * 128, floor_tiles, &sc)) return st;
        p.workspace = sc.partials;
        p.counters = sc.counters;
    }
    const bool vec_b = N % 4 == 0 && ko::aligned16(B);
    constexpr int smem_bytes = S::smem_bytes(kGroups);
    auto go = [&](auto kernel) -> int {
        if (int st = ko::ensure_dynamic_smem(reinterpret_cast<const void *>(kernel), smem_bytes)) return st;
        return ko::launch_overlapped(kernel, (unsigned)ctas, (unsigned)(S::kGroupThreads * kGroups), (size_t)smem_bytes, s, p);
    };
    const int st = vec_b ? go(x2::sgemm_x2_kernel<true, kWarpsM, kWarpsN, kGroups>) : go(x2::sgemm_x2_kernel<false, kWarpsM, kWarpsN, kGroups>);
    return st;
}

// shape: 0 = choose; 1 = 128 x 128 tiles, 128-thread blocks (two per SM); 2 = 128 x 128 tiles, two groups of
// 4 warps halve the block's K range; 3 = 64 x 128 tiles, four groups of 2 warps quarter it.
int launch_x2(ko::Context *ctx, int M, int N, int K, const float *A, const float *B, const float *C, float *D, int split_k, int shape,
              int sm_count, cudaStream_t s) {
    if (shape == 0) {
        // The grouped shapes add K parts like K-slices, so they are chosen only when the caller left the
        // split to us.  At most one 128 x 128 tile per SM: groups give every scheduler a second warp, and
        // the half-height tile doubles the tile count, which saves or shortens the split across blocks
        // (1024^3: 63.8 us as 128-thread blocks, 55.5 us grouped; 512^3: 37.2 -> 22.8 us; 1536^3: 160 -> 152 us;
        // from 2048^3 on two 128-thread blocks per SM are faster).
        const long long wide_tiles = (long long)((M + 127) / 128) * ((N + 127) / 128);
        const int ktiles = (K + ko::sgemm2::BK - 1) / ko::sgemm2::BK;
        // many tiles: the 64 x 128 shape with four groups (one 256-thread block per SM) also beats two 128-thread
        // blocks per SM on long K (4096^3: 2334 vs 2431 us; 3072^3: 1011 vs 1074 us) as long as its waves are full;
        // a partly empty last wave goes to the 128 x 128 shape, whose unit ranges balance it (2048^3: 341 vs 349 us),
        // and so does short K, where a group's quarter of K is too few K-tiles (8192 x 8192 x 1024: 2486 vs 2549 us)
        const long long narrow_tiles = (long long)((M + 63) / 64) * ((N + 127) / 128);
        const long long waves = (narrow_tiles + sm_count - 1) / sm_count;
        const bool full_waves = narrow_tiles * 100 >= waves * sm_count * 95;
        shape = 1;
        if (split_k == 0 && ktiles >= 8 && (wide_tiles <= sm_count || (full_waves && ktiles >= 128 && M > 64)))
            shape = (M > 64 && ktiles >= 16) ? 3 : 2;
    }
    switch (shape) {
        case 1: return launch_x2_shape<2, 2, 1>(ctx, M, N, K, A, B, C, D, split_k, sm_count, s);
        case 2: return launch_x2_shape<2, 2, 2>(ctx, M, N, K, A, B, C, D, split_k, sm_count, s);
        default: return launch_x2_shape<1, 2, 4>(ctx, M, N, K, A, B, C, D, split_k, sm_count, s);
    }
}

}  // namespace

namespace {

// variant: 0 = choose; 1 = 128x128 tiles with 8x8 per thread; 2 = 128x64; 3 = 64x64 (scalar FFMA,
// register-staged); 4 = 128x128 with 16x8 per thread, packed FFMA, cp.async ring, split_k slices
// (split_k 0 = choose, ignored by variants 1-3); 6 / 7 / 8 = variant 4 pinned to one block shape
int sgemm_dispatch(ko_context_t *handle, int64_t M, int64_t N, int64_t K, const float *A, const float *B, const float *C, float *D,
                   int variant, int split_k, void *stream) {
    KO_REQUIRE(M >= 0 && N >= 0 && K >= 0, KO_ERR_INVALID_ARG, "sgemm: negative shape {%lld,%lld,%lld}",
               (long long)M, (long long)N, (long long)K);
    if (M == 0 || N == 0) return KO_OK;
    KO_REQUIRE(M <= 0x7fffffff && N <= 0x7fffffff && K <= 0x7fffffff, KO_ERR_SHAPE, "sgemm: dimension exceeds 2^31-1");
    KO_REQUIRE(D != nullptr && (K == 0 || (A != nullptr && B != nullptr)), KO_ERR_INVALID_ARG, "sgemm: NULL pointer");
    KO_REQUIRE(D != A && D != B, KO_ERR_INVALID_ARG, "sgemm: D must not alias A or B");
    ko::DeviceInfo info;
    if (int st = ko::current_device_info(&info)) return st;
    ko::Context *ctx = nullptr;
    if (int st = ko::resolve_context(handle, &ctx)) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool aligned = K % 4 == 0 && N % 4 == 0 && ko::aligned16(A) && ko::aligned16(B);

    KO_REQUIRE(split_k >= 0 && split_k <= 64, KO_ERR_INVALID_ARG, "sgemm: split_k %d out of range", split_k);
    if (variant == 0) variant = (M >= 64 && N >= 64 && K >= 16) ? 4 : 3;
    if (K == 0 && variant >= 4) variant = 3;  // an empty sum: D = C (or 0), nothing to pipeline
    const int m = (int)M, n = (int)N, k = (int)K;
    switch (variant) {
        case 4: return launch_x2(ctx, m, n, k, A, B, C, D, split_k, 0, info.sm_count, s);
        case 6: return launch_x2(ctx, m, n, k, A, B, C, D, split_k, 1, info.sm_count, s);  // 128 x 128, 128-thread blocks
        case 7: return launch_x2(ctx, m, n, k, A, B, C, D, split_k, 2, info.sm_count, s);  // 128 x 128, two warp groups
        case 8: return launch_x2(ctx, m, n, k, A, B, C, D, split_k, 3, info.sm_count, s);  // 64 x 128, four warp groups
        case 1: return launch<CfgBig>(m, n, k, A, B, C, D, aligned, s);
        case 2: return launch<CfgWide>(m, n, k, A, B, C, D, aligned, s);
        case 3: return launch<CfgSmall>(m, n, k, A, B, C, D, aligned, s);
        default: return ko::fail(KO_ERR_INVALID_ARG, "sgemm: unknown variant %d", variant);
    }
}

}  // namespace

extern "C" {

int ko_sgemm_f32_tuned(int64_t M, int64_t N, int64_t K, const float *A, const float *B, const float *C, float *D,
                       int variant, int split_k, void *stream) {
    return sgemm_dispatch(nullptr, M, N, K, A, B, C, D, variant, split_k, stream);
}

int ko_sgemm_f32(int64_t M, int64_t N, int64_t K, const float *A, const float *B, const float *C, float *D,
                 void *stream) {
    return sgemm_dispatch(nullptr, M, N, K, A, B, C, D, 0, 0, stream);
}

int ko_sgemm_f32_ctx(ko_context_t *ctx, int64_t M, int64_t N, int64_t K, const float *A, const float *B, const float *C,
                     float *D, void *stream) {
    return sgemm_dispatch(ctx, M, N, K, A, B, C, D, 0, 0, stream);
}

}  // extern "C"
