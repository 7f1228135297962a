// C-ABI launchers of the tcgen05 tensor-core GEMM: build the TMA descriptors, pick the tile width,
// launch one persistent CTA per SM.
#include "ko_internal.h"
#include "ko_tuning.h"
#include "row_launch.h"

#include <mutex>

#include <cudaTypedefs.h>

#include "../nn_operators/gemm/tensor_core_gemm.h"

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

template <int BN, bool kTmaStore, int MT = 1>
int launch(const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &md, const ko::tc::GemmParams &p, int sm_count,
           cudaStream_t s) {
    using Cfg = ko::tc::TileConfig<BN, MT>;
    auto kernel = ko::tc::gemm_tcgen05_kernel<BN, kTmaStore, MT>;
    if (int st = ko::ensure_dynamic_smem(reinterpret_cast<const void *>(kernel), Cfg::kSmemBytes)) return st;
    const long long tiles = (long long)((p.M + MT * ko::tc::kBM - 1) / (MT * ko::tc::kBM)) * ((p.N + BN - 1) / BN);
    const unsigned grid = (unsigned)(tiles < sm_count ? tiles : sm_count);
    return ko::launch_overlapped(kernel, grid, (unsigned)ko::tc::kThreads, (size_t)Cfg::kSmemBytes, s, ma, mb, md, p);
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

}  // namespace

extern "C" {

// fmt: A and B, 0 = F16, 1 = BF16; out_fmt: D and C, 0 = FP32, 1 = F16, 2 = BF16; b_row_major: 0 = B[K,N]
// column-major (K contiguous), 1 = row-major (N contiguous); bn: 0 = choose, else 64 / 128 / 256 columns per tile;
// store_mode: 0 = choose, 1 = TMA-store epilogue (error if not possible), 2 = direct stores;
// bn = 512 selects the 256 x 256 tile (two 128-row halves per CTA share every B tile)
int ko_gemm_tc_tuned(int fmt, int out_fmt, int b_row_major, int64_t M, int64_t N, int64_t K, const void *A, const void *B,
                     const void *C, void *D, int bn, int store_mode, void *stream) {
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

    if (bn == 0) {
        const double e256 = wave_efficiency(M, N, 256, info.sm_count);
        const double e128 = 0.80 * wave_efficiency(M, N, 128, info.sm_count);
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
    KO_REQUIRE(bn == 64 || bn == 128 || bn == 256 || bn == 512, KO_ERR_INVALID_ARG, "gemm: tile width %d not in {64,128,256,512}", bn);
    const int mt = bn == 512 ? 2 : 1;
    if (bn == 512) bn = 256;

    alignas(64) CUtensorMap map_a, map_b, map_d;
    if (int st = make_map(encode, &map_a, fmt, A, M, K, mt * ko::tc::kBM)) return st;
    if (int st = b_row_major ? make_map_b_row_major(encode, &map_b, fmt, B, K, N) : make_map(encode, &map_b, fmt, B, N, K, bn))
        return st;
    // TMA-store epilogue when D has a 16-byte pitch and nothing is added to it
    const bool tma_store = store_mode != 2 && C == nullptr && N % (out_fmt == 0 ? 4 : 8) == 0 && ko::aligned16(D);
    KO_REQUIRE(store_mode != 1 || tma_store, KO_ERR_SHAPE,
               "gemm: the TMA-store epilogue needs C == NULL and a 16-byte row pitch and base for D");
    if (tma_store) {
        if (int st = make_store_map(encode, &map_d, out_fmt, D, M, N)) return st;
    } else {
        map_d = map_a;  // unused by the direct-store epilogue
    }

    ko::tc::GemmParams p;
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.C = C; p.D = D; p.fmt = fmt; p.out_fmt = out_fmt; p.b_row_major = b_row_major;
    if (int st = ko::device_status_word(0, &p.status)) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (mt == 2)
        return tma_store ? launch<256, true, 2>(map_a, map_b, map_d, p, info.sm_count, s)
                         : launch<256, false, 2>(map_a, map_b, map_d, p, info.sm_count, s);
    switch (bn) {
        case 64: return tma_store ? launch<64, true>(map_a, map_b, map_d, p, info.sm_count, s) : launch<64, false>(map_a, map_b, map_d, p, info.sm_count, s);
        case 128: return tma_store ? launch<128, true>(map_a, map_b, map_d, p, info.sm_count, s) : launch<128, false>(map_a, map_b, map_d, p, info.sm_count, s);
        default: return tma_store ? launch<256, true>(map_a, map_b, map_d, p, info.sm_count, s) : launch<256, false>(map_a, map_b, map_d, p, info.sm_count, s);
    }
}

int ko_gemm_tc(int in_fmt, int out_fmt, int b_row_major, int64_t M, int64_t N, int64_t K, const void *A, const void *B,
               const void *C, void *D, void *stream) {
    return ko_gemm_tc_tuned(in_fmt, out_fmt, b_row_major, M, N, K, A, B, C, D, 0, 0, stream);
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
