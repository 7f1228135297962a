// LayerNorm forward over the last dimension for sm_100a, FP32 or BF16 I/O, FP32 statistics.
//
// Statistics are Welford/Chan triples (count, mean, M2): every thread forms the exact triple of
// the elements it holds in registers (mean first, then squared deviations from it), and triples
// are merged pairwise across lanes by shuffle and across warps through shared memory.  M2 stays
// a sum of squared deviations through all merge levels and is divided once, by (cols - ddof).
// (The reference's WelfordMerge divides by n-1 at every level, layernorm.h:48, and its
// normalisation adds the mean through the Subtract functor, functors.h:168; neither is kept.)
//
// Tiers by row length (the reference's warp / block-cached / block-no-cache split,
// nn_operators/layernorm/layernorm.h:145-201, :204-252, :254-300):
//   group tier   short rows: a row per group of 4..32 lanes, several rows per warp step, persistent
//                warps with gamma/beta held in registers;
//   staged tier  persistent blocks, a producer warp streams chunks of rows into a shared-memory ring
//                with 1-D bulk copies (TMA), consumer warps work out of shared memory
//                (common/row_pipeline.h);
//   warp tier    one warp owns kRows consecutive rows per step, rows in registers;
//   block tier   one thread block per row, row in registers, one shared-memory exchange;
//   resident tier persistent blocks for long rows: gamma/beta held in registers, packed FP32 math,
//                next row prefetched into registers or the next rows into a per-thread shared-memory ring;
//   cluster tier one row per thread-block cluster, Welford triples exchanged through distributed
//                shared memory (few very long rows);
//   reread tier  rows beyond one block's registers: one row (or a pair sharing gamma/beta) per block in
//                two passes, the second served by the L2; optionally every load through a shared-memory
//                ring of (row, pass, chunk) items;
//   stream tier  one thread block per row, two passes over global memory, scalar accesses, any
//                column count and alignment.
// y = ((x - mean) * rstd) * gamma + beta, gamma/beta optional, in the I/O element type.
//
// The reference's LayerNormWarpImpl / LayerNormBlockImpl / LayerNormBlockNoCacheImpl templates and
// the layer_normalization<Kernel> __global__ wrapper keep their names and parameters.
#pragma once

#include <cooperative_groups.h>

#include "../../common/common.h"
#include "../../common/functors.h"
#include "../../common/row_pipeline.h"

namespace ko {

// 16-byte vector of I/O elements, unpacked to FP32
template <typename T>
struct RowIo;

template <>
struct RowIo<float> {
    static constexpr int kPerVec = 4;
    using Raw = float4;
    __device__ __forceinline__ static void unpack(const Raw &r, float (&f)[4]) {
        f[0] = r.x; f[1] = r.y; f[2] = r.z; f[3] = r.w;
    }
    __device__ __forceinline__ static Raw pack(const float (&f)[4]) { return make_float4(f[0], f[1], f[2], f[3]); }
    __device__ __forceinline__ static void unpack_pairs(const Raw &r, f32x2 *p) {
        p[0] = pair_of(r.x, r.y);
        p[1] = pair_of(r.z, r.w);
    }
    __device__ __forceinline__ static Raw pack_pairs(const f32x2 *p) {
        Raw r;
        pair_split(p[0], r.x, r.y);
        pair_split(p[1], r.z, r.w);
        return r;
    }
    __device__ __forceinline__ static float to_float(float v) { return v; }
    __device__ __forceinline__ static float from_float(float v) { return v; }
};

template <>
struct RowIo<__nv_bfloat16> {
    static constexpr int kPerVec = 8;
    using Raw = uint4;
    __device__ __forceinline__ static void unpack(const Raw &r, float (&f)[8]) {
        f[0] = bf16_lo(r.x); f[1] = bf16_hi(r.x); f[2] = bf16_lo(r.y); f[3] = bf16_hi(r.y);
        f[4] = bf16_lo(r.z); f[5] = bf16_hi(r.z); f[6] = bf16_lo(r.w); f[7] = bf16_hi(r.w);
    }
    __device__ __forceinline__ static Raw pack(const float (&f)[8]) {
        return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
    }
    __device__ __forceinline__ static void unpack_pairs(const Raw &r, f32x2 *p) {
        p[0] = pair_of(bf16_lo(r.x), bf16_hi(r.x));
        p[1] = pair_of(bf16_lo(r.y), bf16_hi(r.y));
        p[2] = pair_of(bf16_lo(r.z), bf16_hi(r.z));
        p[3] = pair_of(bf16_lo(r.w), bf16_hi(r.w));
    }
    __device__ __forceinline__ static Raw pack_pairs(const f32x2 *p) {
        float lo[4], hi[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) pair_split(p[i], lo[i], hi[i]);
        return make_uint4(pack_bf16(lo[0], hi[0]), pack_bf16(lo[1], hi[1]), pack_bf16(lo[2], hi[2]), pack_bf16(lo[3], hi[3]));
    }
    __device__ __forceinline__ static float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ __forceinline__ static __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
};

// FP16 rows (the reference's Rsqrt<half> / MultiplyAdd<half> element type, common/functors.h:105-111, :280-290):
// widened to FP32 on load, statistics and normalisation in FP32, rounded once on store
template <>
struct RowIo<__half> {
    static constexpr int kPerVec = 8;
    using Raw = uint4;
    __device__ __forceinline__ static float2 widen2(uint32_t w) { return __half22float2(*reinterpret_cast<const __half2 *>(&w)); }
    __device__ __forceinline__ static uint32_t narrow2(float lo, float hi) {
        const __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<const uint32_t *>(&h);
    }
    __device__ __forceinline__ static void unpack(const Raw &r, float (&f)[8]) {
        const float2 a = widen2(r.x), b = widen2(r.y), c = widen2(r.z), d = widen2(r.w);
        f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
    }
    __device__ __forceinline__ static Raw pack(const float (&f)[8]) {
        return make_uint4(narrow2(f[0], f[1]), narrow2(f[2], f[3]), narrow2(f[4], f[5]), narrow2(f[6], f[7]));
    }
    __device__ __forceinline__ static void unpack_pairs(const Raw &r, f32x2 *p) {
        const float2 a = widen2(r.x), b = widen2(r.y), c = widen2(r.z), d = widen2(r.w);
        p[0] = pair_of(a.x, a.y);
        p[1] = pair_of(b.x, b.y);
        p[2] = pair_of(c.x, c.y);
        p[3] = pair_of(d.x, d.y);
    }
    __device__ __forceinline__ static Raw pack_pairs(const f32x2 *p) {
        float lo[4], hi[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) pair_split(p[i], lo[i], hi[i]);
        return make_uint4(narrow2(lo[0], hi[0]), narrow2(lo[1], hi[1]), narrow2(lo[2], hi[2]), narrow2(lo[3], hi[3]));
    }
    __device__ __forceinline__ static float to_float(__half v) { return __half2float(v); }
    __device__ __forceinline__ static __half from_float(float v) { return __float2half_rn(v); }
};

// exact (count, mean, M2) of the valid_vecs * kPerVec values a thread holds as raw 16-byte vectors:
// mean first, then the squared deviations from it (both passes run over registers)
template <typename T, int kVecs>
__device__ __forceinline__ Welford welford_of_vectors(const typename RowIo<T>::Raw (&raw)[kVecs], int valid_vecs) {
    using Io = RowIo<T>;
    constexpr int kPer = Io::kPerVec;
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < kVecs; ++j) {
        float f[kPer];
        Io::unpack(raw[j], f);
        float part = 0.f;
#pragma unroll
        for (int e = 0; e < kPer; ++e) part += f[e];
        sum += j < valid_vecs ? part : 0.f;
    }
    Welford w;
    w.n = (float)(valid_vecs * kPer);
    w.mean = valid_vecs > 0 ? sum / w.n : 0.f;
    float m2 = 0.f;
#pragma unroll
    for (int j = 0; j < kVecs; ++j) {
        float f[kPer];
        Io::unpack(raw[j], f);
        float part = 0.f;
#pragma unroll
        for (int e = 0; e < kPer; ++e) {
            const float d = f[e] - w.mean;
            part = fmaf(d, d, part);
        }
        m2 += j < valid_vecs ? part : 0.f;
    }
    w.m2 = m2;
    return w;
}

__device__ __forceinline__ float rstd_from(const Welford &w, int cols, int ddof, float eps) {
    const float denom = (float)(cols - ddof);
    const float var = denom > 0.f ? w.m2 / denom : 0.f;
    return rsqrtf(var + eps);
}

// normalise one raw vector: ((x - mean) * rstd) * gamma + beta
template <typename T>
__device__ __forceinline__ typename RowIo<T>::Raw normalise_vector(const typename RowIo<T>::Raw &raw, float mean, float rstd,
                                                                  const typename RowIo<T>::Raw *gamma_v,
                                                                  const typename RowIo<T>::Raw *beta_v, int v) {
    using Io = RowIo<T>;
    constexpr int kPer = Io::kPerVec;
    float f[kPer], g[kPer], b[kPer], y[kPer];
    Io::unpack(raw, f);
#pragma unroll
    for (int e = 0; e < kPer; ++e) { g[e] = 1.f; b[e] = 0.f; }
    if (gamma_v) Io::unpack(__ldg(gamma_v + v), g);
    if (beta_v) Io::unpack(__ldg(beta_v + v), b);
#pragma unroll
    for (int e = 0; e < kPer; ++e) y[e] = fmaf((f[e] - mean) * rstd, g[e], b[e]);
    return Io::pack(y);
}

// kRows rows spread over the warp (kVecs raw vectors per lane each): statistics, then the
// normalised rows are written to out_v at rows row0 .. row0+kRows-1 (rows >= row_limit are skipped)
template <typename T, int kVecs, int kRows>
__device__ __forceinline__ void layernorm_rows_from_registers(const typename RowIo<T>::Raw (&raw)[kRows][kVecs], int my_vecs,
                                                              int nvec, int lane, long long row0, long long row_limit,
                                                              typename RowIo<T>::Raw *out_v, int cols, float eps,
                                                              const typename RowIo<T>::Raw *gamma_v,
                                                              const typename RowIo<T>::Raw *beta_v, int ddof) {
    using Io = RowIo<T>;
    constexpr int kPer = Io::kPerVec, kPairsPerVec = kPer / 2;
    if constexpr (kVecs * kPer <= 32) {  // depends on the row length only, so a row's bits do not depend on kRows
        // Short rows: the whole row fits in registers as FP32, so it is unpacked once and all three passes
        // run on packed FP32 pairs.  Statistics in their exact two-pass form: the warp-wide sum gives the row
        // mean, then the squared deviations from THAT mean are summed (the value a Welford/Chan merge of the
        // lanes' triples converges to, without the merges' ~70 instructions per row).
        const float inv_cols = 1.0f / (float)cols;
        const float inv_denom = cols - ddof > 0 ? 1.0f / (float)(cols - ddof) : 0.f;
        f32x2 x2[kRows][kVecs * kPairsPerVec];
        float mean[kRows], rstd[kRows];
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            f32x2 acc = pair_of(0.f, 0.f);
#pragma unroll
            for (int j = 0; j < kVecs; ++j) {
                Io::unpack_pairs(raw[r][j], x2[r] + j * kPairsPerVec);  // padded vectors are zero
#pragma unroll
                for (int q = 0; q < kPairsPerVec; ++q) acc = pair_add(acc, x2[r][j * kPairsPerVec + q]);
            }
            float lo, hi;
            pair_split(acc, lo, hi);
            mean[r] = lo + hi;
        }
#pragma unroll
        for (int r = 0; r < kRows; ++r) mean[r] = warp_allreduce_sum(mean[r]) * inv_cols;
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            const f32x2 neg_mean = pair_of(-mean[r], -mean[r]);
            f32x2 dev2 = pair_of(0.f, 0.f);
#pragma unroll
            for (int j = 0; j < kVecs; ++j) {
                f32x2 part = pair_of(0.f, 0.f);
#pragma unroll
                for (int q = 0; q < kPairsPerVec; ++q) {
                    const f32x2 d = pair_add(x2[r][j * kPairsPerVec + q], neg_mean);
                    x2[r][j * kPairsPerVec + q] = d;  // centred value, reused by the last pass
                    part = pair_fma(d, d, part);
                }
                if (j < my_vecs) dev2 = pair_add(dev2, part);  // a padded vector would add mean^2
            }
            float lo, hi;
            pair_split(dev2, lo, hi);
            rstd[r] = lo + hi;
        }
#pragma unroll
        for (int r = 0; r < kRows; ++r) rstd[r] = rsqrtf(warp_allreduce_sum(rstd[r]) * inv_denom + eps);
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            const int v = lane + 32 * j;
            if (v >= nvec) continue;
            f32x2 g2[kPairsPerVec], b2[kPairsPerVec];
            if (gamma_v) Io::unpack_pairs(__ldg(gamma_v + v), g2);
            if (beta_v) Io::unpack_pairs(__ldg(beta_v + v), b2);
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                if (row0 + r >= row_limit) continue;
                const f32x2 rstd2 = pair_of(rstd[r], rstd[r]);
                f32x2 y2[kPairsPerVec];
#pragma unroll
                for (int q = 0; q < kPairsPerVec; ++q) {
                    f32x2 t = pair_mul(x2[r][j * kPairsPerVec + q], rstd2);
                    if (gamma_v) t = beta_v ? pair_fma(t, g2[q], b2[q]) : pair_mul(t, g2[q]);
                    else if (beta_v) t = pair_add(t, b2[q]);
                    y2[q] = t;
                }
                st_stream(out_v + (row0 + r) * nvec + v, Io::pack_pairs(y2));
            }
        }
    } else {
    Welford stats[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) stats[r] = welford_of_vectors<T, kVecs>(raw[r], my_vecs);
#pragma unroll
    for (int r = 0; r < kRows; ++r) stats[r] = warp_allreduce_welford(stats[r]);
    float mean[kRows], rstd[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        mean[r] = stats[r].mean;
        rstd[r] = rstd_from(stats[r], cols, ddof, eps);
    }
#pragma unroll
    for (int j = 0; j < kVecs; ++j) {
        const int v = lane + 32 * j;
        if (v >= nvec) continue;
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            if (row0 + r >= row_limit) continue;
            st_stream(out_v + (row0 + r) * nvec + v, normalise_vector<T>(raw[r][j], mean[r], rstd[r], gamma_v, beta_v, v));
        }
    }
    }  // long rows
}

// ---------------------------------------------------------------------------------------------
// warp tier: kVecs 16-byte vectors per lane per row, kRows rows per warp step
// ---------------------------------------------------------------------------------------------
template <typename T, int kVecs, int kRows>
__device__ __forceinline__ void layernorm_warp_tier(const T *in, T *out, long long rows, int cols, float eps,
                                                    const T *gamma, const T *beta, int ddof) {
    using Raw = typename RowIo<T>::Raw;
    const int lane = threadIdx.x & 31;
    const int nvec = cols / RowIo<T>::kPerVec;
    const long long warps_per_grid = (long long)gridDim.x * (blockDim.x >> 5);
    const long long warp_global = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const Raw *in_v = reinterpret_cast<const Raw *>(in);
    // vectors this lane owns in a row: lane, lane+32, ...
    int my_vecs = 0;
#pragma unroll
    for (int j = 0; j < kVecs; ++j) my_vecs += (lane + 32 * j < nvec) ? 1 : 0;

    for (long long row0 = warp_global * kRows; row0 < rows; row0 += warps_per_grid * kRows) {
        Raw raw[kRows][kVecs];
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
#pragma unroll
            for (int j = 0; j < kVecs; ++j) {
                const int v = lane + 32 * j;
                if (row0 + r < rows && v < nvec) raw[r][j] = ld_stream(in_v + (row0 + r) * nvec + v);
                else raw[r][j] = Raw{};
            }
        }
        layernorm_rows_from_registers<T, kVecs, kRows>(raw, my_vecs, nvec, lane, row0, rows, reinterpret_cast<Raw *>(out),
                                                       cols, eps, reinterpret_cast<const Raw *>(gamma),
                                                       reinterpret_cast<const Raw *>(beta), ddof);
    }
}

// ---------------------------------------------------------------------------------------------
// group tier: short rows.  A row lives in a group of G lanes (kVecs vectors per lane), a warp works on
// kSlots * 32/G rows per step, warps walk the rows in a grid-stride loop
// ---------------------------------------------------------------------------------------------
// For rows that do not fill 32 lanes, or fill them with so little data that the per-row costs dominate (two 32-lane
// reductions, gamma and beta fetched and unpacked again for every row): the reductions span G lanes only and serve
// 32/G rows per instruction, several independent rows per warp are in flight, and -- a lane owning the same columns
// of every row -- gamma and beta are unpacked to FP32 pairs ONCE, before the row loop.  Statistics are the exact
// two-pass form of the warp tier (group-wide sum -> mean, squared deviations from that mean).
template <int G>
__device__ __forceinline__ float lane_group_sum(float v) {
#pragma unroll
    for (int m = G / 2; m > 0; m >>= 1) v += __shfl_xor_sync(kFullMask, v, m);
    return v;
}

template <typename T, int kVecs, int kSlots, int G>
__device__ __forceinline__ void layernorm_group_tier(const T *in, T *out, long long rows, int cols, float eps,
                                                     const T *gamma, const T *beta, int ddof) {
    using Io = RowIo<T>;
    using Raw = typename Io::Raw;
    constexpr int kPer = Io::kPerVec, kPairsPerVec = kPer / 2, kPairs = kVecs * kPairsPerVec;
    constexpr int kRowsPerSlot = 32 / G, kRowsPerStep = kSlots * kRowsPerSlot;
    const int lane = threadIdx.x & 31, sub = lane / G, gl = lane % G;
    const int nvec = cols / kPer;
    const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
    const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const Raw *in_v = reinterpret_cast<const Raw *>(in);
    Raw *out_v = reinterpret_cast<Raw *>(out);
    const Raw *gamma_v = reinterpret_cast<const Raw *>(gamma), *beta_v = reinterpret_cast<const Raw *>(beta);
    const float inv_cols = 1.0f / (float)cols;
    const float inv_denom = cols - ddof > 0 ? 1.0f / (float)(cols - ddof) : 0.f;
    int my_vecs = 0;
#pragma unroll
    for (int j = 0; j < kVecs; ++j) my_vecs += (gl + G * j < nvec) ? 1 : 0;

    f32x2 g2[kPairs], b2[kPairs];
#pragma unroll
    for (int q = 0; q < kPairs; ++q) {
        g2[q] = pair_of(1.f, 1.f);
        b2[q] = pair_of(0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < kVecs; ++j) {
        const int v = gl + G * j;
        if (v < nvec) {
            if (gamma_v) Io::unpack_pairs(__ldg(gamma_v + v), g2 + j * kPairsPerVec);
            if (beta_v) Io::unpack_pairs(__ldg(beta_v + v), b2 + j * kPairsPerVec);
        }
    }

    for (long long row0 = warp * kRowsPerStep; row0 < rows; row0 += warps * kRowsPerStep) {
        f32x2 x2[kSlots][kPairs];
        float mean[kSlots], rstd[kSlots];
#pragma unroll
        for (int r = 0; r < kSlots; ++r) {
            const long long row = row0 + r * kRowsPerSlot + sub;
            Raw raw[kVecs];
#pragma unroll
            for (int j = 0; j < kVecs; ++j) {
                const int v = gl + G * j;
                if (row < rows && v < nvec) raw[j] = ld_stream(in_v + row * nvec + v);
                else raw[j] = Raw{};
            }
            f32x2 acc = pair_of(0.f, 0.f);
#pragma unroll
            for (int j = 0; j < kVecs; ++j) {
                Io::unpack_pairs(raw[j], x2[r] + j * kPairsPerVec);  // padded vectors are zero
#pragma unroll
                for (int q = 0; q < kPairsPerVec; ++q) acc = pair_add(acc, x2[r][j * kPairsPerVec + q]);
            }
            float lo, hi;
            pair_split(acc, lo, hi);
            mean[r] = lo + hi;
        }
#pragma unroll
        for (int r = 0; r < kSlots; ++r) mean[r] = lane_group_sum<G>(mean[r]) * inv_cols;
#pragma unroll
        for (int r = 0; r < kSlots; ++r) {
            const f32x2 neg_mean = pair_of(-mean[r], -mean[r]);
            f32x2 dev2 = pair_of(0.f, 0.f);
#pragma unroll
            for (int j = 0; j < kVecs; ++j) {
                f32x2 part = pair_of(0.f, 0.f);
#pragma unroll
                for (int q = 0; q < kPairsPerVec; ++q) {
                    const f32x2 d = pair_add(x2[r][j * kPairsPerVec + q], neg_mean);
                    x2[r][j * kPairsPerVec + q] = d;  // centred value, reused by the last pass
                    part = pair_fma(d, d, part);
                }
                if (j < my_vecs) dev2 = pair_add(dev2, part);  // a padded vector would add mean^2
            }
            float lo, hi;
            pair_split(dev2, lo, hi);
            rstd[r] = lo + hi;
        }
#pragma unroll
        for (int r = 0; r < kSlots; ++r) rstd[r] = rsqrtf(lane_group_sum<G>(rstd[r]) * inv_denom + eps);
#pragma unroll
        for (int r = 0; r < kSlots; ++r) {
            const long long row = row0 + r * kRowsPerSlot + sub;
            if (row >= rows) continue;
            const f32x2 rstd2 = pair_of(rstd[r], rstd[r]);
#pragma unroll
            for (int j = 0; j < kVecs; ++j) {
                const int v = gl + G * j;
                if (v >= nvec) continue;
                f32x2 y2[kPairsPerVec];
#pragma unroll
                for (int q = 0; q < kPairsPerVec; ++q)
                    y2[q] = pair_fma(pair_mul(x2[r][j * kPairsPerVec + q], rstd2), g2[j * kPairsPerVec + q], b2[j * kPairsPerVec + q]);
                st_stream(out_v + row * nvec + v, Io::pack_pairs(y2));
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// staged tier: consumer side of the row pipeline (common/row_pipeline.h)
// ---------------------------------------------------------------------------------------------
template <typename T, int kVecs, int kRows, int kConsumerWarps>
__device__ __forceinline__ void layernorm_staged_tier(const T *in, T *out, long long rows, int cols, float eps,
                                                      const T *gamma, const T *beta, int ddof, const RowPipeGeometry geo,
                                                      uint8_t *smem, unsigned *status) {
    using Raw = typename RowIo<T>::Raw;
    const int nvec = cols / RowIo<T>::kPerVec;
    row_pipeline<kConsumerWarps>(in, rows, geo, smem, status,
        [&](const uint8_t *stage, long long first_row, int n, int it, int cw, int lane) {
            int my_vecs = 0;
#pragma unroll
            for (int j = 0; j < kVecs; ++j) my_vecs += (lane + 32 * j < nvec) ? 1 : 0;
            const int full_groups = (geo.rows_per_stage + kRows - 1) / kRows;
            const int groups = (n + kRows - 1) / kRows;
            for (int g = first_group_of_warp(it, full_groups, cw, kConsumerWarps); g < groups; g += kConsumerWarps) {
                const int r0 = g * kRows;
                Raw raw[kRows][kVecs];
#pragma unroll
                for (int r = 0; r < kRows; ++r) {
                    const Raw *row = reinterpret_cast<const Raw *>(stage + (size_t)(r0 + r) * geo.row_bytes);
#pragma unroll
                    for (int j = 0; j < kVecs; ++j) {
                        const int v = lane + 32 * j;
                        if (r0 + r < n && v < nvec) raw[r][j] = row[v];
                        else raw[r][j] = Raw{};
                    }
                }
                layernorm_rows_from_registers<T, kVecs, kRows>(raw, my_vecs, nvec, lane, first_row + r0, first_row + n,
                                                               reinterpret_cast<Raw *>(out), cols, eps,
                                                               reinterpret_cast<const Raw *>(gamma),
                                                               reinterpret_cast<const Raw *>(beta), ddof);
            }
        });
}

// ---------------------------------------------------------------------------------------------
// block tier: one row per thread block, kVecs vectors per thread
// ---------------------------------------------------------------------------------------------
// s_exchange: 3 * 32 floats
__device__ __forceinline__ Welford block_allreduce_welford(Welford w, float *s_exchange) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    w = warp_allreduce_welford(w);
    __syncthreads();
    if (lane == 0) {
        s_exchange[warp] = w.n;
        s_exchange[32 + warp] = w.mean;
        s_exchange[64 + warp] = w.m2;
    }
    __syncthreads();
    Welford t;
    t.n = lane < nwarps ? s_exchange[lane] : 0.f;
    t.mean = lane < nwarps ? s_exchange[32 + lane] : 0.f;
    t.m2 = lane < nwarps ? s_exchange[64 + lane] : 0.f;
    return warp_allreduce_welford(t);
}

template <typename T, int kVecs>
__device__ __forceinline__ void layernorm_block_tier(const T *in, T *out, long long rows, int cols, float eps,
                                                     const T *gamma, const T *beta, int ddof, float *s_exchange) {
    using Io = RowIo<T>;
    using Raw = typename Io::Raw;
    constexpr int kPer = Io::kPerVec;
    const int nvec = cols / kPer;
    const Raw *in_v = reinterpret_cast<const Raw *>(in);
    Raw *out_v = reinterpret_cast<Raw *>(out);
    const Raw *gamma_v = reinterpret_cast<const Raw *>(gamma);
    const Raw *beta_v = reinterpret_cast<const Raw *>(beta);
    int my_vecs = 0;
#pragma unroll
    for (int j = 0; j < kVecs; ++j) my_vecs += ((int)threadIdx.x + (int)blockDim.x * j < nvec) ? 1 : 0;

    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        // all loads first, then one unpack to FP32: the three passes below run on registers
        Raw raw[kVecs];
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            const int v = threadIdx.x + blockDim.x * j;
            if (v < nvec) raw[j] = ld_stream(in_v + row * nvec + v);
            else raw[j] = Raw{};
        }
        float x[kVecs][kPer];
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            Io::unpack(raw[j], x[j]);
#pragma unroll
            for (int e = 0; e < kPer; ++e) sum += x[j][e];  // padded vectors are zero
        }
        Welford w;
        w.n = (float)(my_vecs * kPer);
        w.mean = my_vecs > 0 ? sum / w.n : 0.f;
        float m2 = 0.f;
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            float part = 0.f;
#pragma unroll
            for (int e = 0; e < kPer; ++e) {
                const float d = x[j][e] - w.mean;
                part = fmaf(d, d, part);
            }
            m2 += j < my_vecs ? part : 0.f;
        }
        w.m2 = m2;
        w = block_allreduce_welford(w, s_exchange);
        const float mean = w.mean;
        const float rstd = rstd_from(w, cols, ddof, eps);
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            const int v = threadIdx.x + blockDim.x * j;
            if (v >= nvec) continue;
            float g[kPer], b[kPer], y[kPer];
#pragma unroll
            for (int e = 0; e < kPer; ++e) { g[e] = 1.f; b[e] = 0.f; }
            if (gamma_v) Io::unpack(__ldg(gamma_v + v), g);
            if (beta_v) Io::unpack(__ldg(beta_v + v), b);
#pragma unroll
            for (int e = 0; e < kPer; ++e) y[e] = fmaf((x[j][e] - mean) * rstd, g[e], b[e]);
            st_stream(out_v + row * nvec + v, Io::pack(y));
        }
    }
}

// ---------------------------------------------------------------------------------------------
// resident tier: persistent blocks, one row per block at a time, everything in registers
// ---------------------------------------------------------------------------------------------
// For rows too long for a single warp's registers (e.g. 4096 BF16 columns).  A thread always owns the
// same columns, so gamma and beta are unpacked to FP32 pairs once, outside the row loop; a row is
// unpacked once and its three passes (sum, squared deviations, normalise) run on packed FP32 pairs
// (add/mul/fma.f32x2); the next row's loads are issued before the current row is processed.
// sum over the block; `slot` alternates between calls so that one barrier per call suffices
// (a slot is rewritten only after every thread has passed the barrier of the call in between)
template <int kThreads>
__device__ __forceinline__ float block_sum_fixed(float v, float *s_exchange, int slot) {
    constexpr int kWarps = kThreads / 32;
    v = warp_allreduce_sum(v);
    float *mine = s_exchange + slot * 32;
    if ((threadIdx.x & 31) == 0) mine[threadIdx.x >> 5] = v;
    __syncthreads();
    float total = mine[0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) total += mine[w];  // same order in every thread
    return total;
}

// The statistics of this tier are the exact two-pass form of the Welford/Chan result: every thread
// sums its registers, one block-wide sum gives the row mean, then the squared deviations from that
// mean are summed the same way.  (Merging per-thread (n, mean, M2) triples gives the same numbers but
// costs about 100 instructions per thread and row, which dominates when a thread holds 16 values.)
// kRing > 0: the block's next kRing rows are in flight into shared memory (cp.async, 16 bytes per thread and vector)
// instead of one row into registers.  A thread copies exactly the vectors it will consume, so the ring needs no block
// barrier -- only the thread's own cp.async.wait_group -- and works like extra registers that hold loads in flight:
// with 3 blocks of 256 threads per SM, 3 rows of 8 KB each in flight per block are 72 KB per SM instead of 24 KB.
// ring: kRing * kThreads * kVecs vectors of 16 bytes of (dynamic) shared memory.
template <typename T, int kVecs, int kThreads, bool kAffine, int kRing = 0>
__device__ __forceinline__ void layernorm_resident_tier(const T *in, T *out, long long rows, int cols, float eps,
                                                        const T *gamma, const T *beta, int ddof, float *s_exchange,
                                                        uint4 *ring = nullptr) {
    using Io = RowIo<T>;
    using Raw = typename Io::Raw;
    constexpr int kPer = Io::kPerVec, kPairsPerVec = kPer / 2;
    const int nvec = cols / kPer;
    const Raw *in_v = reinterpret_cast<const Raw *>(in);
    Raw *out_v = reinterpret_cast<Raw *>(out);
    int my_vecs = 0;
#pragma unroll
    for (int j = 0; j < kVecs; ++j) my_vecs += ((int)threadIdx.x + kThreads * j < nvec) ? 1 : 0;
    const float inv_cols = 1.0f / (float)cols;
    const float inv_denom = cols - ddof > 0 ? 1.0f / (float)(cols - ddof) : 0.f;

    f32x2 g2[kAffine ? kVecs * kPairsPerVec : 1], b2[kAffine ? kVecs * kPairsPerVec : 1];
    if constexpr (kAffine) {
        const Raw *gamma_v = reinterpret_cast<const Raw *>(gamma), *beta_v = reinterpret_cast<const Raw *>(beta);
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            const int v = threadIdx.x + kThreads * j;
#pragma unroll
            for (int q = 0; q < kPairsPerVec; ++q) {
                g2[j * kPairsPerVec + q] = pair_of(1.f, 1.f);
                b2[j * kPairsPerVec + q] = pair_of(0.f, 0.f);
            }
            if (v < nvec) {
                if (gamma_v) Io::unpack_pairs(__ldg(gamma_v + v), g2 + j * kPairsPerVec);
                if (beta_v) Io::unpack_pairs(__ldg(beta_v + v), b2 + j * kPairsPerVec);
            }
        }
    }

    Raw next[kVecs];
    auto fetch = [&](long long row) {
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            const int v = threadIdx.x + kThreads * j;
            if (row < rows && v < nvec) next[j] = ld_stream(in_v + row * nvec + v);
            else next[j] = Raw{};
        }
    };
    // ring slot `slot`, vector j of this thread; one commit group per row (empty groups keep the count uniform)
    auto ring_fetch = [&](long long row, int slot) {
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            const int v = threadIdx.x + kThreads * j;
            if (row < rows && v < nvec) {
                const uint32_t dst = smem_u32(ring + (slot * kVecs + j) * kThreads + threadIdx.x);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(in_v + row * nvec + v) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    int slot = 0;
    if constexpr (kRing > 0) {
#pragma unroll
        for (int i = 0; i < kRing; ++i) ring_fetch(blockIdx.x + (long long)i * gridDim.x, i);
    } else {
        fetch(blockIdx.x);
    }
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        f32x2 x2[kVecs * kPairsPerVec];
        if constexpr (kRing > 0) {
            asm volatile("cp.async.wait_group %0;" ::"n"(kRing - 1) : "memory");  // this row's copies have landed
#pragma unroll
            for (int j = 0; j < kVecs; ++j) {
                const int v = threadIdx.x + kThreads * j;
                uint4 r = uint4{0u, 0u, 0u, 0u};
                if (v < nvec) r = ring[(slot * kVecs + j) * kThreads + threadIdx.x];
                Io::unpack_pairs(*reinterpret_cast<const Raw *>(&r), x2 + j * kPairsPerVec);
            }
            ring_fetch(row + (long long)kRing * gridDim.x, slot);  // refill the slot just read (same thread: no hazard)
            slot = slot + 1 == kRing ? 0 : slot + 1;
        } else {
#pragma unroll
            for (int j = 0; j < kVecs; ++j) Io::unpack_pairs(next[j], x2 + j * kPairsPerVec);
            fetch(row + gridDim.x);  // in flight while this row is processed
        }

        f32x2 acc = pair_of(0.f, 0.f);
#pragma unroll
        for (int i = 0; i < kVecs * kPairsPerVec; ++i) acc = pair_add(acc, x2[i]);  // padded vectors are zero
        float lo, hi;
        pair_split(acc, lo, hi);
        const float mean = block_sum_fixed<kThreads>(lo + hi, s_exchange, 0) * inv_cols;
        const f32x2 neg_mean = pair_of(-mean, -mean);
        f32x2 dev2 = pair_of(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            f32x2 part = pair_of(0.f, 0.f);
#pragma unroll
            for (int q = 0; q < kPairsPerVec; ++q) {
                const f32x2 d = pair_add(x2[j * kPairsPerVec + q], neg_mean);
                x2[j * kPairsPerVec + q] = d;  // keep the centred value for the last pass
                part = pair_fma(d, d, part);
            }
            if (j < my_vecs) dev2 = pair_add(dev2, part);  // padded vectors would add mean^2
        }
        pair_split(dev2, lo, hi);
        const float var = block_sum_fixed<kThreads>(lo + hi, s_exchange, 1) * inv_denom;
        const float rstd = rsqrtf(var + eps);
        const f32x2 rstd2 = pair_of(rstd, rstd);
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            const int v = threadIdx.x + kThreads * j;
            if (v >= nvec) continue;
            f32x2 y2[kPairsPerVec];
#pragma unroll
            for (int q = 0; q < kPairsPerVec; ++q) {
                const f32x2 t = pair_mul(x2[j * kPairsPerVec + q], rstd2);
                y2[q] = kAffine ? pair_fma(t, g2[j * kPairsPerVec + q], b2[j * kPairsPerVec + q]) : t;
            }
            st_stream(out_v + row * nvec + v, Io::pack_pairs(y2));
        }
    }
}

// ---------------------------------------------------------------------------------------------
// cluster tier: one row per thread-block cluster, Welford triples exchanged through DSMEM
// ---------------------------------------------------------------------------------------------
// Each block of the cluster holds a contiguous slice of the row in registers and reduces it to one
// (n, mean, M2) triple; the triples sit in each block's shared memory and every block merges all of
// them, in rank order, reading its peers' copies through distributed shared memory.  One cluster
// barrier per row (slots double buffered by row parity); the row is read from HBM once.
// mail: every block pushes its (n, mean, M2) into each peer's mailbox and arrives on that peer's mbarrier, a block
// waits only for its own mailbox (bounded; a timeout is reported through `status`); nullptr: partials are read from
// the peers' shared memory between cluster barriers.
struct WelfordMailbox {
    uint64_t bar[2];
    float value[2][8][3];
};

template <typename T, int kVecs>
__device__ __forceinline__ void layernorm_cluster_tier(const T *in, T *out, long long rows, int cols, float eps,
                                                       const T *gamma, const T *beta, int ddof, float *s_exchange,
                                                       float (*s_part)[3], WelfordMailbox *mail = nullptr,
                                                       unsigned *status = nullptr) {
    namespace cg = cooperative_groups;
    using Raw = typename RowIo<T>::Raw;
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned nblocks = cluster.num_blocks(), rank = cluster.block_rank();
    const int nvec = cols / RowIo<T>::kPerVec;
    const int slice = (nvec + (int)nblocks - 1) / (int)nblocks;
    const int v_begin = (int)rank * slice, v_end = min(nvec, v_begin + slice);
    const Raw *in_v = reinterpret_cast<const Raw *>(in);
    Raw *out_v = reinterpret_cast<Raw *>(out);
    const Raw *gamma_v = reinterpret_cast<const Raw *>(gamma);
    const Raw *beta_v = reinterpret_cast<const Raw *>(beta);
    int my_vecs = 0;
#pragma unroll
    for (int j = 0; j < kVecs; ++j) my_vecs += (v_begin + (int)threadIdx.x + (int)blockDim.x * j < v_end) ? 1 : 0;
    const long long clusters = gridDim.x / nblocks, first = blockIdx.x / nblocks;
    if (mail) {
        if (threadIdx.x == 0) {
            mbar_init(smem_u32(&mail->bar[0]), nblocks);
            mbar_init(smem_u32(&mail->bar[1]), nblocks);
            fence_barrier_init();
        }
        cluster.sync();  // every mailbox is ready before anybody pushes into it
    }
    int parity = 0;
    uint32_t use = 0;  // rows done by this cluster: the mailbox of a parity is on its (use / 2)-th phase
    bool gave_up = false;
    for (long long row = first; row < rows; row += clusters, parity ^= 1, ++use) {
        Raw raw[kVecs];
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            const int v = v_begin + (int)threadIdx.x + (int)blockDim.x * j;
            if (v < v_end) raw[j] = ld_stream(in_v + row * nvec + v);
            else raw[j] = Raw{};
        }
        Welford w = welford_of_vectors<T, kVecs>(raw, my_vecs);
        w = block_allreduce_welford(w, s_exchange);
        Welford all{0.f, 0.f, 0.f};
        if (mail) {
            if (threadIdx.x < nblocks) {
                const uint32_t peer = threadIdx.x;
                const uint32_t slot = map_to_cluster_rank(smem_u32(&mail->value[parity][rank][0]), peer);
                st_cluster_f32(slot, w.n);
                st_cluster_f32(slot + 4, w.mean);
                st_cluster_f32(slot + 8, w.m2);
                mbar_arrive_cluster(map_to_cluster_rank(smem_u32(&mail->bar[parity]), peer));
            }
            if (!mbar_wait_cluster(smem_u32(&mail->bar[parity]), (use >> 1) & 1u) && !gave_up) {
                if (threadIdx.x == 0) atomicCAS(status, 0u, kRowPrefetchTimeout);
                gave_up = true;  // keeps pushing (the peers wait for it) but writes nothing
            }
            for (unsigned r = 0; r < nblocks; ++r)
                all = welford_merge(all, Welford{mail->value[parity][r][0], mail->value[parity][r][1], mail->value[parity][r][2]});
        } else {
            if (threadIdx.x == 0) {
                s_part[parity][0] = w.n;
                s_part[parity][1] = w.mean;
                s_part[parity][2] = w.m2;
            }
            cluster.sync();
            for (unsigned r = 0; r < nblocks; ++r) {
                const float *peer = cluster.map_shared_rank(&s_part[parity][0], r);
                all = welford_merge(all, Welford{peer[0], peer[1], peer[2]});
            }
        }
        const float mean = all.mean, rstd = rstd_from(all, cols, ddof, eps);
#pragma unroll
        for (int j = 0; j < kVecs; ++j) {
            const int v = v_begin + (int)threadIdx.x + (int)blockDim.x * j;
            if (v < v_end && !gave_up) st_stream(out_v + row * nvec + v, normalise_vector<T>(raw[j], mean, rstd, gamma_v, beta_v, v));
        }
    }
    cluster.sync();  // no block may exit while a peer can still read (or write) its shared memory
}

// ---------------------------------------------------------------------------------------------
// reread tier: one row per thread block, two passes, the second one served by the L2
// ---------------------------------------------------------------------------------------------
// For rows longer than one block's registers when there are enough rows to fill every SM several times.  Pass 1
// streams the row once (lines marked evict-last): each thread turns every chunk of kUnroll vectors into an exact
// (count, mean, M2) triple -- mean first, then squared deviations from it, as the block tier does -- and merges it
// into its running triple (Chan); the block merges the threads' triples.  Pass 2 reads the row again, from the L2
// as long as the rows in flight (one per block) fit there, normalises and writes.  No block waits for another.
// Statistics of one row for the reread tier: block-wide (count, mean, M2), every thread gets the result.
template <typename T, int kUnroll>
__device__ __forceinline__ Welford reread_row_stats(const typename RowIo<T>::Raw *x_v, int nvec, uint64_t keep, float *s_exchange) {
    using Io = RowIo<T>;
    using Raw = typename Io::Raw;
    constexpr int kPer = Io::kPerVec;
    const int step = (int)blockDim.x * kUnroll;
    Welford run{0.f, 0.f, 0.f};
    for (int base = 0; base < nvec; base += step) {
        Raw raw[kUnroll];
        int have = 0;
#pragma unroll
        for (int j = 0; j < kUnroll; ++j) {
            const int v = base + (int)threadIdx.x + (int)blockDim.x * j;
            if (v < nvec) {
                raw[j] = ld_keep(x_v + v, keep);
                ++have;
            } else {
                raw[j] = Raw{};
            }
        }
        if (have == 0) continue;
        float x[kUnroll][kPer];
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < kUnroll; ++j) {
            Io::unpack(raw[j], x[j]);
#pragma unroll
            for (int e = 0; e < kPer; ++e) sum += x[j][e];  // padded vectors are zero
        }
        Welford c;
        c.n = (float)(have * kPer);
        c.mean = sum / c.n;
        c.m2 = 0.f;
#pragma unroll
        for (int j = 0; j < kUnroll; ++j) {
            float part = 0.f;
#pragma unroll
            for (int e = 0; e < kPer; ++e) {
                const float d = x[j][e] - c.mean;
                part = fmaf(d, d, part);
            }
            c.m2 += j < have ? part : 0.f;
        }
        run = welford_merge(run, c);
    }
    return block_allreduce_welford(run, s_exchange);
}

// kPair: a block takes two consecutive rows at a time -- statistics of both first, then one joint second pass in
// which a gamma / beta vector is loaded once for both rows (the second pass of an affine row is bound by its three
// loads per output vector, all from the L2; pairing makes that two).
template <typename T, int kStatUnroll, int kUnroll, bool kPair>
__device__ __forceinline__ void layernorm_reread_tier(const T *in, T *out, long long rows, int cols, float eps,
                                                      const T *gamma, const T *beta, int ddof, float *s_exchange) {
    using Io = RowIo<T>;
    using Raw = typename Io::Raw;
    constexpr int kPer = Io::kPerVec;
    constexpr int kRows = kPair ? 2 : 1;
    const int nvec = cols / kPer;
    const int step = (int)blockDim.x * kUnroll;
    const Raw *gamma_v = reinterpret_cast<const Raw *>(gamma);
    const Raw *beta_v = reinterpret_cast<const Raw *>(beta);
    const uint64_t keep = l2_keep_policy();
    for (long long row = (long long)blockIdx.x * kRows; row < rows; row += (long long)gridDim.x * kRows) {
        const Raw *x_v = reinterpret_cast<const Raw *>(in) + row * nvec;
        Raw *y_v = reinterpret_cast<Raw *>(out) + row * nvec;
        const bool second = kPair && row + 1 < rows;
        float mean[kRows], rstd[kRows];
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            if (r == 0 || second) {
                const Welford w = reread_row_stats<T, kStatUnroll>(x_v + (long long)r * nvec, nvec, keep, s_exchange);
                mean[r] = w.mean;
                rstd[r] = rstd_from(w, cols, ddof, eps);
            } else {
                mean[r] = 0.f;
                rstd[r] = 0.f;
            }
        }
        for (int base = 0; base < nvec; base += step) {
            Raw raw[kRows][kUnroll];
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                const int v = base + (int)threadIdx.x + (int)blockDim.x * j;
                if (v < nvec) {
                    raw[0][j] = ld_stream(x_v + v);
                    if (kPair && second) raw[kRows - 1][j] = ld_stream(x_v + nvec + v);
                }
            }
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                const int v = base + (int)threadIdx.x + (int)blockDim.x * j;
                if (v >= nvec) continue;
                if (!kPair) {
                    st_stream(y_v + v, normalise_vector<T>(raw[0][j], mean[0], rstd[0], gamma_v, beta_v, v));
                } else {
                    float g[kPer], b[kPer], x[kPer], y[kPer];
#pragma unroll
                    for (int e = 0; e < kPer; ++e) { g[e] = 1.f; b[e] = 0.f; }
                    if (gamma_v) Io::unpack(__ldg(gamma_v + v), g);
                    if (beta_v) Io::unpack(__ldg(beta_v + v), b);
#pragma unroll
                    for (int r = 0; r < kRows; ++r) {
                        if (r == 1 && !second) continue;
                        Io::unpack(raw[r][j], x);
#pragma unroll
                        for (int e = 0; e < kPer; ++e) y[e] = fmaf((x[e] - mean[r]) * rstd[r], g[e], b[e]);
                        st_stream(y_v + (long long)r * nvec + v, Io::pack(y));
                    }
                }
            }
        }
    }
}

// The single-row reread tier with every row load going through a per-thread shared-memory ring (cp.async): the
// block's work is a stream of items -- (row, pass, chunk of kUnroll vectors per thread) -- and the loads of the next
// kDepth - 1 items are always in flight, across the end of a pass and of a row (see softmax_reread_ring_tier).
// ring: kDepth * kUnroll * kThreads vectors of 16 bytes.
template <typename T, int kUnroll, int kThreads, int kDepth>
__device__ __forceinline__ void layernorm_reread_ring_tier(const T *in, T *out, long long rows, int cols, float eps,
                                                           const T *gamma, const T *beta, int ddof, float *s_exchange,
                                                           uint4 *ring) {
    using Io = RowIo<T>;
    using Raw = typename Io::Raw;
    constexpr int kPer = Io::kPerVec, kStep = kThreads * kUnroll;
    const int nvec = cols / kPer;
    const int chunks = (nvec + kStep - 1) / kStep;
    const Raw *in_v = reinterpret_cast<const Raw *>(in);
    const Raw *gamma_v = reinterpret_cast<const Raw *>(gamma), *beta_v = reinterpret_cast<const Raw *>(beta);
    const uint64_t keep = l2_keep_policy(), once = l2_stream_policy();
    long long p_row = blockIdx.x;
    int p_pass = 0, p_chunk = 0, p_slot = 0;
    auto produce = [&]() {
        if (p_row < rows) {
            const Raw *x_v = in_v + p_row * nvec;
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                const int v = p_chunk * kStep + (int)threadIdx.x + kThreads * j;
                if (v < nvec) cp_async16_policy(ring + (p_slot * kUnroll + j) * kThreads + threadIdx.x, x_v + v, p_pass == 0 ? keep : once);
            }
            if (++p_chunk == chunks) {
                p_chunk = 0;
                if (++p_pass == 2) {
                    p_pass = 0;
                    p_row += gridDim.x;
                }
            }
        }
        cp_async_commit_group();  // also when nothing was issued: one group per item
        p_slot = p_slot + 1 == kDepth ? 0 : p_slot + 1;
    };
#pragma unroll
    for (int i = 0; i < kDepth - 1; ++i) produce();
    int c_slot = 0;
    // this thread's vectors of the item, zero where the row has ended; returns how many are real
    auto consume = [&](int chunk, Raw (&raw)[kUnroll]) -> int {
        produce();  // refills the slot read one item ago (by this same thread)
        cp_async_wait_group<kDepth - 1>();
        int have = 0;
#pragma unroll
        for (int j = 0; j < kUnroll; ++j) {
            const int v = chunk * kStep + (int)threadIdx.x + kThreads * j;
            uint4 r = uint4{0u, 0u, 0u, 0u};
            if (v < nvec) {
                r = ring[(c_slot * kUnroll + j) * kThreads + threadIdx.x];
                ++have;
            }
            raw[j] = *reinterpret_cast<const Raw *>(&r);
        }
        c_slot = c_slot + 1 == kDepth ? 0 : c_slot + 1;
        return have;
    };
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        Raw *y_v = reinterpret_cast<Raw *>(out) + row * nvec;
        Welford run{0.f, 0.f, 0.f};
        for (int chunk = 0; chunk < chunks; ++chunk) {
            Raw raw[kUnroll];
            const int have = consume(chunk, raw);
            if (have == 0) continue;
            float x[kUnroll][kPer];
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                Io::unpack(raw[j], x[j]);
#pragma unroll
                for (int e = 0; e < kPer; ++e) sum += x[j][e];  // padded vectors are zero
            }
            Welford c;
            c.n = (float)(have * kPer);
            c.mean = sum / c.n;
            c.m2 = 0.f;
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                float part = 0.f;
#pragma unroll
                for (int e = 0; e < kPer; ++e) {
                    const float d = x[j][e] - c.mean;
                    part = fmaf(d, d, part);
                }
                c.m2 += j < have ? part : 0.f;
            }
            run = welford_merge(run, c);
        }
        const Welford w = block_allreduce_welford(run, s_exchange);
        const float mean = w.mean;
        const float rstd = rstd_from(w, cols, ddof, eps);
        for (int chunk = 0; chunk < chunks; ++chunk) {
            Raw raw[kUnroll];
            consume(chunk, raw);
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                const int v = chunk * kStep + (int)threadIdx.x + kThreads * j;
                if (v < nvec) st_stream(y_v + v, normalise_vector<T>(raw[j], mean, rstd, gamma_v, beta_v, v));
            }
        }
    }
    cp_async_wait_group<0>();
}

// ---------------------------------------------------------------------------------------------
// stream tier: any cols / alignment; per-thread running Welford, two passes over global memory
// ---------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void layernorm_stream_tier(const T *in, T *out, long long rows, int cols, float eps,
                                                      const T *gamma, const T *beta, int ddof, float *s_exchange) {
    using Io = RowIo<T>;
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const T *x = in + row * cols;
        T *y = out + row * cols;
        Welford w{0.f, 0.f, 0.f};
        for (int c = threadIdx.x; c < cols; c += blockDim.x) {
            // streaming update (the reference's WelfordUpdate, layernorm.h:13-23)
            const float v = Io::to_float(x[c]);
            w.n += 1.f;
            const float d = v - w.mean;
            w.mean += d / w.n;
            w.m2 = fmaf(d, v - w.mean, w.m2);
        }
        w = block_allreduce_welford(w, s_exchange);
        const float mean = w.mean;
        const float rstd = rstd_from(w, cols, ddof, eps);
        for (int c = threadIdx.x; c < cols; c += blockDim.x) {
            const float g = gamma ? Io::to_float(gamma[c]) : 1.f;
            const float b = beta ? Io::to_float(beta[c]) : 0.f;
            y[c] = Io::from_float(fmaf((Io::to_float(x[c]) - mean) * rstd, g, b));
        }
        __syncthreads();
    }
}

// runtime-shape kernels used by the C ABI
template <typename T, int kVecs, int kRows>
__global__ void __launch_bounds__(256) layernorm_warp_kernel(const T *in, T *out, long long rows, int cols, float eps,
                                                             const T *gamma, const T *beta, int ddof) {
    grid_launch_dependents();  // the next kernel of the stream may take SMs as this one's blocks retire
    grid_dependency_wait();    // nothing is read before the previous kernel's writes are visible
    layernorm_warp_tier<T, kVecs, kRows>(in, out, rows, cols, eps, gamma, beta, ddof);
}
template <typename T, int kVecs, int kSlots, int G>
__global__ void __launch_bounds__(256) layernorm_group_kernel(const T *in, T *out, long long rows, int cols, float eps,
                                                              const T *gamma, const T *beta, int ddof) {
    grid_launch_dependents();
    grid_dependency_wait();
    layernorm_group_tier<T, kVecs, kSlots, G>(in, out, rows, cols, eps, gamma, beta, ddof);
}
template <typename T, int kVecs, int kRows, int kConsumerWarps>
__global__ void __launch_bounds__((kConsumerWarps + 1) * 32)
layernorm_staged_kernel(const T *in, T *out, long long rows, int cols, float eps, const T *gamma, const T *beta, int ddof,
                        const RowPipeGeometry geo, unsigned *status) {
    extern __shared__ __align__(128) uint8_t ko_row_stage_smem[];
    layernorm_staged_tier<T, kVecs, kRows, kConsumerWarps>(in, out, rows, cols, eps, gamma, beta, ddof, geo,
                                                           ko_row_stage_smem, status);
}
template <typename T, int kVecs, int kThreads>
__global__ void __launch_bounds__(kThreads) layernorm_block_kernel(const T *in, T *out, long long rows, int cols,
                                                                   float eps, const T *gamma, const T *beta, int ddof) {
    __shared__ float s_exchange[96];
    grid_launch_dependents();
    grid_dependency_wait();
    layernorm_block_tier<T, kVecs>(in, out, rows, cols, eps, gamma, beta, ddof, s_exchange);
}
template <typename T, int kVecs, int kThreads, bool kAffine, int kRing = 0>
__global__ void __launch_bounds__(kThreads) layernorm_resident_kernel(const T *in, T *out, long long rows, int cols,
                                                                      float eps, const T *gamma, const T *beta, int ddof) {
    __shared__ float s_exchange[96];
    extern __shared__ __align__(16) uint4 ko_ln_row_ring[];  // kRing * kThreads * kVecs vectors (dynamic: up to 128 KB)
    grid_launch_dependents();
    grid_dependency_wait();
    layernorm_resident_tier<T, kVecs, kThreads, kAffine, kRing>(in, out, rows, cols, eps, gamma, beta, ddof, s_exchange, ko_ln_row_ring);
}
template <typename T, int kVecs, int kThreads>
__global__ void __launch_bounds__(kThreads) layernorm_cluster_kernel(const T *in, T *out, long long rows, int cols, float eps,
                                                                     const T *gamma, const T *beta, int ddof, unsigned *status,
                                                                     int use_mailbox) {
    __shared__ float s_exchange[96];
    __shared__ float s_part[2][3];
    __shared__ __align__(8) WelfordMailbox s_mail;
    layernorm_cluster_tier<T, kVecs>(in, out, rows, cols, eps, gamma, beta, ddof, s_exchange, s_part, use_mailbox ? &s_mail : nullptr,
                                     status);
}
template <typename T, int kStatUnroll, int kUnroll, int kThreads, bool kPair>
__global__ void __launch_bounds__(kThreads) layernorm_reread_kernel(const T *in, T *out, long long rows, int cols, float eps,
                                                                    const T *gamma, const T *beta, int ddof) {
    grid_launch_dependents();
    grid_dependency_wait();
    __shared__ float s_exchange[96];
    layernorm_reread_tier<T, kStatUnroll, kUnroll, kPair>(in, out, rows, cols, eps, gamma, beta, ddof, s_exchange);
}
template <typename T, int kUnroll, int kThreads, int kDepth>
__global__ void __launch_bounds__(kThreads) layernorm_reread_ring_kernel(const T *in, T *out, long long rows, int cols, float eps,
                                                                         const T *gamma, const T *beta, int ddof) {
    grid_launch_dependents();
    grid_dependency_wait();
    __shared__ float s_exchange[96];
    extern __shared__ __align__(16) uint4 ko_ln_item_ring[];
    layernorm_reread_ring_tier<T, kUnroll, kThreads, kDepth>(in, out, rows, cols, eps, gamma, beta, ddof, s_exchange, ko_ln_item_ring);
}
template <typename T>
__global__ void __launch_bounds__(256) layernorm_stream_kernel(const T *in, T *out, long long rows, int cols, float eps,
                                                               const T *gamma, const T *beta, int ddof) {
    __shared__ float s_exchange[96];
    layernorm_stream_tier<T>(in, out, rows, cols, eps, gamma, beta, ddof, s_exchange);
}

}  // namespace ko

// ---------------------------------------------------------------------------------------------
// reference-named Welford helpers (scalar forms), kept for code written against the reference
// ---------------------------------------------------------------------------------------------
template <typename T>
struct WelfordUpdate {
    __device__ __forceinline__ void operator()(T &count, T &mean, T &m2, const T &new_value) const {
        count += T(1);
        const T delta = new_value - mean;
        mean += delta / count;
        m2 += delta * (new_value - mean);
    }
};

// Merges (count_b, mean_b, m2_b) into the a-triple; m2 is a sum of squared deviations.
template <typename T>
struct WelfordMerge {
    __device__ __forceinline__ void operator()(T &count_a, T &mean_a, T &m2_a, const T &count_b, const T &mean_b,
                                               const T &m2_b) const {
        const T count_ab = count_a + count_b;
        if (count_ab == T(0)) return;
        const T delta = mean_b - mean_a;
        const T w = count_b / count_ab;
        m2_a = m2_a + m2_b + delta * delta * count_a * w;
        mean_a += delta * w;
        count_a = count_ab;
    }
};

// One independent stream per vector slot (the reference's vector form, layernorm.h:25-34).
template <typename T, int N>
struct WelfordUpdate<AlignedArray<T, N>> {
    __device__ __forceinline__ void operator()(AlignedArray<T, N> &count, AlignedArray<T, N> &mean, AlignedArray<T, N> &m2,
                                               const AlignedArray<T, N> &new_value) const {
#pragma unroll
        for (int i = 0; i < N; ++i) WelfordUpdate<T>()(count[i], mean[i], m2[i], new_value[i]);
    }
};

// The combiners below keep the reference's names, argument order and shared-memory footprint
// (layernorm.h:52-62, :64-78, :80-91, :93-126, :128-143).  Unlike the reference's, they
//   * return M2 as the SUM of squared deviations (divide by count - ddof once, after the last
//     combine; the reference's merge divides at every level);
//   * are correct for every block size that is a multiple of 32 (the reference's block forms fold
//     stale lanes in unless blockDim.x == 1024);
//   * leave the warp result in every lane and the block result in every thread, so the *Reduce
//     forms satisfy their "valid in lane 0 / thread 0" contract with room to spare.

// In-place combine of the 32 lanes' triples.
template <typename T>
__device__ __forceinline__ void WelfordWarpReduce(T &result_count, T &result_mean, T &result_m2) {
#pragma unroll
    for (int mask = 16; mask > 0; mask >>= 1) {
        const T other_count = __shfl_xor_sync(0xffffffffu, result_count, mask);
        const T other_mean = __shfl_xor_sync(0xffffffffu, result_mean, mask);
        const T other_m2 = __shfl_xor_sync(0xffffffffu, result_m2, mask);
        WelfordMerge<T>()(result_count, result_mean, result_m2, other_count, other_mean, other_m2);
    }
    // merge(a, b) and merge(b, a) may differ in the last bit: every lane takes lane 0's value
    result_mean = __shfl_sync(0xffffffffu, result_mean, 0);
    result_m2 = __shfl_sync(0xffffffffu, result_m2, 0);
}

// Folds a lane's N per-slot triples into one, then combines the lanes.
template <typename T, int N>
__device__ __forceinline__ void WelfordWarpReduce(const AlignedArray<T, N> &count, const AlignedArray<T, N> &mean,
                                                  const AlignedArray<T, N> &m2, T &result_count, T &result_mean,
                                                  T &result_m2) {
    result_count = count[0];
    result_mean = mean[0];
    result_m2 = m2[0];
#pragma unroll
    for (int i = 1; i < N; ++i) WelfordMerge<T>()(result_count, result_mean, result_m2, count[i], mean[i], m2[i]);
    WelfordWarpReduce<T>(result_count, result_mean, result_m2);
}

template <typename T, int N>
__device__ __forceinline__ void WelfordWarpAllReduce(const AlignedArray<T, N> &count, const AlignedArray<T, N> &mean,
                                                     const AlignedArray<T, N> &m2, T &result_count, T &result_mean,
                                                     T &result_m2) {
    WelfordWarpReduce<T, N>(count, mean, m2, result_count, result_mean, result_m2);  // already in every lane
}

// s_reduce_cache: 3 * 32 elements of T.  Every thread of the block must call it.
template <typename T, int N>
__device__ __forceinline__ void WelfordBlockAllReduce(const AlignedArray<T, N> &count, const AlignedArray<T, N> &mean,
                                                      const AlignedArray<T, N> &m2, T &result_count, T &result_mean,
                                                      T &result_m2, T *s_reduce_cache) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    WelfordWarpReduce<T, N>(count, mean, m2, result_count, result_mean, result_m2);
    __syncthreads();  // the cache may still be read by a previous call
    if (lane == 0) {
        s_reduce_cache[warp] = result_count;
        s_reduce_cache[32 + warp] = result_mean;
        s_reduce_cache[64 + warp] = result_m2;
    }
    __syncthreads();
    // every warp combines the per-warp triples; slots beyond the warp count are empty triples
    result_count = lane < nwarps ? s_reduce_cache[lane] : T(0);
    result_mean = lane < nwarps ? s_reduce_cache[32 + lane] : T(0);
    result_m2 = lane < nwarps ? s_reduce_cache[64 + lane] : T(0);
    WelfordWarpReduce<T>(result_count, result_mean, result_m2);
}

template <typename T, int N>
__device__ __forceinline__ void WelfordBlockReduce(const AlignedArray<T, N> &count, const AlignedArray<T, N> &mean,
                                                   const AlignedArray<T, N> &m2, T &result_count, T &result_mean,
                                                   T &result_m2, T *s_reduce_cache) {
    WelfordBlockAllReduce<T, N>(count, mean, m2, result_count, result_mean, result_m2, s_reduce_cache);
}

// ---------------------------------------------------------------------------------------------
// source-level drop-in for the reference's launch syntax (compile-time shapes)
// ---------------------------------------------------------------------------------------------
// ddof of the drop-in templates: population variance (divide by cols), as in BERT's LayerNorm.
template <typename Element_, int vec_len_, int num_row_, int num_column_, bool elementwise_affine_>
struct LayerNormWarpImpl {
    using Element = Element_;
    static constexpr int vec_len = vec_len_, num_row = num_row_, num_column = num_column_;
    static constexpr bool elementwise_affine = elementwise_affine_;
    static constexpr int smem_in_bytes = 0;
    static constexpr int kPer = ko::RowIo<Element>::kPerVec;
    static_assert(num_column % kPer == 0, "the warp tier moves 128-bit vectors");
    static constexpr int kVecs = (num_column / kPer + 31) / 32;
    static_assert(kVecs <= 16, "row too long for the warp tier; use LayerNormBlockImpl");
    static constexpr int kRows = kVecs <= 4 ? 2 : 1;
    __device__ __forceinline__ static void run(Element *in_data, Element *out_data, Element epsilon,
                                               Element *gamma = nullptr, Element *beta = nullptr) {
        ko::layernorm_warp_tier<Element, kVecs, kRows>(in_data, out_data, num_row, num_column,
                                                       ko::RowIo<Element>::to_float(epsilon),
                                                       elementwise_affine ? gamma : nullptr,
                                                       elementwise_affine ? beta : nullptr, 0);
    }
};

template <typename Element_, int vec_len_, int num_row_, int num_column_, bool elementwise_affine_>
struct LayerNormBlockImpl {
    using Element = Element_;
    static constexpr int vec_len = vec_len_, num_row = num_row_, num_column = num_column_;
    static constexpr bool elementwise_affine = elementwise_affine_;
    static constexpr int smem_in_bytes = 96 * sizeof(float);
    static constexpr int kPer = ko::RowIo<Element>::kPerVec;
    __device__ __forceinline__ static void run(Element *in_data, Element *out_data, Element epsilon,
                                               Element *gamma = nullptr, Element *beta = nullptr) {
        extern __shared__ float ko_layernorm_dyn_smem[];
        Element *g = elementwise_affine ? gamma : nullptr, *b = elementwise_affine ? beta : nullptr;
        const float eps = ko::RowIo<Element>::to_float(epsilon);
        if (num_column % kPer == 0 && num_column / kPer <= 8 * (int)blockDim.x)
            ko::layernorm_block_tier<Element, 8>(in_data, out_data, num_row, num_column, eps, g, b, 0, ko_layernorm_dyn_smem);
        else
            ko::layernorm_stream_tier<Element>(in_data, out_data, num_row, num_column, eps, g, b, 0, ko_layernorm_dyn_smem);
    }
};

template <typename Element_, int vec_len_, int num_row_, int num_column_, bool elementwise_affine_>
struct LayerNormBlockNoCacheImpl {
    using Element = Element_;
    static constexpr int vec_len = vec_len_, num_row = num_row_, num_column = num_column_;
    static constexpr bool elementwise_affine = elementwise_affine_;
    static constexpr int smem_in_bytes = 96 * sizeof(float);
    __device__ __forceinline__ static void run(Element *in_data, Element *out_data, Element epsilon,
                                               Element *gamma = nullptr, Element *beta = nullptr) {
        extern __shared__ float ko_layernorm_dyn_smem[];
        ko::layernorm_stream_tier<Element>(in_data, out_data, num_row, num_column,
                                           ko::RowIo<Element>::to_float(epsilon), elementwise_affine ? gamma : nullptr,
                                           elementwise_affine ? beta : nullptr, 0, ko_layernorm_dyn_smem);
    }
};

template <typename LayerNormKernel>
__global__ void layer_normalization(typename LayerNormKernel::Element *in_data,
                                    typename LayerNormKernel::Element *out_data,
                                    typename LayerNormKernel::Element epsilon,
                                    typename LayerNormKernel::Element *gamma = nullptr,
                                    typename LayerNormKernel::Element *beta = nullptr) {
    LayerNormKernel::run(in_data, out_data, epsilon, gamma, beta);
}
