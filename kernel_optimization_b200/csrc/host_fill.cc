// Seeded, counter-based host fills (ko_fill_*): Philox4x32-10 keyed by (seed, tensor_id) with the
// element index / 4 as the counter, so a value depends only on (seed, tensor_id, element index)
// and is identical for any thread count, shard boundary or call order.
//
// Stands in for the reference drivers' inline fill loops (nn_operators/softmax/main.cu:31-36,
// nn_operators/gemm/main.cu:46-66), whose std::default_random_engine + std::normal_distribution
// stream is library-specific and default-seeded.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <thread>
#include <vector>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ko_internal.h"

namespace {

struct Philox {
    uint32_t key0, key1;
    // ten rounds of the Philox-4x32 bijection on counter (lo, hi, 0, 0)
    void block(uint64_t counter, uint32_t out[4]) const {
        uint32_t c[4] = {static_cast<uint32_t>(counter), static_cast<uint32_t>(counter >> 32), 0u, 0u};
        uint32_t k0 = key0, k1 = key1;
        for (int r = 0; r < 10; ++r) {
            const uint64_t a = 0xD2511F53ull * c[0];
            const uint64_t b = 0xCD9E8D57ull * c[2];
            const uint32_t t0 = static_cast<uint32_t>(b >> 32) ^ c[1] ^ k0;
            const uint32_t t2 = static_cast<uint32_t>(a >> 32) ^ c[3] ^ k1;
            c[1] = static_cast<uint32_t>(b);
            c[3] = static_cast<uint32_t>(a);
            c[0] = t0;
            c[2] = t2;
            k0 += 0x9E3779B9u;
            k1 += 0xBB67AE85u;
        }
        std::memcpy(out, c, sizeof c);
    }
};

inline void store(void *dst, int dtype, int64_t i, double v) {
    const float f = static_cast<float>(v);
    if (dtype == KO_DTYPE_F32) {
        static_cast<float *>(dst)[i] = f;
    } else if (dtype == KO_DTYPE_F16) {
        const __half h = __float2half_rn(f);
        std::memcpy(static_cast<uint16_t *>(dst) + i, &h, 2);
    } else {
        const __nv_bfloat16 h = __float2bfloat16_rn(f);
        std::memcpy(static_cast<uint16_t *>(dst) + i, &h, 2);
    }
}

template <typename Body>
void parallel_for(int64_t n, const Body &body) {
    unsigned hw = std::thread::hardware_concurrency();
    int64_t nthreads = std::max<int64_t>(1, std::min<int64_t>(hw ? hw : 1, n / (1 << 16)));
    nthreads = std::min<int64_t>(nthreads, 64);
    if (nthreads == 1) {
        body(0, n);
        return;
    }
    std::vector<std::thread> pool;
    const int64_t chunk = (n + nthreads - 1) / nthreads;
    for (int64_t t = 0; t < nthreads; ++t) {
        const int64_t lo = t * chunk, hi = std::min(n, lo + chunk);
        if (lo < hi) pool.emplace_back([=, &body] { body(lo, hi); });
    }
    for (auto &th : pool) th.join();
}

int check_fill_args(const void *dst, int dtype, int64_t n, int64_t elem_offset) {
    KO_REQUIRE(n >= 0 && elem_offset >= 0, KO_ERR_INVALID_ARG, "fill: negative count or offset");
    KO_REQUIRE(n == 0 || dst != nullptr, KO_ERR_INVALID_ARG, "fill: NULL destination");
    KO_REQUIRE(dtype == KO_DTYPE_F32 || dtype == KO_DTYPE_F16 || dtype == KO_DTYPE_BF16, KO_ERR_INVALID_ARG,
               "fill: unknown dtype %d", dtype);
    return KO_OK;
}

}  // namespace

extern "C" {

int ko_fill_uniform(void *host_dst, int dtype, int64_t n, uint32_t seed, uint32_t tensor_id, int64_t elem_offset,
                    float lo, float hi) {
    if (int st = check_fill_args(host_dst, dtype, n, elem_offset)) return st;
    const Philox gen{seed, tensor_id};
    const double base = lo, span = static_cast<double>(hi) - static_cast<double>(lo);
    parallel_for(n, [&](int64_t begin, int64_t end) {
        for (int64_t i = begin; i < end; ++i) {
            const uint64_t e = static_cast<uint64_t>(elem_offset + i);
            uint32_t w[4];
            gen.block(e >> 2, w);
            // top 24 bits, centred in their cell: strictly inside (0,1)
            const double u = (static_cast<double>(w[e & 3] >> 8) + 0.5) * 0x1p-24;
            store(host_dst, dtype, i, base + span * u);
        }
    });
    return KO_OK;
}

int ko_fill_normal(void *host_dst, int dtype, int64_t n, uint32_t seed, uint32_t tensor_id, int64_t elem_offset,
                   float mean, float stddev) {
    if (int st = check_fill_args(host_dst, dtype, n, elem_offset)) return st;
    const Philox gen{seed, tensor_id};
    constexpr double kTwoPi = 6.283185307179586476925286766559;
    parallel_for(n, [&](int64_t begin, int64_t end) {
        for (int64_t i = begin; i < end; ++i) {
            const uint64_t e = static_cast<uint64_t>(elem_offset + i);
            uint32_t w[4];
            gen.block(e >> 2, w);
            // Box-Muller: words (0,1) give elements 4b, 4b+1; words (2,3) give 4b+2, 4b+3
            const int pair = static_cast<int>((e >> 1) & 1);
            const double u1 = (static_cast<double>(w[2 * pair]) + 0.5) * 0x1p-32;
            const double u2 = (static_cast<double>(w[2 * pair + 1]) + 0.5) * 0x1p-32;
            const double radius = std::sqrt(-2.0 * std::log(u1));
            const double z = (e & 1) ? radius * std::sin(kTwoPi * u2) : radius * std::cos(kTwoPi * u2);
            store(host_dst, dtype, i, static_cast<double>(mean) + static_cast<double>(stddev) * z);
        }
    });
    return KO_OK;
}

int ko_fill_causal_mask_f32(float *host_dst, int64_t rows, int32_t cols, int64_t row_offset, int32_t block,
                            float value) {
    KO_REQUIRE(rows >= 0 && cols >= 0 && row_offset >= 0 && block > 0, KO_ERR_INVALID_ARG,
               "causal mask: bad shape [%lld, %d], offset %lld, block %d", (long long)rows, cols,
               (long long)row_offset, block);
    KO_REQUIRE(rows == 0 || cols == 0 || host_dst != nullptr, KO_ERR_INVALID_ARG, "causal mask: NULL destination");
    parallel_for(rows, [&](int64_t begin, int64_t end) {
        for (int64_t r = begin; r < end; ++r) {
            const int64_t first_masked = (row_offset + r) % block + 1;
            float *row = host_dst + r * static_cast<int64_t>(cols);
            for (int64_t c = first_masked; c < cols; ++c) row[c] = value;
        }
    });
    return KO_OK;
}

}  // extern "C"
