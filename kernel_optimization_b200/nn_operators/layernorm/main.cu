// Stand-alone LayerNorm driver (counterpart of the reference's nn_operators/layernorm/main.cu):
//   layernorm_driver [--rows R] [--cols C] [--iters N] [--sets S] [--seed X] [--bf16] [--ddof D]
// Default: BERT-Base hidden shape FP32 [16384, 768], x ~ N(0,1), gamma ~ U(0.5,1.5), beta ~ N(0,0.1^2),
// eps 1e-12, seed 1.  The check runs a second, un-affined pass and verifies mean 0 / variance 1 per row.
#include <cmath>

#include "../driver_common.h"

int main(int argc, char **argv) {
    const long long rows = driver::arg_int(argc, argv, "--rows", 128 * 128);
    const int cols = (int)driver::arg_int(argc, argv, "--cols", 768);
    const int iters = (int)driver::arg_int(argc, argv, "--iters", 50);
    const int sets = (int)driver::arg_int(argc, argv, "--sets", 8);
    const unsigned seed = (unsigned)driver::arg_int(argc, argv, "--seed", 1);
    const int ddof = (int)driver::arg_int(argc, argv, "--ddof", 0);
    const bool bf16 = driver::arg_flag(argc, argv, "--bf16");
    const int dtype = bf16 ? KO_DTYPE_BF16 : KO_DTYPE_F32;
    const size_t esz = bf16 ? 2 : 4, bytes = (size_t)rows * cols * esz;
    const float eps = 1e-12f;

    cudaStream_t stream;
    checkCudaErrors(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    std::vector<Tensor> in, out;
    for (int s = 0; s < sets; ++s) {
        in.emplace_back(bytes);
        out.emplace_back(bytes);
    }
    Tensor gamma((size_t)cols * esz), beta((size_t)cols * esz);
    in[0].fill_normal(dtype, seed, 0, 0.f, 1.f);
    gamma.fill_uniform(dtype, seed, 1, 0.5f, 1.5f);
    beta.fill_normal(dtype, seed, 2, 0.f, 0.1f);
    gamma.host_to_device_async(stream);
    beta.host_to_device_async(stream);
    for (int s = 0; s < sets; ++s) {
        if (s) std::memcpy(in[s].host_ref<char>(), in[0].host_ref<char>(), bytes);
        in[s].host_to_device_async(stream);
    }
    auto run = [&](int i, bool affine) {
        void *x = in[i % sets].device_ref<void>(), *y = out[i % sets].device_ref<void>();
        const void *g = affine ? gamma.device_ref<void>() : nullptr, *b = affine ? beta.device_ref<void>() : nullptr;
        const int st = bf16 ? ko_layernorm_bf16((const uint16_t *)x, (uint16_t *)y, rows, cols, eps, (const uint16_t *)g, (const uint16_t *)b, ddof, stream)
                            : ko_layernorm_f32((const float *)x, (float *)y, rows, cols, eps, (const float *)g, (const float *)b, ddof, stream);
        driver::require_ok(st, "ko_layernorm");
    };
    const double us = driver::time_us(stream, 5, iters, [&](int i) { run(i, true); });
    run(0, false);
    out[0].device_to_host_async(stream);
    checkCudaErrors(cudaStreamSynchronize(stream));
    double worst_mean = 0.0, worst_var = 0.0;
    const long long check_rows = std::min<long long>(rows, 2048);
    for (long long r = 0; r < check_rows; ++r) {
        double s = 0.0, s2 = 0.0;
        for (int c = 0; c < cols; ++c) {
            double v;
            if (bf16) {
                const uint32_t bits = (uint32_t)out[0].host_ref<uint16_t>()[r * cols + c] << 16;
                float f;
                std::memcpy(&f, &bits, 4);
                v = f;
            } else {
                v = out[0].host_ref<float>()[r * cols + c];
            }
            s += v;
            s2 += v * v;
        }
        const double mean = s / cols, var = s2 / cols - mean * mean;
        worst_mean = std::max(worst_mean, std::fabs(mean));
        worst_var = std::max(worst_var, std::fabs(var * cols / (cols - ddof) - 1.0));
    }
    const double tol = bf16 ? 2e-2 : 1e-4;
    const bool ok = worst_mean <= tol && worst_var <= tol;
    const double gbs = 2.0 * bytes / us / 1e3;
    std::printf("======Num row %lld, num column %d (%s)======\n", rows, cols, bf16 ? "bf16" : "f32");
    std::printf("Median time %.4fms  %.0f GB/s  |mean| %.3g  |var-1| %.3g  %s\n", us / 1e3, gbs, worst_mean, worst_var, ok ? "Passed." : "FAILED");
    std::printf("{\"op\": \"layernorm_%s\", \"rows\": %lld, \"cols\": %d, \"us\": %.3f, \"gbs\": %.1f}\n", bf16 ? "bf16" : "f32", rows, cols, us, gbs);
    return ok ? 0 : 1;
}
