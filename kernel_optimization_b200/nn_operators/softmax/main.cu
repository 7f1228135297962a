// Stand-alone softmax driver (counterpart of the reference's nn_operators/softmax/main.cu):
//   softmax_driver [--rows R] [--cols C] [--iters N] [--sets S] [--seed X] [--causal]
// Default: BERT-Base attention shape FP32 [196608, 128], logits N(0, 2^2), seed 0.
#include "../driver_common.h"

int main(int argc, char **argv) {
    const long long rows = driver::arg_int(argc, argv, "--rows", 128 * 12 * 128);
    const int cols = (int)driver::arg_int(argc, argv, "--cols", 128);
    const int iters = (int)driver::arg_int(argc, argv, "--iters", 50);
    const int sets = (int)driver::arg_int(argc, argv, "--sets", 4);
    const unsigned seed = (unsigned)driver::arg_int(argc, argv, "--seed", 0);
    const size_t bytes = (size_t)rows * cols * sizeof(float);

    cudaStream_t stream;
    checkCudaErrors(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    std::vector<Tensor> in, out;
    for (int s = 0; s < sets; ++s) {
        in.emplace_back(bytes);
        out.emplace_back(bytes);
    }
    in[0].fill_normal(KO_DTYPE_F32, seed, 0, 0.f, 2.f);
    if (driver::arg_flag(argc, argv, "--causal"))
        driver::require_ok(ko_fill_causal_mask_f32(in[0].host_ref<float>(), rows, cols, 0, 512, -1e4f), "causal mask");
    for (int s = 0; s < sets; ++s) {
        if (s) std::memcpy(in[s].host_ref<float>(), in[0].host_ref<float>(), bytes);
        in[s].host_to_device_async(stream);
    }
    const double us = driver::time_us(stream, 5, iters, [&](int i) {
        driver::require_ok(ko_softmax_f32(in[i % sets].device_ref<float>(), out[i % sets].device_ref<float>(), rows, cols, stream),
                           "ko_softmax_f32");
    });
    out[0].device_to_host_async(stream);
    checkCudaErrors(cudaStreamSynchronize(stream));
    double rowsum_err = 0.0;
    driver::require_ok(ko_check_max_rowsum_err_f32(out[0].host_ref<float>(), rows, cols, &rowsum_err), "row-sum check");
    const double gbs = 2.0 * bytes / us / 1e3;
    std::printf("======Num row %lld, num column %d======\n", rows, cols);
    std::printf("Median time %.4fms  %.0f GB/s  max |rowsum-1| %.3g  %s\n", us / 1e3, gbs, rowsum_err, rowsum_err <= 1e-5 ? "Passed." : "FAILED");
    std::printf("{\"op\": \"softmax_f32\", \"rows\": %lld, \"cols\": %d, \"us\": %.3f, \"gbs\": %.1f, \"rowsum_err\": %.3g}\n", rows, cols, us, gbs, rowsum_err);
    return rowsum_err <= 1e-5 ? 0 : 1;
}
