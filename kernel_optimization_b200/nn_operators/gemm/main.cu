// Stand-alone GEMM driver (counterpart of the reference's nn_operators/gemm/main.cu):
//   gemm_driver [--m M --n N --k K] [--iters I] [--bf16 | --f16]
// Default: SGEMM M = N = K = 1024, A and B ~ U(-1,1), seed 2, C overwritten.  With --bf16 / --f16 the
// tcgen05 kernel runs (A row-major, B column-major, FP32 out).  Timed next to cuBLAS and checked
// against it the way the reference does (gemm/main.cu:144-176), with a relative instead of an absolute bound.
#include <cmath>

#include <cublas_v2.h>

#include "../driver_common.h"

int main(int argc, char **argv) {
    const bool bf16 = driver::arg_flag(argc, argv, "--bf16"), f16 = driver::arg_flag(argc, argv, "--f16");
    const bool tc = bf16 || f16;
    const long long M = driver::arg_int(argc, argv, "--m", tc ? 4096 : 1024), N = driver::arg_int(argc, argv, "--n", tc ? 4096 : 1024),
                    K = driver::arg_int(argc, argv, "--k", tc ? 4096 : 1024);
    const int iters = (int)driver::arg_int(argc, argv, "--iters", 20);
    const size_t esz = tc ? 2 : 4;
    const int dtype = bf16 ? KO_DTYPE_BF16 : (f16 ? KO_DTYPE_F16 : KO_DTYPE_F32);

    cudaStream_t stream;
    checkCudaErrors(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    Tensor A((size_t)M * K * esz), B((size_t)K * N * esz), D((size_t)M * N * 4), Dref((size_t)M * N * 4);
    A.fill_uniform(dtype, tc ? 3 : 2, 0, -1.f, 1.f);
    B.fill_uniform(dtype, tc ? 3 : 2, 1, -1.f, 1.f);
    A.host_to_device_async(stream);
    B.host_to_device_async(stream);

    auto ours = [&](int) {
        int st;
        if (bf16) st = ko_gemm_bf16_f32(M, N, K, A.device_ref<uint16_t>(), B.device_ref<uint16_t>(), nullptr, D.device_ref<float>(), stream);
        else if (f16) st = ko_gemm_f16_f32(M, N, K, A.device_ref<uint16_t>(), B.device_ref<uint16_t>(), nullptr, D.device_ref<float>(), stream);
        else st = ko_sgemm_f32(M, N, K, A.device_ref<float>(), B.device_ref<float>(), nullptr, D.device_ref<float>(), stream);
        driver::require_ok(st, "gemm");
    };
    cublasHandle_t blas;
    if (cublasCreate(&blas) != CUBLAS_STATUS_SUCCESS) { std::fprintf(stderr, "cublasCreate failed\n"); return 1; }
    cublasSetStream(blas, stream);
    cublasSetMathMode(blas, CUBLAS_DEFAULT_MATH);
    const float one = 1.f, zero = 0.f;
    auto cublas = [&](int) {
        cublasStatus_t st;
        if (tc) {
            // row-major D[M,N] = A[M,K] * B(col-major [K,N]) is column-major D^T = B^T(op T) * A^T(op N)
            const cudaDataType_t t = bf16 ? CUDA_R_16BF : CUDA_R_16F;
            st = cublasGemmEx(blas, CUBLAS_OP_T, CUBLAS_OP_N, (int)N, (int)M, (int)K, &one, B.device_ref<void>(), t, (int)K,
                              A.device_ref<void>(), t, (int)K, &zero, Dref.device_ref<void>(), CUDA_R_32F, (int)N, CUBLAS_COMPUTE_32F,
                              CUBLAS_GEMM_DEFAULT);
        } else {
            st = cublasSgemm(blas, CUBLAS_OP_N, CUBLAS_OP_N, (int)N, (int)M, (int)K, &one, B.device_ref<float>(), (int)N,
                             A.device_ref<float>(), (int)K, &zero, Dref.device_ref<float>(), (int)N);
        }
        if (st != CUBLAS_STATUS_SUCCESS) { std::fprintf(stderr, "cuBLAS call failed (%d)\n", (int)st); std::exit(1); }
    };
    const double us = driver::time_us(stream, 3, iters, ours);
    const double us_blas = driver::time_us(stream, 3, iters, cublas);
    driver::require_ok(ko_poll_device_status(), "device status");
    D.device_to_host_async(stream);
    Dref.device_to_host_async(stream);
    checkCudaErrors(cudaStreamSynchronize(stream));
    double fro = 0.0;
    driver::require_ok(ko_check_rel_frobenius_f32(D.host_ref<float>(), Dref.host_ref<float>(), M * N, &fro), "check");
    const double tol = tc ? 1e-3 : 1e-5;
    const double tflops = 2.0 * M * N * K / us / 1e6, tflops_blas = 2.0 * M * N * K / us_blas / 1e6;
    std::printf("======Problem size {%lld,%lld,%lld} %s======\n", M, N, K, bf16 ? "bf16->f32 tcgen05" : (f16 ? "f16->f32 tcgen05" : "f32 FFMA"));
    std::printf("Median time %.4fms  %.1f TFLOP/s  (cuBLAS %.4fms %.1f TFLOP/s, ratio %.2f)  rel-Frobenius vs cuBLAS %.3g  %s\n", us / 1e3, tflops,
                us_blas / 1e3, tflops_blas, us_blas / us, fro, fro <= tol ? "Passed." : "FAILED");
    std::printf("{\"op\": \"gemm\", \"m\": %lld, \"n\": %lld, \"k\": %lld, \"us\": %.3f, \"tflops\": %.2f, \"cublas_us\": %.3f, \"vs_cublas\": %.3f}\n", M, N, K, us,
                tflops, us_blas, us_blas / us);
    cublasDestroy(blas);
    return fro <= tol ? 0 : 1;
}
