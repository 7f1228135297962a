// Compile-only check: a translation unit that uses every helper name of the reference's
// common/common.h, common/functors.h and nn_operators/layernorm/layernorm.h:13-143 with the
// reference's template arguments and call shapes must compile against this repository's headers.
// Built by tests/test_helper_names_compile.py with nvcc -c; nothing here is launched.
#include "common/common.h"
#include "common/functors.h"
#include "nn_operators/gemm/gemm.h"
#include "nn_operators/layernorm/layernorm.h"
#include "nn_operators/softmax/softmax.h"

using Access = AlignedArray<float, 4>;
using AccessH = AlignedArray<half, 8>;
static_assert(sizeof(Access) == 16 && alignof(Access) == 16, "128-bit vector of FP32");
static_assert(sizeof(AccessH) == 16 && alignof(AccessH) == 16, "128-bit vector of FP16");
static_assert(Access::kElements == 4 && AccessH::kElements == 8, "kElements");
static_assert(shape::GemmShape<64, 64, 8>::kMN == 4096 && shape::GemmShape<64, 64, 8>::kMK == 512 &&
                  shape::GemmShape<64, 64, 8>::kKN == 512 && shape::GemmShape<64, 64, 8>::kMNK == 32768,
              "GemmShape products");
static_assert(shape::MatrixShape<3, 5>::kM == 3 && shape::MatrixShape<3, 5>::kN == 5, "MatrixShape");

__global__ void every_helper_name(float *data, half *hdata, int32_t *idata) {
    __shared__ float s_reduce_cache[96];
    // AlignedArray: broadcast constructor from a scalar, from an int literal, indexing, at(), clear()
    Access v = *reinterpret_cast<Access *>(data);
    Access acc = -limits::numeric_limits<float>::max();
    Access zero = 0;
    zero.clear();
    acc = ReduceMax<Access>()(acc, v);
    acc = ReduceSum<Access>()(acc, zero);
    acc = Add<Access>()(acc, v);
    acc = Add<Access>()(acc, 1.0f);
    acc = Subtract<Access>()(acc, v);
    acc = Subtract<Access>()(acc, 1.0f);
    acc = Multiply<Access>()(acc, v);
    acc = Multiply<Access>()(acc, 2.0f);
    acc = Divide<Access>()(acc, v);
    acc = Divide<Access>()(acc, 2.0f);
    acc = Exp<Access>()(acc);
    acc = Rsqrt<Access>()(acc);
    acc = MultiplyAdd<Access>()(acc, v, zero);
    acc.at(0) = acc[1];
    float s = to_scalar<ReduceMax<float>, float, 4>(acc) + to_scalar<ReduceSum<float>, float, 4>(acc);
    s = ReduceMax<float>()(s, Exp<float>()(Rsqrt<float>()(MultiplyAdd<float>()(s, s, s))));
    s = WarpReduce<ReduceMax, float>(s) + WarpReduce<ReduceSum, float>(s);
    s = BlockReduce<ReduceMax, float>(s, s_reduce_cache) + BlockReduce<ReduceSum, float>(s, s_reduce_cache);

    // half forms
    AccessH hv = *reinterpret_cast<AccessH *>(hdata);
    AccessH hacc = -limits::numeric_limits<half>::max();
    hacc = ReduceMax<AccessH>()(hacc, hv);
    hacc = Exp<AccessH>()(Subtract<AccessH>()(hv, to_scalar<ReduceMax<half>, half, 8>(hacc)));
    hacc = Rsqrt<AccessH>()(MultiplyAdd<AccessH>()(hacc, hv, hv));
    half hs = Exp<half>()(Rsqrt<half>()(MultiplyAdd<half>()(hacc[0], hacc[1], hacc[2])));
    hs = WarpReduce<ReduceSum, half>(hs);

    int32_t best = -limits::numeric_limits<int32_t>::max();
    best = WarpReduce<ReduceMax, int32_t>(ReduceMax<int32_t>()(best, idata[threadIdx.x]));

    // Welford: scalar and vector updates, merge, the two warp forms, all-reduce, both block forms
    float count = 0, mean = 0, m2 = 0;
    WelfordUpdate<float>()(count, mean, m2, s);
    float count_b = 1, mean_b = 2, m2_b = 0;
    WelfordMerge<float>()(count, mean, m2, count_b, mean_b, m2_b);
    WelfordWarpReduce<float>(count, mean, m2);
    Access thread_count = 0, thread_mean = 0, thread_m2 = 0;
    WelfordUpdate<Access>()(thread_count, thread_mean, thread_m2, v);
    WelfordWarpReduce(thread_count, thread_mean, thread_m2, count, mean, m2);
    WelfordWarpReduce<float, 4>(thread_count, thread_mean, thread_m2, count, mean, m2);
    WelfordWarpAllReduce(thread_count, thread_mean, thread_m2, count, mean, m2);
    WelfordBlockReduce<float, 4>(thread_count, thread_mean, thread_m2, count, mean, m2, s_reduce_cache);
    WelfordBlockAllReduce<float, 4>(thread_count, thread_mean, thread_m2, count, mean, m2, s_reduce_cache);

    *reinterpret_cast<Access *>(data) = acc;
    *reinterpret_cast<AccessH *>(hdata) = hacc;
    data[4] = s + count + mean + m2 + (float)divide_up(7, 2) + (float)const_max(1, 2);
    hdata[8] = hs;
    idata[0] = best;
}

// the reference's warp-level tensor-core helpers (nn_operators/gemm/tensor_core_gemm.h:30-99), in the call shapes of
// its warp loop (:207, :218, :231)
__global__ void tensor_core_helper_names(half *tile_a, half *tile_b, half *out) {
    __shared__ __align__(16) half s_a[16 * 8];
    __shared__ __align__(16) half s_b[8 * 8];
    const int lane_id = threadIdx.x % 32;
    for (int i = lane_id; i < 16 * 8; i += 32) s_a[i] = tile_a[i];
    for (int i = lane_id; i < 8 * 8; i += 32) s_b[i] = tile_b[i];
    __syncwarp();
    AlignedArray<uint32_t, 2> warp_frag_a, warp_frag_accum;
    uint32_t warp_frag_b;
    warp_frag_accum.clear();
    LDMatrix<2, false>()(&warp_frag_a, s_a + (lane_id % 16) * 8);
    LDMatrix<1, true>()(&warp_frag_b, s_b + (lane_id % 8) * 8);
    MMA<16, 8, 8>()(&warp_frag_a, &warp_frag_b, &warp_frag_accum, &warp_frag_accum);
    uint32_t one, two[2];
    LDMatrix<1, false>()(&one, s_b + (lane_id % 8) * 8);
    LDMatrix<2, true>()(two, s_a + (lane_id % 16) * 8);
    *reinterpret_cast<uint32_t *>(out + lane_id * 2) = warp_frag_accum[0] ^ one ^ two[0];
}

// the operator templates and their launch wrappers, with the reference drivers' template arguments
void launch_syntax(float *in, float *out, cudaStream_t stream) {
    using Softmax = SoftMaxWarpImpl<float, 4, 196608, 128>;
    softmax<Softmax><<<320, 128, Softmax::smem_in_bytes, stream>>>(in, out);
    using SoftmaxBlock = SoftMaxBlockImpl<float, 4, 49152, 1024>;
    softmax<SoftmaxBlock><<<320, 128, SoftmaxBlock::smem_in_bytes, stream>>>(in, out);
    using SoftmaxNoCache = SoftMaxBlockNoCacheImpl<float, 4, 49152, 1024>;
    softmax<SoftmaxNoCache><<<320, 128, SoftmaxNoCache::smem_in_bytes, stream>>>(in, out);
    using Ln = LayerNormWarpImpl<float, 4, 16384, 768, false>;
    layer_normalization<Ln><<<320, 128, Ln::smem_in_bytes, stream>>>(in, out, 0.0001f);
    using LnBlock = LayerNormBlockImpl<float, 4, 16384, 768, true>;
    layer_normalization<LnBlock><<<640, 64, LnBlock::smem_in_bytes, stream>>>(in, out, 0.0001f, in, in);
    using LnNoCache = LayerNormBlockNoCacheImpl<float, 4, 16384, 768, false>;
    layer_normalization<LnNoCache><<<640, 64, LnNoCache::smem_in_bytes, stream>>>(in, out, 0.0001f);
    using Gemm = GemmKernelSimt<float, float, float, shape::GemmShape<64, 64, 8>, shape::GemmShape<32, 32, 8>, 4, 4, 4>;
    shape::GemmCoord problem(1024, 1024, 1024);
    gemm<Gemm><<<256, Gemm::thread_per_block, Gemm::smem_total_size_in_bytes, stream>>>(problem, in, in, nullptr, out);
    (void)problem.mk(); (void)problem.kn(); (void)problem.mn(); (void)problem.mnk(); (void)problem.to_string();
    using Tc = GemmKernelTensorCore<half, half, half, shape::GemmShape<128, 128, 32>, shape::GemmShape<64, 64, 32>, shape::GemmShape<16, 8, 8>, 8, 8, 8>;
    half *h_in = reinterpret_cast<half *>(in), *h_out = reinterpret_cast<half *>(out);
    gemm<Tc><<<64, Tc::thread_per_block, Tc::smem_total_size_in_bytes, stream>>>(problem, h_in, h_in, nullptr, h_out);
    checkCudaErrors(cudaGetLastError());
}
