// Probes of the source-level helper templates: every functor of common/functors.h (scalar and
// AlignedArray forms), to_scalar, limits::numeric_limits, WarpReduce, BlockReduce and the
// reference-named Welford update / merge / warp / block combiners are instantiated in device code
// here and driven with caller-supplied data, so that a host-side test can compare what they compute
// with a CPU restatement.  The kernels are written the way a user of the reference's headers writes
// code (its names, its argument order) -- they are the compile-and-run proof that such code keeps
// working -- and are not on the operator hot path.
#include "ko_internal.h"

#include "../common/common.h"
#include "../common/functors.h"
#include "../nn_operators/layernorm/layernorm.h"

namespace {

enum Functor { kReduceMax = 0, kReduceSum, kExp, kRsqrt, kAdd, kSubtract, kMultiply, kDivide, kMultiplyAdd, kFunctorCount };
enum Form { kScalar = 0, kVectorVector = 1, kVectorScalar = 2 };

template <int F, typename X>
struct Apply;
#define KO_APPLY_BINARY(code, Name)                                                                         \
    template <typename X>                                                                                   \
    struct Apply<code, X> {                                                                                 \
        static constexpr int kArity = 2;                                                                    \
        template <typename B>                                                                               \
        __device__ static X run(const X &a, const B &b, const X &) { return Name<X>()(a, b); }              \
    }
KO_APPLY_BINARY(kReduceMax, ReduceMax);
KO_APPLY_BINARY(kReduceSum, ReduceSum);
KO_APPLY_BINARY(kAdd, Add);
KO_APPLY_BINARY(kSubtract, Subtract);
KO_APPLY_BINARY(kMultiply, Multiply);
KO_APPLY_BINARY(kDivide, Divide);
#undef KO_APPLY_BINARY
template <typename X>
struct Apply<kExp, X> {
    static constexpr int kArity = 1;
    template <typename B>
    __device__ static X run(const X &a, const B &, const X &) { return Exp<X>()(a); }
};
template <typename X>
struct Apply<kRsqrt, X> {
    static constexpr int kArity = 1;
    template <typename B>
    __device__ static X run(const X &a, const B &, const X &) { return Rsqrt<X>()(a); }
};
template <typename X>
struct Apply<kMultiplyAdd, X> {
    static constexpr int kArity = 3;
    __device__ static X run(const X &a, const X &b, const X &c) { return MultiplyAdd<X>()(a, b, c); }
    // no (vector, scalar) form exists for the ternary functor
    template <typename B>
    __device__ static X run(const X &a, const B &, const X &) { return a; }
};

// scalar form: one element per thread
template <int F, typename T>
__global__ void functor_scalar_kernel(const T *a, const T *b, const T *c, T *out, long long n) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= n) return;
    const T bv = Apply<F, T>::kArity >= 2 ? b[i] : a[i];
    const T cv = Apply<F, T>::kArity >= 3 ? c[i] : a[i];
    out[i] = Apply<F, T>::run(a[i], bv, cv);
}

// vector forms: one 16-byte AlignedArray per thread, moved with single 128-bit accesses
template <int F, typename T, bool kScalarRhs>
__global__ void functor_vector_kernel(const T *a, const T *b, const T *c, T *out, long long nvec) {
    constexpr int N = 16 / sizeof(T);
    using Vec = AlignedArray<T, N>;
    static_assert(sizeof(Vec) == 16 && alignof(Vec) == 16, "AlignedArray must be one 128-bit access");
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= nvec) return;
    const Vec av = reinterpret_cast<const Vec *>(a)[i];
    Vec r;
    if constexpr (kScalarRhs) {
        r = Apply<F, Vec>::run(av, b[i], av);  // the scalar operand of vector i is b[i]
    } else {
        const Vec bv = Apply<F, Vec>::kArity >= 2 ? reinterpret_cast<const Vec *>(b)[i] : av;
        const Vec cv = Apply<F, Vec>::kArity >= 3 ? reinterpret_cast<const Vec *>(c)[i] : av;
        r = Apply<F, Vec>::run(av, bv, cv);
    }
    reinterpret_cast<Vec *>(out)[i] = r;
}

template <int F, typename T>
int launch_functor(int form, const void *a, const void *b, const void *c, void *out, long long n, cudaStream_t s) {
    constexpr int N = 16 / sizeof(T);
    const T *ta = static_cast<const T *>(a), *tb = static_cast<const T *>(b), *tc = static_cast<const T *>(c);
    T *to = static_cast<T *>(out);
    if (form == kScalar) {
        functor_scalar_kernel<F, T><<<(unsigned)((n + 127) / 128), 128, 0, s>>>(ta, tb, tc, to, n);
    } else {
        KO_REQUIRE(n % N == 0, KO_ERR_SHAPE, "probe: vector forms need n %% %d == 0", N);
        KO_REQUIRE(ko::aligned16(a) && ko::aligned16(out) && (form == kVectorScalar || Apply<F, T>::kArity < 2 || ko::aligned16(b)) &&
                       (Apply<F, T>::kArity < 3 || ko::aligned16(c)),
                   KO_ERR_ALIGN, "probe: vector forms need 16-byte aligned operands");
        const long long nvec = n / N;
        const unsigned grid = (unsigned)((nvec + 127) / 128);
        if (form == kVectorScalar)
            functor_vector_kernel<F, T, true><<<grid, 128, 0, s>>>(ta, tb, tc, to, nvec);
        else
            functor_vector_kernel<F, T, false><<<grid, 128, 0, s>>>(ta, tb, tc, to, nvec);
    }
    KO_CHECK_LAUNCH("functor probe");
    return KO_OK;
}

template <typename T>
int dispatch_functor(int functor, int form, const void *a, const void *b, const void *c, void *out, long long n,
                     cudaStream_t s) {
    switch (functor) {
        case kReduceMax: return launch_functor<kReduceMax, T>(form, a, b, c, out, n, s);
        case kReduceSum: return launch_functor<kReduceSum, T>(form, a, b, c, out, n, s);
        case kExp: return launch_functor<kExp, T>(form, a, b, c, out, n, s);
        case kRsqrt: return launch_functor<kRsqrt, T>(form, a, b, c, out, n, s);
        case kAdd: return launch_functor<kAdd, T>(form, a, b, c, out, n, s);
        case kSubtract: return launch_functor<kSubtract, T>(form, a, b, c, out, n, s);
        case kMultiply: return launch_functor<kMultiply, T>(form, a, b, c, out, n, s);
        case kDivide: return launch_functor<kDivide, T>(form, a, b, c, out, n, s);
        default: return launch_functor<kMultiplyAdd, T>(form, a, b, c, out, n, s);
    }
}

}  // namespace

extern "C" int ko_probe_functor(int functor, int form, int dtype, const void *a, const void *b, const void *c, void *out,
                                int64_t n, void *stream) {
    KO_REQUIRE(functor >= 0 && functor < kFunctorCount, KO_ERR_INVALID_ARG, "probe: unknown functor %d", functor);
    KO_REQUIRE(form >= kScalar && form <= kVectorScalar, KO_ERR_INVALID_ARG, "probe: unknown form %d", form);
    KO_REQUIRE(n >= 0, KO_ERR_INVALID_ARG, "probe: negative n");
    const int arity = (functor == kExp || functor == kRsqrt) ? 1 : functor == kMultiplyAdd ? 3 : 2;
    KO_REQUIRE(!(form == kVectorScalar && arity != 2), KO_ERR_INVALID_ARG,
               "probe: only binary functors have a (vector, scalar) form");
    if (n == 0) return KO_OK;
    KO_REQUIRE(a && out && (arity < 2 || b) && (arity < 3 || c), KO_ERR_INVALID_ARG, "probe: NULL operand");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case KO_DTYPE_F32: return dispatch_functor<float>(functor, form, a, b, c, out, n, s);
        case KO_DTYPE_F16: return dispatch_functor<half>(functor, form, a, b, c, out, n, s);
        case KO_DTYPE_BF16: return dispatch_functor<__nv_bfloat16>(functor, form, a, b, c, out, n, s);
        default: return ko::fail(KO_ERR_INVALID_ARG, "probe: unknown dtype %d", dtype);
    }
}

// ---------------------------------------------------------------------------------------------
// reductions: WarpReduce, BlockReduce, to_scalar
// ---------------------------------------------------------------------------------------------
namespace {

enum ReduceKind { kWarp = 0, kBlock = 1, kToScalar = 2, kWarpInt32 = 3 };

template <template <typename> typename Op>
__global__ void warp_reduce_kernel(const float *in, float *out) {
    // one warp per block; lane 0 holds the result by the reference's contract
    const float r = WarpReduce<Op, float>(in[blockIdx.x * 32 + threadIdx.x]);
    if (threadIdx.x == 0) out[blockIdx.x] = r;
}

// WarpReduce over int32 keys, starting every lane from the identity built from limits::numeric_limits
__global__ void warp_reduce_int32_kernel(const float *in, float *out) {
    int32_t best = -limits::numeric_limits<int32_t>::max();
    const int32_t mine = __float2int_rn(in[blockIdx.x * 32 + threadIdx.x]);
    best = ReduceMax<int32_t>()(best, mine);
    best = WarpReduce<ReduceMax, int32_t>(best);
    if (threadIdx.x == 0) out[blockIdx.x] = (float)best;
}

// One value per thread, blockDim.x threads per block.  The reduction runs twice back to back on the
// same cache (as a softmax does for max and sum): out[g] is the first result, out[groups + g] the
// second, both read from thread 0.
template <template <typename> typename Op>
__global__ void block_reduce_kernel(const float *in, float *out, long long groups) {
    __shared__ float s_reduce_cache[32];
    const float v = in[blockIdx.x * (long long)blockDim.x + threadIdx.x];
    const float first = BlockReduce<Op, float>(v, s_reduce_cache);
    const float second = BlockReduce<Op, float>(v, s_reduce_cache);
    if (threadIdx.x == 0) {
        out[blockIdx.x] = first;
        out[groups + blockIdx.x] = second;
    }
}

template <typename Op>
__global__ void to_scalar_kernel(const float *in, float *out, long long groups) {
    using Vec = AlignedArray<float, 4>;
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i < groups) out[i] = to_scalar<Op, float, 4>(reinterpret_cast<const Vec *>(in)[i]);
}

__global__ void limits_kernel(float *f32_max, int32_t *i32_max, uint16_t *f16_max, uint16_t *bf16_max) {
    *f32_max = limits::numeric_limits<float>::max();
    *i32_max = limits::numeric_limits<int32_t>::max();
    *f16_max = __half_as_ushort(limits::numeric_limits<half>::max());
    *bf16_max = __bfloat16_as_ushort(limits::numeric_limits<__nv_bfloat16>::max());
}

}  // namespace

extern "C" int ko_probe_reduce(int kind, int op, const float *in, float *out, int64_t groups, int width, void *stream) {
    KO_REQUIRE(kind >= kWarp && kind <= kWarpInt32, KO_ERR_INVALID_ARG, "probe: unknown reduction kind %d", kind);
    KO_REQUIRE(op == 0 || op == 1, KO_ERR_INVALID_ARG, "probe: op must be 0 (max) or 1 (sum)");
    KO_REQUIRE(groups >= 0 && groups <= 0x7fffffff, KO_ERR_INVALID_ARG, "probe: groups out of range");
    if (groups == 0) return KO_OK;
    KO_REQUIRE(in && out, KO_ERR_INVALID_ARG, "probe: NULL operand");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned g = (unsigned)groups;
    if (kind == kWarp) {
        if (op == 0) warp_reduce_kernel<ReduceMax><<<g, 32, 0, s>>>(in, out);
        else warp_reduce_kernel<ReduceSum><<<g, 32, 0, s>>>(in, out);
    } else if (kind == kWarpInt32) {
        warp_reduce_int32_kernel<<<g, 32, 0, s>>>(in, out);
    } else if (kind == kBlock) {
        KO_REQUIRE(width >= 32 && width <= 1024 && width % 32 == 0, KO_ERR_SHAPE,
                   "probe: BlockReduce needs a block of 32..1024 threads, a multiple of 32");
        if (op == 0) block_reduce_kernel<ReduceMax><<<g, width, 0, s>>>(in, out, groups);
        else block_reduce_kernel<ReduceSum><<<g, width, 0, s>>>(in, out, groups);
    } else {
        KO_REQUIRE(ko::aligned16(in), KO_ERR_ALIGN, "probe: to_scalar reads 16-byte vectors");
        if (op == 0) to_scalar_kernel<ReduceMax<float>><<<(g + 127) / 128, 128, 0, s>>>(in, out, groups);
        else to_scalar_kernel<ReduceSum<float>><<<(g + 127) / 128, 128, 0, s>>>(in, out, groups);
    }
    KO_CHECK_LAUNCH("reduction probe");
    return KO_OK;
}

extern "C" int ko_probe_limits(float *f32_max, int32_t *i32_max, uint16_t *f16_max, uint16_t *bf16_max, void *stream) {
    KO_REQUIRE(f32_max && i32_max && f16_max && bf16_max, KO_ERR_INVALID_ARG, "probe: NULL operand");
    limits_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(f32_max, i32_max, f16_max, bf16_max);
    KO_CHECK_LAUNCH("limits probe");
    return KO_OK;
}

// ---------------------------------------------------------------------------------------------
// Welford: WelfordUpdate (scalar and vector), WelfordMerge, WelfordWarpReduce (both overloads),
// WelfordWarpAllReduce, WelfordBlockReduce, WelfordBlockAllReduce.  out is [rows, 3] =
// (count, mean, M2) with M2 the sum of squared deviations.
// ---------------------------------------------------------------------------------------------
namespace {

enum WelfordKind {
    kUpdateSerial = 0,    // one thread per row: WelfordUpdate<float> over the whole row
    kMergeChunks = 1,     // one thread per row: chunks of 32 by WelfordUpdate, chunks joined by WelfordMerge
    kWarpAllReduce = 2,   // one warp per row: WelfordUpdate<AlignedArray<float,4>> + WelfordWarpAllReduce, read from lane 31
    kWarpReduceVec = 3,   // ... + WelfordWarpReduce(count, mean, m2, result...), read from lane 0
    kWarpReduceInPlace = 4,  // one warp per row: scalar updates + WelfordWarpReduce(count, mean, m2) in place, lane 0
    kBlockAllReduce = 5,  // one block per row: vector updates + WelfordBlockAllReduce, read from the last thread
    kBlockReduce = 6      // ... + WelfordBlockReduce, read from thread 0
};

using Vec4 = AlignedArray<float, 4>;

__device__ __forceinline__ void put_triple(float *out, long long row, float count, float mean, float m2) {
    out[row * 3 + 0] = count;
    out[row * 3 + 1] = mean;
    out[row * 3 + 2] = m2;
}

template <int kKind>
__global__ void welford_thread_kernel(const float *in, long long rows, int cols, float *out) {
    const long long row = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (row >= rows) return;
    const float *x = in + row * cols;
    float count = 0.f, mean = 0.f, m2 = 0.f;
    if (kKind == kUpdateSerial) {
        for (int c = 0; c < cols; ++c) WelfordUpdate<float>()(count, mean, m2, x[c]);
    } else {
        for (int c0 = 0; c0 < cols; c0 += 32) {
            float n_b = 0.f, mean_b = 0.f, m2_b = 0.f;
            for (int c = c0; c < min(c0 + 32, cols); ++c) WelfordUpdate<float>()(n_b, mean_b, m2_b, x[c]);
            WelfordMerge<float>()(count, mean, m2, n_b, mean_b, m2_b);
        }
    }
    put_triple(out, row, count, mean, m2);
}

// lane-strided 128-bit loads of one row, one Welford stream per vector slot
__device__ __forceinline__ void accumulate_row(const float *x, int cols, int first, int step, Vec4 &count, Vec4 &mean,
                                               Vec4 &m2) {
    count = 0.f;
    mean = 0.f;
    m2 = 0.f;
    for (int v = first; v < cols / 4; v += step) {
        const Vec4 value = reinterpret_cast<const Vec4 *>(x)[v];
        WelfordUpdate<Vec4>()(count, mean, m2, value);
    }
}

template <int kKind>
__global__ void welford_warp_kernel(const float *in, long long rows, int cols, float *out) {
    const long long row = blockIdx.x;
    const int lane = threadIdx.x;
    const float *x = in + row * cols;
    float count, mean, m2;
    if (kKind == kWarpReduceInPlace) {
        count = mean = m2 = 0.f;
        for (int c = lane; c < cols; c += 32) WelfordUpdate<float>()(count, mean, m2, x[c]);
        WelfordWarpReduce<float>(count, mean, m2);
    } else {
        Vec4 thread_count, thread_mean, thread_m2;
        accumulate_row(x, cols, lane, 32, thread_count, thread_mean, thread_m2);
        if (kKind == kWarpAllReduce) WelfordWarpAllReduce(thread_count, thread_mean, thread_m2, count, mean, m2);
        else WelfordWarpReduce(thread_count, thread_mean, thread_m2, count, mean, m2);
    }
    if (lane == (kKind == kWarpAllReduce ? 31 : 0)) put_triple(out, row, count, mean, m2);
}

template <int kKind>
__global__ void welford_block_kernel(const float *in, long long rows, int cols, float *out) {
    __shared__ float s_reduce_cache[96];
    const long long row = blockIdx.x;
    Vec4 thread_count, thread_mean, thread_m2;
    accumulate_row(in + row * cols, cols, threadIdx.x, blockDim.x, thread_count, thread_mean, thread_m2);
    float count, mean, m2;
    if (kKind == kBlockAllReduce) WelfordBlockAllReduce(thread_count, thread_mean, thread_m2, count, mean, m2, s_reduce_cache);
    else WelfordBlockReduce(thread_count, thread_mean, thread_m2, count, mean, m2, s_reduce_cache);
    if (threadIdx.x == (kKind == kBlockAllReduce ? blockDim.x - 1 : 0)) put_triple(out, row, count, mean, m2);
}

}  // namespace

extern "C" int ko_probe_welford(int kind, const float *in, int64_t rows, int32_t cols, float *out, int block, void *stream) {
    KO_REQUIRE(kind >= kUpdateSerial && kind <= kBlockReduce, KO_ERR_INVALID_ARG, "probe: unknown Welford kind %d", kind);
    KO_REQUIRE(rows >= 0 && rows <= 0x7fffffff && cols >= 1, KO_ERR_INVALID_ARG, "probe: bad shape");
    if (rows == 0) return KO_OK;
    KO_REQUIRE(in && out, KO_ERR_INVALID_ARG, "probe: NULL operand");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned r = (unsigned)rows;
    if (kind != kUpdateSerial && kind != kMergeChunks && kind != kWarpReduceInPlace) {
        KO_REQUIRE(cols % 4 == 0, KO_ERR_SHAPE, "probe: vector Welford forms need cols %% 4 == 0");
        KO_REQUIRE(ko::aligned16(in), KO_ERR_ALIGN, "probe: vector Welford forms read 16-byte vectors");
    }
    switch (kind) {
        case kUpdateSerial: welford_thread_kernel<kUpdateSerial><<<(r + 63) / 64, 64, 0, s>>>(in, rows, cols, out); break;
        case kMergeChunks: welford_thread_kernel<kMergeChunks><<<(r + 63) / 64, 64, 0, s>>>(in, rows, cols, out); break;
        case kWarpAllReduce: welford_warp_kernel<kWarpAllReduce><<<r, 32, 0, s>>>(in, rows, cols, out); break;
        case kWarpReduceVec: welford_warp_kernel<kWarpReduceVec><<<r, 32, 0, s>>>(in, rows, cols, out); break;
        case kWarpReduceInPlace: welford_warp_kernel<kWarpReduceInPlace><<<r, 32, 0, s>>>(in, rows, cols, out); break;
        default:
            KO_REQUIRE(block >= 32 && block <= 1024 && block % 32 == 0, KO_ERR_SHAPE,
                       "probe: block forms need 32..1024 threads, a multiple of 32");
            if (kind == kBlockAllReduce) welford_block_kernel<kBlockAllReduce><<<r, block, 0, s>>>(in, rows, cols, out);
            else welford_block_kernel<kBlockReduce><<<r, block, 0, s>>>(in, rows, cols, out);
    }
    KO_CHECK_LAUNCH("Welford probe");
    return KO_OK;
}

// ---------------------------------------------------------------------------------------------
// Two whole row operators composed ONLY of the helper names above, block per row, three passes over
// global memory: what a user's own kernel on top of these headers looks like.  They prove the pieces
// fit together (Subtract subtracts; BlockReduce and the Welford block forms work at any block size).
// ---------------------------------------------------------------------------------------------
namespace {

__global__ void composed_softmax_kernel(const float *in, float *out, int cols) {
    __shared__ float s_reduce_cache[32];
    __shared__ float s_broadcast[2];
    using Access = AlignedArray<float, 4>;
    const Access *x = reinterpret_cast<const Access *>(in + blockIdx.x * (long long)cols);
    Access *y = reinterpret_cast<Access *>(out + blockIdx.x * (long long)cols);
    const int nvec = cols / 4;

    Access running = -limits::numeric_limits<float>::max();
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) running = ReduceMax<Access>()(running, x[v]);
    float row_max = BlockReduce<ReduceMax, float>(to_scalar<ReduceMax<float>, float, 4>(running), s_reduce_cache);
    if (threadIdx.x == 0) s_broadcast[0] = row_max;
    __syncthreads();
    row_max = s_broadcast[0];

    running = 0.f;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x)
        running = ReduceSum<Access>()(running, Exp<Access>()(Subtract<Access>()(x[v], row_max)));
    float row_sum = BlockReduce<ReduceSum, float>(to_scalar<ReduceSum<float>, float, 4>(running), s_reduce_cache);
    if (threadIdx.x == 0) s_broadcast[1] = row_sum;
    __syncthreads();
    row_sum = s_broadcast[1];

    for (int v = threadIdx.x; v < nvec; v += blockDim.x)
        y[v] = Divide<Access>()(Exp<Access>()(Subtract<Access>()(x[v], row_max)), row_sum);
}

__global__ void composed_layernorm_kernel(const float *in, float *out, int cols, float epsilon, const float *gamma,
                                          const float *beta) {
    __shared__ float s_reduce_cache[96];
    using Access = AlignedArray<float, 4>;
    const Access *x = reinterpret_cast<const Access *>(in + blockIdx.x * (long long)cols);
    Access *y = reinterpret_cast<Access *>(out + blockIdx.x * (long long)cols);
    const int nvec = cols / 4;

    Access thread_count = 0.f, thread_mean = 0.f, thread_m2 = 0.f;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) WelfordUpdate<Access>()(thread_count, thread_mean, thread_m2, x[v]);
    float count, mean, m2;
    WelfordBlockAllReduce(thread_count, thread_mean, thread_m2, count, mean, m2, s_reduce_cache);

    const float rstd = Rsqrt<float>()(Add<float>()(Divide<float>()(m2, count), epsilon));
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
        Access r = Multiply<Access>()(Subtract<Access>()(x[v], mean), rstd);
        if (gamma != nullptr) r = MultiplyAdd<Access>()(r, reinterpret_cast<const Access *>(gamma)[v],
                                                        reinterpret_cast<const Access *>(beta)[v]);
        y[v] = r;
    }
}

}  // namespace

extern "C" int ko_probe_composed_rowop(int op, const float *in, float *out, int64_t rows, int32_t cols, float eps,
                                       const float *gamma, const float *beta, int block, void *stream) {
    KO_REQUIRE(op == 0 || op == 1, KO_ERR_INVALID_ARG, "probe: op must be 0 (softmax) or 1 (LayerNorm)");
    KO_REQUIRE(rows >= 0 && rows <= 0x7fffffff && cols >= 4 && cols % 4 == 0, KO_ERR_SHAPE, "probe: cols must be a multiple of 4");
    KO_REQUIRE(block >= 32 && block <= 1024 && block % 32 == 0, KO_ERR_SHAPE, "probe: block must be 32..1024, a multiple of 32");
    KO_REQUIRE((gamma == nullptr) == (beta == nullptr), KO_ERR_INVALID_ARG, "probe: gamma and beta go together");
    if (rows == 0) return KO_OK;
    KO_REQUIRE(in && out, KO_ERR_INVALID_ARG, "probe: NULL operand");
    KO_REQUIRE(ko::aligned16(in) && ko::aligned16(out) && ko::aligned16(gamma) && ko::aligned16(beta), KO_ERR_ALIGN,
               "probe: 16-byte aligned operands");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (op == 0) composed_softmax_kernel<<<(unsigned)rows, block, 0, s>>>(in, out, cols);
    else composed_layernorm_kernel<<<(unsigned)rows, block, 0, s>>>(in, out, cols, eps, gamma, beta);
    KO_CHECK_LAUNCH("composed row operator probe");
    return KO_OK;
}

// ---------------------------------------------------------------------------------------------
// The reference's tensor-core kernel template, launched the way its driver would
// (nn_operators/gemm/main.cu:179-339, call disabled at :344): half A [M,K], B [K,N], C / D [M,N],
// all row-major, gemm<GemmKernelTensorCore<...>><<<grid, thread_per_block, smem_total_size_in_bytes>>>.
// ---------------------------------------------------------------------------------------------
#include "../nn_operators/gemm/gemm.h"

extern "C" int ko_probe_gemm_tensor_core_template(int64_t M, int64_t N, int64_t K, const uint16_t *A, const uint16_t *B,
                                                  const uint16_t *C, uint16_t *D, void *stream) {
    using Kernel = GemmKernelTensorCore<half, half, half, shape::GemmShape<128, 128, 32>, shape::GemmShape<64, 64, 32>,
                                        shape::GemmShape<16, 8, 8>, 8, 8, 8>;
    KO_REQUIRE(M >= 1 && N >= 1 && K >= 0 && M <= 0x7fffffff && N <= 0x7fffffff && K <= 0x7fffffff, KO_ERR_INVALID_ARG,
               "probe: bad GEMM shape");
    KO_REQUIRE(A && B && D, KO_ERR_INVALID_ARG, "probe: NULL operand");
    const long long tiles = ((M + 127) / 128) * ((N + 127) / 128);
    const unsigned grid = (unsigned)(tiles < 4096 ? tiles : 4096);
    const shape::GemmCoord problem((size_t)M, (size_t)N, (size_t)K);
    // what the reference's driver does before every launch (nn_operators/gemm/main.cu:75-82)
    if (Kernel::smem_total_size_in_bytes >= (48 << 10))
        KO_CUDA(cudaFuncSetAttribute(gemm<Kernel>, cudaFuncAttributeMaxDynamicSharedMemorySize, Kernel::smem_total_size_in_bytes));
    gemm<Kernel><<<grid, Kernel::thread_per_block, Kernel::smem_total_size_in_bytes, static_cast<cudaStream_t>(stream)>>>(
        problem, reinterpret_cast<half *>(const_cast<uint16_t *>(A)), reinterpret_cast<half *>(const_cast<uint16_t *>(B)),
        reinterpret_cast<half *>(const_cast<uint16_t *>(C)), reinterpret_cast<half *>(D));
    KO_CHECK_LAUNCH("gemm<GemmKernelTensorCore>");
    return KO_OK;
}

// ---------------------------------------------------------------------------------------------
// MMA<16,8,8> and LDMatrix<2,false> / <1,true> as the reference's warp loop uses them
// (nn_operators/gemm/tensor_core_gemm.h:207, :218, :231): one warp, D[16,8] = A[16,K] * B[K,8] + C, FP16 everywhere,
// K a multiple of 8 up to 64; A, C, D row-major, B row-major [K,8]
// ---------------------------------------------------------------------------------------------
namespace {
__global__ void __launch_bounds__(32) probe_mma_ldmatrix_kernel(const half *A, const half *B, const half *C, half *D, int K) {
    __shared__ __align__(16) half s_a[16 * 64];
    __shared__ __align__(16) half s_b[64 * 8];
    const int lane = threadIdx.x;
    for (int i = lane; i < 16 * K; i += 32) s_a[(i / K) * 64 + i % K] = A[i];
    for (int i = lane; i < K * 8; i += 32) s_b[i] = B[i];
    __syncwarp();
    const int row = lane >> 2, col = (lane & 3) * 2;
    uint32_t acc[2];
    acc[0] = *reinterpret_cast<const uint32_t *>(C + row * 8 + col);
    acc[1] = *reinterpret_cast<const uint32_t *>(C + (row + 8) * 8 + col);
    for (int k0 = 0; k0 < K; k0 += 8) {
        uint32_t frag_a[2], frag_b;
        // lanes 0..15 address the 16 rows of the A tile (8 halves = 16 bytes each); the other lanes' addresses are ignored
        LDMatrix<2, false>()(frag_a, s_a + (lane % 16) * 64 + k0);
        // lanes 0..7 address the 8 k-rows of the B tile; transposed on the way in: the "col" operand of the MMA
        LDMatrix<1, true>()(&frag_b, s_b + (k0 + lane % 8) * 8);
        MMA<16, 8, 8>()(frag_a, &frag_b, acc, acc);
    }
    *reinterpret_cast<uint32_t *>(D + row * 8 + col) = acc[0];
    *reinterpret_cast<uint32_t *>(D + (row + 8) * 8 + col) = acc[1];
}
}  // namespace

extern "C" int ko_probe_mma_ldmatrix(const uint16_t *A, const uint16_t *B, const uint16_t *C, uint16_t *D, int32_t K, void *stream) {
    KO_REQUIRE(A && B && C && D, KO_ERR_INVALID_ARG, "probe: NULL operand");
    KO_REQUIRE(K >= 8 && K <= 64 && K % 8 == 0, KO_ERR_INVALID_ARG, "probe: K must be a multiple of 8 in [8, 64], got %d", K);
    probe_mma_ldmatrix_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const half *>(A), reinterpret_cast<const half *>(B), reinterpret_cast<const half *>(C), reinterpret_cast<half *>(D), K);
    KO_CHECK_LAUNCH("probe_mma_ldmatrix_kernel");
    return KO_OK;
}
