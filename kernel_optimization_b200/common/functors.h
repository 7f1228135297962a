// Reduction and elementwise functors, scalar and AlignedArray forms.
//
// Same names and call shapes as the reference's common/functors.h (ReduceMax :13-34,
// ReduceSum :37-58, Exp :60-92, Rsqrt :94-126, Add :129-162, Subtract :164-197,
// Multiply :199-232, Divide :234-267, MultiplyAdd :269-301).  The vector forms are produced by
// one lifting template instead of being written out per functor.
//
// Deliberate differences from the reference:
//   * Subtract subtracts (the reference returns a + b, functors.h:168);
//   * MultiplyAdd<float> rounds to nearest (the reference rounds toward -inf, functors.h:274);
//   * __nv_bfloat16 specialisations exist beside the half ones.
#pragma once

#include "common.h"

namespace ko {
namespace detail {

// Applies a scalar binary functor lane by lane: (vector, vector) and (vector, scalar).
template <typename ScalarOp, typename T, int N>
struct LiftBinary {
    using Vec = AlignedArray<T, N>;
    __host__ __device__ __forceinline__ Vec operator()(const Vec &a, const Vec &b) const {
        Vec r;
#pragma unroll
        for (int i = 0; i < N; ++i) r[i] = ScalarOp()(a[i], b[i]);
        return r;
    }
    __host__ __device__ __forceinline__ Vec operator()(const Vec &a, const T &b) const {
        Vec r;
#pragma unroll
        for (int i = 0; i < N; ++i) r[i] = ScalarOp()(a[i], b);
        return r;
    }
};

template <typename ScalarOp, typename T, int N>
struct LiftUnary {
    using Vec = AlignedArray<T, N>;
    __host__ __device__ __forceinline__ Vec operator()(const Vec &a) const {
        Vec r;
#pragma unroll
        for (int i = 0; i < N; ++i) r[i] = ScalarOp()(a[i]);
        return r;
    }
};

template <typename ScalarOp, typename T, int N>
struct LiftTernary {
    using Vec = AlignedArray<T, N>;
    __host__ __device__ __forceinline__ Vec operator()(const Vec &a, const Vec &b, const Vec &c) const {
        Vec r;
#pragma unroll
        for (int i = 0; i < N; ++i) r[i] = ScalarOp()(a[i], b[i], c[i]);
        return r;
    }
};

}  // namespace detail
}  // namespace ko

#define KO_BINARY_FUNCTOR(Name, expr)                                                         \
    template <typename T>                                                                     \
    struct Name {                                                                             \
        __host__ __device__ __forceinline__ T operator()(const T &a, const T &b) const { return (expr); } \
    };                                                                                        \
    template <typename T, int N>                                                              \
    struct Name<AlignedArray<T, N>> : ko::detail::LiftBinary<Name<T>, T, N> {}

KO_BINARY_FUNCTOR(ReduceMax, a > b ? a : b);
KO_BINARY_FUNCTOR(ReduceSum, a + b);
KO_BINARY_FUNCTOR(Add, a + b);
KO_BINARY_FUNCTOR(Subtract, a - b);
KO_BINARY_FUNCTOR(Multiply, a * b);
KO_BINARY_FUNCTOR(Divide, a / b);
#undef KO_BINARY_FUNCTOR

template <typename T>
struct Exp;
template <>
struct Exp<float> {
    __device__ __forceinline__ float operator()(const float &a) const { return expf(a); }
};
template <>
struct Exp<half> {
    __device__ __forceinline__ half operator()(const half &a) const { return hexp(a); }
};
template <>
struct Exp<__nv_bfloat16> {
    __device__ __forceinline__ __nv_bfloat16 operator()(const __nv_bfloat16 &a) const { return hexp(a); }
};
template <typename T, int N>
struct Exp<AlignedArray<T, N>> : ko::detail::LiftUnary<Exp<T>, T, N> {};

template <typename T>
struct Rsqrt;
template <>
struct Rsqrt<float> {
    __device__ __forceinline__ float operator()(const float &a) const { return rsqrtf(a); }
};
template <>
struct Rsqrt<half> {
    __device__ __forceinline__ half operator()(const half &a) const { return hrsqrt(a); }
};
template <>
struct Rsqrt<__nv_bfloat16> {
    __device__ __forceinline__ __nv_bfloat16 operator()(const __nv_bfloat16 &a) const { return hrsqrt(a); }
};
template <typename T, int N>
struct Rsqrt<AlignedArray<T, N>> : ko::detail::LiftUnary<Rsqrt<T>, T, N> {};

template <typename T>
struct MultiplyAdd;
template <>
struct MultiplyAdd<float> {
    __device__ __forceinline__ float operator()(const float &a, const float &b, const float &c) const {
        return __fmaf_rn(a, b, c);
    }
};
template <>
struct MultiplyAdd<half> {
    __device__ __forceinline__ half operator()(const half &a, const half &b, const half &c) const {
        return __hfma(a, b, c);
    }
};
template <>
struct MultiplyAdd<__nv_bfloat16> {
    __device__ __forceinline__ __nv_bfloat16 operator()(const __nv_bfloat16 &a, const __nv_bfloat16 &b,
                                                        const __nv_bfloat16 &c) const {
        return __hfma(a, b, c);
    }
};
template <typename T, int N>
struct MultiplyAdd<AlignedArray<T, N>> : ko::detail::LiftTernary<MultiplyAdd<T>, T, N> {};
