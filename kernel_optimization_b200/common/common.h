// Shared device/host building blocks of the sm_100a operator set.
//
// Keeps the names the reference project exposes in common/common.h (checkCudaErrors :25,
// WarpReduce :37-46, BlockReduce :48-65, AlignedArray :67-130, to_scalar :138-149,
// limits::numeric_limits :151-178, shape::{GemmCoord,MatrixShape,GemmShape} :180-231) so that
// code written against that header keeps compiling, and adds the `ko` namespace with what the
// Blackwell kernels need: butterfly all-reduces, streaming 128-bit accesses, Chan/Welford
// merging and a cluster-wide exchange.
//
// Deliberate differences from the reference:
//   * BlockReduce is correct for every block size that is a multiple of 32 (the reference
//     folds stale lanes in unless blockDim.x == 1024, common.h:59-63);
//   * WarpReduce leaves the result in every lane, not only lane 0.
#pragma once

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <string>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

// ---------------------------------------------------------------------------------------------
// error handling for the drivers (the C ABI returns status codes instead)
// ---------------------------------------------------------------------------------------------
template <typename T>
void check(T result, char const *const func, const char *const file, int const line) {
    if (result != 0) {
        std::fprintf(stderr, "CUDA error at %s:%d code=%d(%s) \"%s\"\n", file, line,
                     static_cast<int>(result), cudaGetErrorName(static_cast<cudaError_t>(result)), func);
        std::exit(EXIT_FAILURE);
    }
}
#define checkCudaErrors(val) check((val), #val, __FILE__, __LINE__)

__host__ __device__ constexpr int divide_up(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ constexpr int const_max(int a, int b) { return a > b ? a : b; }

// ---------------------------------------------------------------------------------------------
// AlignedArray: N elements of T aligned to the whole vector, so one object moves with a single
// 32/64/128-bit access.
// ---------------------------------------------------------------------------------------------
template <typename T, int N>
struct alignas(sizeof(T) * N) AlignedArray {
    using Element = T;
    static constexpr int kElements = N;

    AlignedArray() = default;
    __host__ __device__ AlignedArray(const T &fill) {
#pragma unroll
        for (int i = 0; i < N; ++i) buffer[i] = fill;
    }
    __host__ __device__ T &operator[](int i) { return buffer[i]; }
    __host__ __device__ const T &operator[](int i) const { return buffer[i]; }
    __host__ __device__ T &at(int i) { return buffer[i]; }
    __host__ __device__ const T &at(int i) const { return buffer[i]; }
    __host__ __device__ void clear() {
#pragma unroll
        for (int i = 0; i < N; ++i) buffer[i] = T(0);
    }

    T buffer[N];
};

template <typename ReductionOp, typename T, int N>
__host__ __device__ __forceinline__ T to_scalar(const AlignedArray<T, N> &v) {
    T acc = v[0];
#pragma unroll
    for (int i = 1; i < N; ++i) acc = ReductionOp()(acc, v[i]);
    return acc;
}

// ---------------------------------------------------------------------------------------------
// warp / block reductions
// ---------------------------------------------------------------------------------------------
// Butterfly over the 32 lanes: every lane ends with the reduced value (a superset of the
// reference's contract, which only defines lane 0).
template <template <typename> typename ReductionOp, typename T>
__device__ __forceinline__ T WarpReduce(T val) {
#pragma unroll
    for (int mask = 16; mask > 0; mask >>= 1) val = ReductionOp<T>()(val, __shfl_xor_sync(0xffffffffu, val, mask));
    return val;
}

// Reduce over the whole thread block; the result is valid in warp 0 (all of its lanes).
// s_reduce_cache needs one T per warp.  Works for any blockDim.x that is a multiple of 32.
template <template <typename> typename ReductionOp, typename T>
__device__ __forceinline__ T BlockReduce(T val, T *s_reduce_cache) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    val = WarpReduce<ReductionOp, T>(val);
    __syncthreads();  // the cache may still be read from a previous reduction
    if (lane == 0) s_reduce_cache[warp] = val;
    __syncthreads();
    if (warp == 0) {
        // lanes beyond the warp count re-read slot 0: harmless for the idempotent ops, and for
        // sums they are masked out by the clamped tree below
        T mine = s_reduce_cache[lane < nwarps ? lane : 0];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            T other = __shfl_down_sync(0xffffffffu, mine, off);
            if (lane + off < nwarps) mine = ReductionOp<T>()(mine, other);
        }
        val = __shfl_sync(0xffffffffu, mine, 0);
    }
    return val;
}

// ---------------------------------------------------------------------------------------------
// numeric limits used as reduction identities
// ---------------------------------------------------------------------------------------------
namespace limits {
template <typename T>
struct numeric_limits;
template <>
struct numeric_limits<float> {
    __host__ __device__ static constexpr float max() { return 3.402823466e+38f; }
};
template <>
struct numeric_limits<int32_t> {
    __host__ __device__ static constexpr int32_t max() { return 2147483647; }
};
template <>
struct numeric_limits<half> {
    __host__ __device__ static half max() { return __ushort_as_half((unsigned short)0x7bffu); }  // 65504
};
template <>
struct numeric_limits<__nv_bfloat16> {
    __host__ __device__ static __nv_bfloat16 max() { return __ushort_as_bfloat16((unsigned short)0x7f7fu); }
};
}  // namespace limits

// ---------------------------------------------------------------------------------------------
// GEMM shapes
// ---------------------------------------------------------------------------------------------
namespace shape {
class GemmCoord {
public:
    __host__ __device__ GemmCoord(size_t m, size_t n, size_t k) : m_(m), n_(n), k_(k) {}
    __host__ __device__ size_t m() const { return m_; }
    __host__ __device__ size_t n() const { return n_; }
    __host__ __device__ size_t k() const { return k_; }
    __host__ __device__ size_t mk() const { return m_ * k_; }
    __host__ __device__ size_t kn() const { return k_ * n_; }
    __host__ __device__ size_t mn() const { return m_ * n_; }
    __host__ __device__ size_t mnk() const { return m_ * n_ * k_; }
    std::string to_string() const {
        return "{" + std::to_string(m_) + "," + std::to_string(n_) + "," + std::to_string(k_) + "}";
    }

private:
    size_t m_, n_, k_;
};

template <int M_, int N_>
struct MatrixShape {
    static constexpr int kM = M_, kN = N_;
};

template <int M_, int N_, int K_>
struct GemmShape {
    static constexpr int kM = M_, kN = N_, kK = K_;
    static constexpr int kMN = M_ * N_, kMK = M_ * K_, kKN = K_ * N_, kMNK = M_ * N_ * K_;
    static std::string to_string() {
        return "{" + std::to_string(kM) + "," + std::to_string(kN) + "," + std::to_string(kK) + "}";
    }
};
}  // namespace shape

// ---------------------------------------------------------------------------------------------
// ko:: device helpers for the Blackwell kernels
// ---------------------------------------------------------------------------------------------
namespace ko {

constexpr unsigned kFullMask = 0xffffffffu;

__device__ __forceinline__ float warp_allreduce_max(float v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v = fmaxf(v, __shfl_xor_sync(kFullMask, v, m));
    return v;
}
__device__ __forceinline__ float warp_allreduce_sum(float v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(kFullMask, v, m);
    return v;
}

// Streaming (evict-first) 128-bit global accesses: row ops touch every byte exactly once.
__device__ __forceinline__ float4 ld_stream(const float4 *p) { return __ldcs(p); }
__device__ __forceinline__ uint4 ld_stream(const uint4 *p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(float4 *p, float4 v) { __stcs(p, v); }
__device__ __forceinline__ void st_stream(uint4 *p, uint4 v) { __stcs(p, v); }

// Loads whose lines should stay in the L2 because the same block reads them a second time soon (the two-pass tiers
// for rows too long for registers): L1 is bypassed, the L2 line is marked evict-last.  The second read uses
// ld_stream, which marks it evict-first again.
__device__ __forceinline__ uint64_t l2_keep_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ float4 ld_keep(const float4 *p, uint64_t policy) {
    float4 v;
    asm volatile("ld.global.L1::no_allocate.L2::cache_hint.v4.f32 {%0, %1, %2, %3}, [%4], %5;"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p), "l"(policy));
    return v;
}

__device__ __forceinline__ uint64_t l2_stream_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
// 16 bytes global -> this thread's shared-memory slot, asynchronously, with an L2 eviction policy; completion through
// cp.async.commit_group / wait_group of the issuing thread
__device__ __forceinline__ void cp_async16_policy(void *smem_dst, const void *src, uint64_t policy) {
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)),
                 "l"(src), "l"(policy)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit_group() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ uint4 ld_keep(const uint4 *p, uint64_t policy) {
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p), "l"(policy));
    return v;
}

// Running (count, mean, M2) triple; M2 is the sum of squared deviations from the mean.
struct Welford {
    float n, mean, m2;
};

// Chan et al. pairwise combination of two partial statistics.  M2 stays a sum of squared
// deviations through every level (the reference divides it by n-1 at each merge,
// layernorm.h:48); the caller divides once at the end.
__device__ __forceinline__ Welford welford_merge(const Welford &a, const Welford &b) {
    Welford r;
    r.n = a.n + b.n;
    float w = 0.5f;  // equal counts (the common case) need no division
    if (a.n != b.n) w = r.n > 0.f ? b.n / r.n : 0.f;
    const float delta = b.mean - a.mean;
    r.mean = fmaf(delta, w, a.mean);
    r.m2 = a.m2 + b.m2 + delta * delta * a.n * w;
    return r;
}

__device__ __forceinline__ Welford warp_allreduce_welford(Welford w) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        Welford o;
        o.n = __shfl_xor_sync(kFullMask, w.n, m);
        o.mean = __shfl_xor_sync(kFullMask, w.mean, m);
        o.m2 = __shfl_xor_sync(kFullMask, w.m2, m);
        w = welford_merge(w, o);
    }
    // merge(a,b) and merge(b,a) can differ in the last bit, so make the lanes agree
    w.mean = __shfl_sync(kFullMask, w.mean, 0);
    w.m2 = __shfl_sync(kFullMask, w.m2, 0);
    return w;
}

// ---------------------------------------------------------------------------------------------
// programmatic dependent launch: a kernel launched with the stream-serialization attribute may have
// its blocks placed on SMs while the previous kernel of the stream is still draining; it must not
// touch global memory before grid_dependency_wait() (which returns once that kernel has completed
// and its writes are visible).  Both are no-ops in a kernel launched the ordinary way.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// fast scalar math for the memory-bound row kernels
// ---------------------------------------------------------------------------------------------
// 2^x on the special-function unit (relative error <= 2^-22; -inf and large negative x give +0)
__device__ __forceinline__ float exp2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// 1/x on the special-function unit (about 1 ulp)
__device__ __forceinline__ float rcp_approx(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// maximum over the warp in one instruction (sm_100a: redux.sync on FP32)
__device__ __forceinline__ float warp_redux_max(float v) {
    float r;
    asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
    return r;
}

// ---------------------------------------------------------------------------------------------
// packed FP32 pairs (sm_100a: add/mul/fma on two IEEE FP32 values per instruction)
// ---------------------------------------------------------------------------------------------
using f32x2 = unsigned long long;
__device__ __forceinline__ f32x2 pair_of(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void pair_split(f32x2 v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2 pair_add(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 pair_mul(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 pair_fma(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// ---------------------------------------------------------------------------------------------
// mbarrier + bulk-copy (TMA) primitives shared by the staged row kernels and the tcgen05 GEMM
// ---------------------------------------------------------------------------------------------
constexpr uint32_t kSpinLimit = 1u << 24;  // polls before a bounded wait gives up

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: false when the limit ran out or another role of the block already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 1023u) == 1023u && *abort_flag) return false;
    }
    return false;
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- distributed shared memory: push a value into a peer block's shared memory and signal its mbarrier
// address of the peer's copy of a shared-memory object of this block (same offset in every block of the cluster)
__device__ __forceinline__ uint32_t map_to_cluster_rank(uint32_t local_smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t cluster_addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_addr), "f"(v) : "memory");
}
// arrive on a peer's mbarrier; release at cluster scope: this thread's earlier stores into the cluster's shared
// memory are visible to whoever observes the arrival with an acquire
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// bounded like mbar_wait
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity) {
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin)
        if (mbar_try_wait_cluster(bar, parity)) return true;
    return false;
}

// 1-D bulk copy global -> this block's shared memory, completion counted in bytes on `bar`.
// Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ float bf16_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

}  // namespace ko
