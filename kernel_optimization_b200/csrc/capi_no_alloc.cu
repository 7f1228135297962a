// ko_sgemm_f32_no_alloc: the split-K SGEMM for callers that must not allocate device memory.
//
// Who needs this.  ko_sgemm_f32 keeps its split-K partial tiles in a buffer it obtains from
// cudaMalloc the first time a stream needs one.  Some hosts cannot let a library do that: a serving
// process that has handed the whole GPU to its own pool allocator (a later cudaMalloc simply fails),
// a latency-critical loop that cannot tolerate the device-wide synchronisation an allocation may
// imply, or code that runs where the allocation calls are off limits altogether.  For them this
// entry point runs the same kernel with its scratch in a fixed array that is part of the library
// image: nothing is allocated or freed, here or in any routine this file calls.
//
// The price.  The array has a fixed size (kMaxPartialFloats partial-tile floats and kMaxTiles arrival
// counters, see below); every GPU that loads the library carries it until the process exits; a split
// that needs more is refused with KO_ERR_SHAPE rather than shrunk silently.  All calls on a device
// share the one array and it keeps whatever the previous call left there: the arrival counters are
// cleared on the stream before every launch, the partial tiles are fully rewritten before they are
// read.  Two calls whose kernels overlap on the GPU (different streams, or the same call from two
// threads) therefore race on the scratch; callers must order them.
//
// Set-up.  In host code the array's name is only a handle, not a device address, so the first call
// on each device asks the runtime for the real address (cudaGetSymbolAddress, with that device
// current) and raises the kernel's dynamic shared-memory limit; later calls reuse both.  Make that
// first call per device during initialisation, before any stream capture begins.
#include "ko_internal.h"

#include <mutex>

#include "../nn_operators/gemm/simt_gemm_x2.h"

namespace {

namespace x2 = ko::sgemm2;
using Wide = x2::Shape<2, 2>;  // 128 x 128 tiles, one group of 4 warps per block

constexpr size_t kMaxPartialFloats = (size_t)2 << 20;  // 2 Mi floats = 8 MiB, e.g. 1024 x 1024 outputs in 2 K-slices
constexpr size_t kMaxTiles = 128;                      // arrival counters (one per 128 x 128 output tile; a split needs
                                                       // tiles * split_k <= 128 partial tiles, so at most 64 tiles ever split)
constexpr size_t kCounterOffset = kMaxPartialFloats * sizeof(float);
constexpr size_t kScratchBytes = kCounterOffset + kMaxTiles * sizeof(unsigned);

static __device__ __align__(256) unsigned char g_no_alloc_scratch[kScratchBytes];

struct DeviceSetup {
    bool ready = false;
    unsigned char *scratch = nullptr;  // device address of g_no_alloc_scratch on this device
};

// once per device, with that device current
int setup_for_current_device(DeviceSetup **out) {
    static std::mutex mu;
    static DeviceSetup per_device[64];
    int dev = -1;
    KO_CUDA(cudaGetDevice(&dev));
    KO_REQUIRE(dev >= 0 && dev < 64, KO_ERR_NO_DEVICE, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    DeviceSetup &st = per_device[dev];
    if (!st.ready) {
        unsigned char *ptr = nullptr;
        KO_CUDA(cudaGetSymbolAddress((void **)&ptr, g_no_alloc_scratch));
        KO_REQUIRE(ptr != nullptr, KO_ERR_CUDA, "cudaGetSymbolAddress returned a null scratch address");
        KO_CUDA(cudaFuncSetAttribute(x2::sgemm_x2_kernel<true, 2, 2, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, Wide::smem_bytes(1)));
        KO_CUDA(cudaFuncSetAttribute(x2::sgemm_x2_kernel<false, 2, 2, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, Wide::smem_bytes(1)));
        st.scratch = ptr;
        st.ready = true;
    }
    *out = &st;
    return KO_OK;
}

}  // namespace

extern "C" int ko_sgemm_f32_no_alloc(int64_t M, int64_t N, int64_t K, const float *A, const float *B, const float *C,
                                     float *D, int split_k, void *stream) {
    KO_REQUIRE(M >= 0 && N >= 0 && K >= 0, KO_ERR_INVALID_ARG, "sgemm (no-alloc): negative shape {%lld,%lld,%lld}",
               (long long)M, (long long)N, (long long)K);
    KO_REQUIRE(split_k >= 0 && split_k <= 64, KO_ERR_INVALID_ARG, "sgemm (no-alloc): split_k %d out of range", split_k);
    if (M == 0 || N == 0) return KO_OK;
    if (K == 0) return ko_sgemm_f32(M, N, K, A, B, C, D, stream);  // empty sum: no scratch involved
    KO_REQUIRE(M <= 0x7fffffff && N <= 0x7fffffff && K <= 0x7fffffff, KO_ERR_SHAPE, "sgemm (no-alloc): dimension exceeds 2^31-1");
    KO_REQUIRE(D != nullptr && (K == 0 || (A != nullptr && B != nullptr)), KO_ERR_INVALID_ARG, "sgemm (no-alloc): NULL pointer");
    KO_REQUIRE(D != A && D != B, KO_ERR_INVALID_ARG, "sgemm (no-alloc): D must not alias A or B");
    ko::DeviceInfo info;
    if (int st = ko::current_device_info(&info)) return st;
    DeviceSetup *setup = nullptr;
    if (int st = setup_for_current_device(&setup)) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    const long long tiles = ((M + Wide::BM - 1) / Wide::BM) * ((N + Wide::BN - 1) / Wide::BN);
    const int ktiles = (int)((K + x2::BK - 1) / x2::BK);
    // how many K slices the fixed scratch can hold for this output size
    long long fits = tiles <= (long long)kMaxTiles ? (long long)(kMaxPartialFloats / ((size_t)tiles * Wide::kTileFloats)) : 0;
    if (fits < 1) fits = 1;  // one slice needs no scratch at all
    if (split_k == 0) {
        // same rule as ko_sgemm_f32 (fill the SMs, keep >= 8 K-tiles per slice), capped by the scratch
        split_k = 1;
        while (tiles * split_k * 2 <= (long long)info.sm_count * 2 && ktiles / (split_k * 2) >= 8 && split_k * 2 <= fits) split_k *= 2;
    }
    if (split_k > ktiles) split_k = ktiles > 0 ? ktiles : 1;
    KO_REQUIRE(split_k <= fits, KO_ERR_SHAPE,
               "sgemm (no-alloc): %lld output tiles in %d K-slices need %lld scratch floats (and %lld counters); the "
               "fixed scratch holds %zu floats and %zu counters -- use fewer slices (at most %lld here) or ko_sgemm_f32",
               tiles, split_k, tiles * split_k * (long long)Wide::kTileFloats, tiles, kMaxPartialFloats, kMaxTiles, fits);
    KO_REQUIRE(tiles * split_k <= 0x7fffffffLL, KO_ERR_SHAPE, "sgemm (no-alloc): too many blocks");

    // tiles * split_k blocks: every tile is cut into split_k K-slices, one scratch slot per slice
    x2::Params p{(int)M, (int)N, (int)K, A, B, C, D, (int)(tiles * split_k), split_k, 0, nullptr, nullptr};
    if (split_k > 1) {
        p.workspace = reinterpret_cast<float *>(setup->scratch);
        p.counters = reinterpret_cast<unsigned *>(setup->scratch + kCounterOffset);
        // the counters must start at zero whatever an earlier (possibly interrupted) call left behind
        KO_CUDA(cudaMemsetAsync(p.counters, 0, (size_t)tiles * sizeof(unsigned), s));
    }
    const bool vec_b = N % 4 == 0 && ko::aligned16(B);
    const unsigned grid = (unsigned)(tiles * split_k);
    if (vec_b) x2::sgemm_x2_kernel<true, 2, 2, 1><<<grid, Wide::kGroupThreads, Wide::smem_bytes(1), s>>>(p);
    else x2::sgemm_x2_kernel<false, 2, 2, 1><<<grid, Wide::kGroupThreads, Wide::smem_bytes(1), s>>>(p);
    KO_CHECK_LAUNCH("sgemm_x2_kernel (no-alloc)");
    return KO_OK;
}
