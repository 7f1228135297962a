// Device status words: kernels with bounded waits (mbarrier / tcgen05 pipelines) record here when a
// wait runs out instead of spinning forever.  The host reads and clears them with
// ko_poll_device_status().  The words are file-scope __device__ storage, so nothing is allocated.
#include "ko_internal.h"

namespace {
__device__ unsigned int g_status_words[ko::kStatusWordCount];
const char *const kWordNames[ko::kStatusWordCount] = {"tensor-core GEMM", "staged row operator", "reserved", "reserved"};
}  // namespace

namespace ko {
int device_status_word(int which, unsigned int **out) {
    KO_REQUIRE(which >= 0 && which < kStatusWordCount, KO_ERR_INVALID_ARG, "status word %d out of range", which);
    void *base = nullptr;
    KO_CUDA(cudaGetSymbolAddress(&base, g_status_words));
    *out = static_cast<unsigned int *>(base) + which;
    return KO_OK;
}
}  // namespace ko

extern "C" int ko_poll_device_status(void) {
    unsigned int words[ko::kStatusWordCount] = {};
    // every stream of the device, non-blocking ones included (a copy on the legacy default stream alone would
    // not wait for those), has drained before the words are read: nothing can write between the read and the clear
    KO_CUDA(cudaDeviceSynchronize());
    KO_CUDA(cudaMemcpyFromSymbol(words, g_status_words, sizeof words));
    for (int i = 0; i < ko::kStatusWordCount; ++i) {
        if (words[i] != 0) {
            const unsigned int zeros[ko::kStatusWordCount] = {};
            KO_CUDA(cudaMemcpyToSymbol(g_status_words, zeros, sizeof zeros));
            return ko::fail(KO_ERR_TIMEOUT, "%s: a bounded device-side wait ran out (code %u)", kWordNames[i], words[i]);
        }
    }
    return KO_OK;
}

// ---------------------------------------------------------------------------------------------
// Self-test of the failure-detection path: a kernel waits, with a short bound, on an mbarrier that
// nothing ever arrives at; the wait runs out, the kernel records a code in the "reserved" status word
// and returns normally.  The host then sees KO_ERR_TIMEOUT from ko_poll_device_status().  Nothing
// faults, traps or hangs: this is how a stuck pipeline would surface in production.
// ---------------------------------------------------------------------------------------------
#include "../common/common.h"

namespace {
__global__ void bounded_wait_selftest_kernel(unsigned *status, unsigned polls) {
    __shared__ unsigned long long bar;
    const unsigned addr = ko::smem_u32(&bar);
    if (threadIdx.x == 0) {
        ko::mbar_init(addr, 1);
        ko::fence_barrier_init();
        bool arrived = false;
        for (unsigned spin = 0; spin < polls && !arrived; ++spin) arrived = ko::mbar_try_wait(addr, 0);
        if (!arrived) atomicCAS(status, 0u, 0x7e57u);
    }
}
}  // namespace

extern "C" int ko_selftest_bounded_wait(unsigned polls, void *stream) {
    unsigned *status = nullptr;
    if (int st = ko::device_status_word(2, &status)) return st;
    KO_REQUIRE(polls > 0 && polls <= (1u << 20), KO_ERR_INVALID_ARG, "selftest: polls must be in [1, 2^20]");
    bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, polls);
    KO_CHECK_LAUNCH("bounded_wait_selftest_kernel");
    return KO_OK;
}
