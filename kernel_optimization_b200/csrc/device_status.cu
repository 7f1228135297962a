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
    KO_CUDA(cudaMemcpyFromSymbol(words, g_status_words, sizeof words));  // synchronises with prior work
    for (int i = 0; i < ko::kStatusWordCount; ++i) {
        if (words[i] != 0) {
            const unsigned int zeros[ko::kStatusWordCount] = {};
            KO_CUDA(cudaMemcpyToSymbol(g_status_words, zeros, sizeof zeros));
            return ko::fail(KO_ERR_TIMEOUT, "%s: a bounded device-side wait ran out (code %u)", kWordNames[i], words[i]);
        }
    }
    return KO_OK;
}
