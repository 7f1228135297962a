// placeholder until the tcgen05 kernel lands
#include "ko_internal.h"
extern "C" {
int ko_gemm_f16_f32(int64_t, int64_t, int64_t, const uint16_t *, const uint16_t *, const float *, float *, void *) {
    return ko::fail(KO_ERR_SHAPE, "tensor-core GEMM is not built into this library yet");
}
int ko_gemm_bf16_f32(int64_t, int64_t, int64_t, const uint16_t *, const uint16_t *, const float *, float *, void *) {
    return ko::fail(KO_ERR_SHAPE, "tensor-core GEMM is not built into this library yet");
}
}
