// Row operators over HOST tensors with the copies overlapped: the rows are cut into chunks and three
// streams form a pipeline -- host-to-device copy of chunk c+1, kernel on chunk c and device-to-host
// copy of chunk c-1 run at the same time, so a step costs about one direction of the PCIe link instead
// of both plus the kernel.
//
// The reference's drivers copy whole tensors synchronously before and after the launch
// (nn_operators/softmax/main.cu:38, :55, :62; nn_operators/layernorm/main.cu:37, :54, :61); this is the
// same data path for a caller whose data lives on the host, with nothing serialized that the hardware
// can overlap.  It has no counterpart in the reference.
//
// Ordering contract: the whole call is ordered after earlier work on `stream`, and later work on
// `stream` is ordered after the last copy of the call -- a caller sees plain stream semantics although
// two more streams (owned by the library, one pair per device) do the copies.
#include "ko_internal.h"

#include <mutex>

namespace {

constexpr int kMaxChunks = 64;
constexpr int kMaxDevices = 64;

struct Lanes {
    bool ready = false;
    cudaStream_t copy_in = nullptr, copy_out = nullptr;
    cudaEvent_t start = nullptr, done = nullptr;
    cudaEvent_t landed[kMaxChunks] = {}, computed[kMaxChunks] = {};
};
Lanes g_lanes[kMaxDevices];
std::mutex g_mutex;  // one pipelined call is issued at a time: the events are shared

int lanes_for(int device, Lanes **out) {
    KO_REQUIRE(device >= 0 && device < kMaxDevices, KO_ERR_INVALID_ARG, "host pipeline: device %d out of range", device);
    Lanes &l = g_lanes[device];
    if (!l.ready) {
        KO_CUDA(cudaStreamCreateWithFlags(&l.copy_in, cudaStreamNonBlocking));
        KO_CUDA(cudaStreamCreateWithFlags(&l.copy_out, cudaStreamNonBlocking));
        KO_CUDA(cudaEventCreateWithFlags(&l.start, cudaEventDisableTiming));
        KO_CUDA(cudaEventCreateWithFlags(&l.done, cudaEventDisableTiming));
        for (int c = 0; c < kMaxChunks; ++c) {
            KO_CUDA(cudaEventCreateWithFlags(&l.landed[c], cudaEventDisableTiming));
            KO_CUDA(cudaEventCreateWithFlags(&l.computed[c], cudaEventDisableTiming));
        }
        l.ready = true;
    }
    *out = &l;
    return KO_OK;
}

// elem_bytes: 4 (FP32) -- the operators called per chunk
template <typename Launch>
int run_pipeline(ko_tensor_t *in, ko_tensor_t *out, int64_t rows, int32_t cols, size_t elem_bytes, int chunks, cudaStream_t stream,
                 Launch &&launch) {
    KO_REQUIRE(in != nullptr && out != nullptr, KO_ERR_INVALID_ARG, "host pipeline: NULL tensor");
    KO_REQUIRE(rows >= 0 && cols >= 0, KO_ERR_INVALID_ARG, "host pipeline: negative shape [%lld, %d]", (long long)rows, cols);
    const size_t bytes = (size_t)rows * (size_t)cols * elem_bytes;
    KO_REQUIRE(ko_tensor_size_in_bytes(in) >= bytes && ko_tensor_size_in_bytes(out) >= bytes, KO_ERR_SHAPE,
               "host pipeline: [%lld, %d] x %zu bytes exceeds a tensor (%zu / %zu bytes)", (long long)rows, cols, elem_bytes,
               ko_tensor_size_in_bytes(in), ko_tensor_size_in_bytes(out));
    KO_REQUIRE(ko_tensor_device(in) == ko_tensor_device(out), KO_ERR_INVALID_ARG, "host pipeline: tensors live on devices %d and %d",
               ko_tensor_device(in), ko_tensor_device(out));
    int device = -1;
    KO_CUDA(cudaGetDevice(&device));
    KO_REQUIRE(device == ko_tensor_device(in), KO_ERR_INVALID_ARG, "host pipeline: current device %d, tensors on %d", device,
               ko_tensor_device(in));
    if (bytes == 0) return KO_OK;
    if (chunks <= 0) chunks = 8;
    if (chunks > kMaxChunks - 4) chunks = kMaxChunks - 4;
    if (chunks > rows) chunks = (int)rows;
    // Row ranges.  The first chunk's copy in and the last chunk's copy out overlap with nothing (the other direction of
    // the link is idle meanwhile), so the ends of the sequence are cut finer: with n >= 4 nominal chunks the pieces weigh
    // 1/4, 1/4, 1/2, 1 x (n - 2), 1/2, 1/4, 1/4 of a nominal chunk (n + 4 pieces), which shrinks both idle stretches
    // four-fold for a handful of extra copies.
    int64_t bounds[kMaxChunks + 1];
    int pieces = 0;
    if (chunks >= 4 && rows >= 64LL * chunks) {
        const int quarter_units[3] = {1, 1, 2};  // in quarters of a nominal chunk
        int64_t done_q = 0;
        const int64_t total_q = 4LL * chunks;
        bounds[0] = 0;
        auto push = [&](int q) {
            done_q += q;
            bounds[++pieces] = rows * done_q / total_q;
        };
        for (int q : quarter_units) push(q);
        for (int c = 0; c < chunks - 2; ++c) push(4);
        for (int i = 2; i >= 0; --i) push(quarter_units[i]);
    } else {
        for (int c = 0; c <= chunks; ++c) bounds[c] = rows * c / chunks;
        pieces = chunks;
    }
    chunks = pieces;

    std::lock_guard<std::mutex> lock(g_mutex);
    Lanes *l = nullptr;
    if (int st = lanes_for(device, &l)) return st;
    char *h_in = static_cast<char *>(ko_tensor_host_ptr(in)), *d_in = static_cast<char *>(ko_tensor_device_ptr(in));
    char *h_out = static_cast<char *>(ko_tensor_host_ptr(out)), *d_out = static_cast<char *>(ko_tensor_device_ptr(out));
    const size_t row_bytes = (size_t)cols * elem_bytes;

    // the copies may not overtake work already queued on the caller's stream (it may still read d_in / write d_out)
    KO_CUDA(cudaEventRecord(l->start, stream));
    KO_CUDA(cudaStreamWaitEvent(l->copy_in, l->start, 0));
    KO_CUDA(cudaStreamWaitEvent(l->copy_out, l->start, 0));
    // one chunk: copy in, wait, launch, copy out; the first failing step ends the call
    auto enqueue_chunk = [&](int c) -> int {
        const int64_t r0 = bounds[c], r1 = bounds[c + 1];
        if (r1 == r0) return KO_OK;
        const size_t off = (size_t)r0 * row_bytes, len = (size_t)(r1 - r0) * row_bytes;
        KO_CUDA(cudaMemcpyAsync(d_in + off, h_in + off, len, cudaMemcpyHostToDevice, l->copy_in));
        KO_CUDA(cudaEventRecord(l->landed[c], l->copy_in));
        KO_CUDA(cudaStreamWaitEvent(stream, l->landed[c], 0));
        if (int st = launch(d_in + off, d_out + off, r1 - r0)) return st;
        KO_CUDA(cudaEventRecord(l->computed[c], stream));
        KO_CUDA(cudaStreamWaitEvent(l->copy_out, l->computed[c], 0));
        KO_CUDA(cudaMemcpyAsync(h_out + off, d_out + off, len, cudaMemcpyDeviceToHost, l->copy_out));
        return KO_OK;
    };
    int status = KO_OK;
    for (int c = 0; c < chunks && status == KO_OK; ++c) status = enqueue_chunk(c);
    // Success or not, the caller's stream continues only after everything that was enqueued on the two copy
    // streams: a call that failed half way leaves no copy running behind the caller's back.
    const cudaError_t join_in = cudaEventRecord(l->start, l->copy_in);
    const cudaError_t wait_in = join_in == cudaSuccess ? cudaStreamWaitEvent(stream, l->start, 0) : join_in;
    const cudaError_t join_out = cudaEventRecord(l->done, l->copy_out);
    const cudaError_t wait_out = join_out == cudaSuccess ? cudaStreamWaitEvent(stream, l->done, 0) : join_out;
    if (status != KO_OK) return status;
    if (wait_in != cudaSuccess) return ko::fail_cuda(wait_in, "host pipeline: joining the copy-in stream");
    if (wait_out != cudaSuccess) return ko::fail_cuda(wait_out, "host pipeline: joining the copy-out stream");
    return KO_OK;
}

}  // namespace

extern "C" {

int ko_softmax_f32_host(ko_tensor_t *in, ko_tensor_t *out, int64_t rows, int32_t cols, int chunks, void *stream) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return run_pipeline(in, out, rows, cols, sizeof(float), chunks, s, [&](char *src, char *dst, int64_t n) {
        return ko_softmax_f32(reinterpret_cast<const float *>(src), reinterpret_cast<float *>(dst), n, cols, stream);
    });
}

int ko_layernorm_f32_host(ko_tensor_t *in, ko_tensor_t *out, int64_t rows, int32_t cols, float eps, const float *gamma,
                          const float *beta, int ddof, int chunks, void *stream) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return run_pipeline(in, out, rows, cols, sizeof(float), chunks, s, [&](char *src, char *dst, int64_t n) {
        return ko_layernorm_f32(reinterpret_cast<const float *>(src), reinterpret_cast<float *>(dst), n, cols, eps, gamma, beta, ddof,
                                stream);
    });
}

}  // extern "C"
