// ko::Context and the ko_context_* entry points (see ko_context.h).
#include "ko_context.h"

#include <memory>

struct ko_context {
    ko::Context impl;
    explicit ko_context(int device) : impl(device) {}
};

namespace ko {

Context::~Context() {
    for (void *p : blocks_) cudaFree(p);
}

int Context::sgemm_scratch(cudaStream_t s, size_t partial_floats, size_t counter_count, size_t floor_floats,
                           size_t floor_counters, SgemmScratch *out) {
    std::lock_guard<std::mutex> lock(mu_);
    SgemmScratch &lane = lanes_[s];
    const bool grow_partials = lane.partial_floats < partial_floats, grow_counters = lane.counter_count < counter_count;
    if (grow_partials || grow_counters) {
        cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
        KO_CUDA(cudaStreamIsCapturing(s, &capturing));
        KO_REQUIRE(capturing == cudaStreamCaptureStatusNone, KO_ERR_INVALID_ARG,
                   "sgemm: this stream's scratch lane (%zu floats, %zu counters) is too small for the request (%zu, %zu) and "
                   "cannot grow during stream capture: run the call once eagerly on this stream first",
                   lane.partial_floats, lane.counter_count, partial_floats, counter_count);
    }
    if (grow_partials) {
        const size_t want = partial_floats > floor_floats ? partial_floats : floor_floats;
        float *fresh = nullptr;
        KO_CUDA(cudaMalloc(&fresh, want * sizeof(float)));
        blocks_.push_back(fresh);  // the previous block, if any, stays alive in blocks_
        device_bytes_ += want * sizeof(float);
        lane.partials = fresh;
        lane.partial_floats = want;
    }
    if (grow_counters) {
        const size_t want = counter_count > floor_counters ? counter_count : floor_counters;
        unsigned *fresh = nullptr;
        KO_CUDA(cudaMalloc(&fresh, want * sizeof(unsigned)));
        blocks_.push_back(fresh);
        device_bytes_ += want * sizeof(unsigned);
        // counters are zero whenever no launch is in flight (the last block of a tile resets its counter)
        KO_CUDA(cudaMemset(fresh, 0, want * sizeof(unsigned)));
        lane.counters = fresh;
        lane.counter_count = want;
    }
    *out = lane;
    return KO_OK;
}

void Context::stats(size_t *device_bytes, size_t *maps, size_t *hits, size_t *misses) {
    std::lock_guard<std::mutex> lock(mu_);
    if (device_bytes) *device_bytes = device_bytes_;
    if (maps) *maps = maps_.size();
    if (hits) *hits = map_hits_;
    if (misses) *misses = map_misses_;
}

int resolve_context(ko_context_t *handle, Context **out) {
    int dev = -1;
    KO_CUDA(cudaGetDevice(&dev));
    if (handle != nullptr) {
        KO_REQUIRE(handle->impl.device() == dev, KO_ERR_INVALID_ARG, "context belongs to device %d, the current device is %d",
                   handle->impl.device(), dev);
        *out = &handle->impl;
        return KO_OK;
    }
    constexpr int kMaxDevices = 64;
    KO_REQUIRE(dev >= 0 && dev < kMaxDevices, KO_ERR_NO_DEVICE, "device ordinal %d out of range", dev);
    static std::mutex mu;
    static Context *defaults[kMaxDevices] = {};  // never destroyed: the driver reclaims the memory at exit
    std::lock_guard<std::mutex> lock(mu);
    if (defaults[dev] == nullptr) defaults[dev] = new Context(dev);
    *out = defaults[dev];
    return KO_OK;
}

}  // namespace ko

extern "C" {

int ko_context_create(int device, ko_context_t **out) {
    KO_REQUIRE(out != nullptr, KO_ERR_INVALID_ARG, "ko_context_create: NULL out");
    *out = nullptr;
    int count = 0;
    KO_CUDA(cudaGetDeviceCount(&count));
    if (device < 0) KO_CUDA(cudaGetDevice(&device));
    KO_REQUIRE(device < count, KO_ERR_INVALID_ARG, "ko_context_create: device %d of %d", device, count);
    *out = new ko_context(device);
    return KO_OK;
}

int ko_context_destroy(ko_context_t *ctx) {
    if (ctx == nullptr) return KO_OK;
    int prev = -1;
    KO_CUDA(cudaGetDevice(&prev));
    KO_CUDA(cudaSetDevice(ctx->impl.device()));
    const cudaError_t err = cudaDeviceSynchronize();  // nothing may still be using the scratch
    delete ctx;
    cudaSetDevice(prev);
    if (err != cudaSuccess) return ko::fail_cuda(err, "cudaDeviceSynchronize (ko_context_destroy)");
    return KO_OK;
}

int ko_context_stats(ko_context_t *ctx, size_t *device_bytes, size_t *tensor_maps, size_t *map_hits, size_t *map_misses) {
    ko::Context *c = nullptr;
    if (ctx != nullptr) c = &ctx->impl;
    else if (int st = ko::resolve_context(nullptr, &c)) return st;
    c->stats(device_bytes, tensor_maps, map_hits, map_misses);
    return KO_OK;
}

}  // extern "C"
