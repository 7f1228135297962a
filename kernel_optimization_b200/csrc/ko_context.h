// ko::Context: the owner of everything the operator launchers keep between calls -- the SGEMM's
// split-K scratch (one lane per stream) and the cache of encoded TMA descriptors of the tensor-core
// GEMM.  A context belongs to one device.  Callers either create one (ko_context_create /
// ko_context_destroy, which frees what it owns) and pass it to the *_ctx entry points, or use the plain
// entry points, which work on the device's default context (created on first use, kept until exit).
#pragma once

#include "ko_internal.h"

#include <cuda.h>

#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace ko {

struct SgemmScratch {
    float *partials = nullptr;
    size_t partial_floats = 0;
    unsigned *counters = nullptr;
    size_t counter_count = 0;
};

// what identifies an encoded 2-D tensor map
struct TensorMapKey {
    const void *base;
    uint64_t dim0, dim1;     // innermost extent, outer extent (elements)
    uint32_t box0, box1;     // box extents (elements)
    uint32_t kind;           // data type, swizzle and L2-promotion choice packed by the caller
    bool operator==(const TensorMapKey &o) const {
        return base == o.base && dim0 == o.dim0 && dim1 == o.dim1 && box0 == o.box0 && box1 == o.box1 && kind == o.kind;
    }
};
struct TensorMapKeyHash {
    size_t operator()(const TensorMapKey &k) const {
        uint64_t h = reinterpret_cast<uintptr_t>(k.base) * 0x9e3779b97f4a7c15ull;
        h ^= (k.dim0 + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2));
        h ^= (k.dim1 + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2));
        h ^= (((uint64_t)k.box0 << 40) ^ ((uint64_t)k.box1 << 20) ^ k.kind) + (h << 6) + (h >> 2);
        return (size_t)h;
    }
};

class Context {
public:
    explicit Context(int device) : device_(device) {}
    ~Context();  // frees every block; the caller guarantees that no kernel using them is in flight
    Context(const Context &) = delete;
    Context &operator=(const Context &) = delete;

    int device() const { return device_; }

    // Scratch of at least the requested size for launches on stream `s`.  A lane is allocated the first time a
    // stream needs one (at least `floor_floats` / `floor_counters`, the most the shape heuristics can ask for, so
    // that later default calls never allocate) and never shrinks.  When a later request is larger, a new block is
    // allocated and the old one is kept until the context dies: pointers handed out earlier (to launches in
    // flight, to captured graphs) stay valid.  While `s` is being captured nothing can be allocated: a request
    // that does not fit the existing lane fails with KO_ERR_INVALID_ARG.
    int sgemm_scratch(cudaStream_t s, size_t partial_floats, size_t counter_count, size_t floor_floats, size_t floor_counters,
                      SgemmScratch *out);

    // Cached cuTensorMapEncodeTiled: `encode` is called only for a key not seen before.
    template <typename Encode>
    int tensor_map(const TensorMapKey &key, CUtensorMap *out, Encode &&encode) {
        {
            std::lock_guard<std::mutex> lock(mu_);
            auto it = maps_.find(key);
            if (it != maps_.end()) {
                *out = it->second;
                ++map_hits_;
                return KO_OK;
            }
        }
        alignas(64) CUtensorMap fresh;
        if (int st = encode(&fresh)) return st;
        std::lock_guard<std::mutex> lock(mu_);
        if (maps_.size() >= kMaxMaps) maps_.clear();  // a caller cycling through thousands of buffers: start over
        maps_.emplace(key, fresh);
        ++map_misses_;
        *out = fresh;
        return KO_OK;
    }

    // bytes of device memory this context holds, cached tensor maps, and how often the cache answered
    void stats(size_t *device_bytes, size_t *maps, size_t *hits, size_t *misses);

private:
    static constexpr size_t kMaxMaps = 4096;
    int device_;
    std::mutex mu_;
    std::map<cudaStream_t, SgemmScratch> lanes_;
    std::vector<void *> blocks_;  // every allocation ever made, freed by the destructor
    size_t device_bytes_ = 0;
    std::unordered_map<TensorMapKey, CUtensorMap, TensorMapKeyHash> maps_;
    size_t map_hits_ = 0, map_misses_ = 0;
};

// The context a call runs on: `handle` when given (its device must be the current one), else the current
// device's default context.
int resolve_context(ko_context_t *handle, Context **out);

}  // namespace ko
