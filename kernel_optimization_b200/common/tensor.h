// Tensor: a host buffer and a device buffer of the same size, with copies in both directions.
//
// Same public surface as the reference's class Tensor (common/tensor.h:11-40):
// Tensor(bytes), Tensor(shape, bytes_per_element), host_ref<T>(), device_ref<T>(),
// host_to_device[_async], device_to_host[_async], move-assignment, non-copyable.
//
// Differences, all deliberate:
//   * the host side is page-locked (cudaMallocHost), so the async copies really are asynchronous
//     and reach PCIe/C2C line rate (the reference uses pageable new[]);
//   * the tensor remembers its device ordinal and size (device(), size_in_bytes());
//   * the shape product is taken in size_t (the reference folds it in int, tensor.h:15);
//   * move-assignment releases what the destination held and carries the size over (the reference
//     leaks both buffers and drops the size, tensor.cu:13-21); a move constructor exists;
//   * seeded fills and a host-side comparison are members (the reference fills inline in its
//     drivers and has no check); they call the same routines as the C ABI.
#pragma once

#include <cstddef>
#include <cstdint>
#include <functional>
#include <numeric>
#include <vector>

#include <cuda_runtime.h>

class Tensor {
public:
    explicit Tensor(size_t size_in_bytes, int device = -1);
    Tensor(const std::vector<size_t> &shape, size_t byte_per_element, int device = -1)
        : Tensor(byte_per_element * std::accumulate(shape.begin(), shape.end(), size_t(1), std::multiplies<size_t>()),
                 device) {}
    Tensor(Tensor &&rhs) noexcept;
    Tensor &operator=(Tensor &&rhs) noexcept;
    Tensor(const Tensor &) = delete;
    Tensor &operator=(const Tensor &) = delete;
    ~Tensor();

    template <typename T>
    T *host_ref() { return static_cast<T *>(host_ptr_); }
    template <typename T>
    T *device_ref() { return static_cast<T *>(device_ptr_); }

    void host_to_device();
    void host_to_device_async(cudaStream_t &stream);
    void device_to_host();
    void device_to_host_async(cudaStream_t &stream);

    size_t size_in_bytes() const { return size_in_bytes_; }
    int device() const { return device_; }

    // seeded host fills (dtype: KO_DTYPE_F32 / KO_DTYPE_F16 / KO_DTYPE_BF16); the whole buffer is filled
    void fill_uniform(int dtype, uint32_t seed, uint32_t tensor_id, float lo, float hi, int64_t elem_offset = 0);
    void fill_normal(int dtype, uint32_t seed, uint32_t tensor_id, float mean, float stddev, int64_t elem_offset = 0);

    // max |host[i] - expected[i]| over the buffer viewed as FP32
    double max_abs_diff_f32(const float *expected) const;

private:
    void release();
    void *host_ptr_ = nullptr;
    void *device_ptr_ = nullptr;
    size_t size_in_bytes_ = 0;
    int device_ = -1;
};
