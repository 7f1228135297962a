// Tensor implementation and its C handles (ko_tensor_*).  See tensor.h for how it differs from
// the reference's common/tensor.cu:8-42.
#include "tensor.h"

#include <new>
#include <utility>

#include "../csrc/ko_internal.h"
#include "common.h"

namespace {
// RAII switch to the tensor's device for calls that need it current
struct DeviceGuard {
    int previous = -1;
    bool switched = false;
    explicit DeviceGuard(int device) {
        if (device >= 0 && cudaGetDevice(&previous) == cudaSuccess && previous != device)
            switched = cudaSetDevice(device) == cudaSuccess;
    }
    ~DeviceGuard() {
        if (switched) cudaSetDevice(previous);
    }
};
}  // namespace

Tensor::Tensor(size_t size_in_bytes, int device) : size_in_bytes_(size_in_bytes), device_(device) {
    if (device_ < 0) checkCudaErrors(cudaGetDevice(&device_));
    DeviceGuard guard(device_);
    const size_t bytes = size_in_bytes_ ? size_in_bytes_ : 1;
    checkCudaErrors(cudaMallocHost(&host_ptr_, bytes));
    checkCudaErrors(cudaMalloc(&device_ptr_, bytes));
}

Tensor::Tensor(Tensor &&rhs) noexcept { *this = std::move(rhs); }

Tensor &Tensor::operator=(Tensor &&rhs) noexcept {
    if (this != &rhs) {
        release();
        host_ptr_ = std::exchange(rhs.host_ptr_, nullptr);
        device_ptr_ = std::exchange(rhs.device_ptr_, nullptr);
        size_in_bytes_ = std::exchange(rhs.size_in_bytes_, 0);
        device_ = rhs.device_;
    }
    return *this;
}

void Tensor::release() {
    if (!host_ptr_ && !device_ptr_) return;
    DeviceGuard guard(device_);
    if (host_ptr_) cudaFreeHost(host_ptr_);
    if (device_ptr_) cudaFree(device_ptr_);
    host_ptr_ = device_ptr_ = nullptr;
}

Tensor::~Tensor() { release(); }

void Tensor::host_to_device() {
    DeviceGuard guard(device_);
    checkCudaErrors(cudaMemcpy(device_ptr_, host_ptr_, size_in_bytes_, cudaMemcpyHostToDevice));
}
void Tensor::host_to_device_async(cudaStream_t &stream) {
    checkCudaErrors(cudaMemcpyAsync(device_ptr_, host_ptr_, size_in_bytes_, cudaMemcpyHostToDevice, stream));
}
void Tensor::device_to_host() {
    DeviceGuard guard(device_);
    checkCudaErrors(cudaMemcpy(host_ptr_, device_ptr_, size_in_bytes_, cudaMemcpyDeviceToHost));
}
void Tensor::device_to_host_async(cudaStream_t &stream) {
    checkCudaErrors(cudaMemcpyAsync(host_ptr_, device_ptr_, size_in_bytes_, cudaMemcpyDeviceToHost, stream));
}

static size_t dtype_size(int dtype) { return dtype == KO_DTYPE_F32 ? 4 : 2; }

void Tensor::fill_uniform(int dtype, uint32_t seed, uint32_t tensor_id, float lo, float hi, int64_t elem_offset) {
    ko_fill_uniform(host_ptr_, dtype, (int64_t)(size_in_bytes_ / dtype_size(dtype)), seed, tensor_id, elem_offset, lo, hi);
}
void Tensor::fill_normal(int dtype, uint32_t seed, uint32_t tensor_id, float mean, float stddev, int64_t elem_offset) {
    ko_fill_normal(host_ptr_, dtype, (int64_t)(size_in_bytes_ / dtype_size(dtype)), seed, tensor_id, elem_offset, mean, stddev);
}
double Tensor::max_abs_diff_f32(const float *expected) const {
    double worst = 0.0;
    ko_check_max_abs_f32(static_cast<const float *>(host_ptr_), expected, (int64_t)(size_in_bytes_ / 4), &worst);
    return worst;
}

// ---------------------------------------------------------------------------------------------
// C handles: unlike the class (whose constructor exits on failure, as the reference's does), these
// report failures as status codes.
// ---------------------------------------------------------------------------------------------
struct ko_tensor {
    void *host = nullptr;
    void *dev = nullptr;
    size_t bytes = 0;
    int device = -1;
};

extern "C" {

int ko_tensor_create(size_t size_in_bytes, int device, ko_tensor_t **out) {
    KO_REQUIRE(out != nullptr, KO_ERR_INVALID_ARG, "ko_tensor_create: out is NULL");
    *out = nullptr;
    if (device < 0) KO_CUDA(cudaGetDevice(&device));
    DeviceGuard guard(device);
    ko_tensor *t = new (std::nothrow) ko_tensor;
    KO_REQUIRE(t != nullptr, KO_ERR_INVALID_ARG, "ko_tensor_create: out of host memory");
    t->bytes = size_in_bytes;
    t->device = device;
    const size_t bytes = size_in_bytes ? size_in_bytes : 1;
    cudaError_t e = cudaMallocHost(&t->host, bytes);
    if (e == cudaSuccess) e = cudaMalloc(&t->dev, bytes);
    if (e != cudaSuccess) {
        if (t->host) cudaFreeHost(t->host);
        delete t;
        return ko::fail_cuda(e, "ko_tensor_create allocation");
    }
    *out = t;
    return KO_OK;
}

int ko_tensor_destroy(ko_tensor_t *t) {
    if (!t) return KO_OK;
    DeviceGuard guard(t->device);
    cudaError_t e1 = t->host ? cudaFreeHost(t->host) : cudaSuccess;
    cudaError_t e2 = t->dev ? cudaFree(t->dev) : cudaSuccess;
    delete t;
    if (e1 != cudaSuccess) return ko::fail_cuda(e1, "cudaFreeHost");
    if (e2 != cudaSuccess) return ko::fail_cuda(e2, "cudaFree");
    return KO_OK;
}

void *ko_tensor_host_ptr(ko_tensor_t *t) { return t ? t->host : nullptr; }
void *ko_tensor_device_ptr(ko_tensor_t *t) { return t ? t->dev : nullptr; }
size_t ko_tensor_size_in_bytes(const ko_tensor_t *t) { return t ? t->bytes : 0; }
int ko_tensor_device(const ko_tensor_t *t) { return t ? t->device : -1; }

int ko_tensor_host_to_device(ko_tensor_t *t) {
    KO_REQUIRE(t != nullptr, KO_ERR_INVALID_ARG, "ko_tensor_host_to_device: NULL tensor");
    DeviceGuard guard(t->device);
    KO_CUDA(cudaMemcpy(t->dev, t->host, t->bytes, cudaMemcpyHostToDevice));
    return KO_OK;
}
int ko_tensor_host_to_device_async(ko_tensor_t *t, void *stream) {
    KO_REQUIRE(t != nullptr, KO_ERR_INVALID_ARG, "ko_tensor_host_to_device_async: NULL tensor");
    KO_CUDA(cudaMemcpyAsync(t->dev, t->host, t->bytes, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)));
    return KO_OK;
}
int ko_tensor_device_to_host(ko_tensor_t *t) {
    KO_REQUIRE(t != nullptr, KO_ERR_INVALID_ARG, "ko_tensor_device_to_host: NULL tensor");
    DeviceGuard guard(t->device);
    KO_CUDA(cudaMemcpy(t->host, t->dev, t->bytes, cudaMemcpyDeviceToHost));
    return KO_OK;
}
int ko_tensor_device_to_host_async(ko_tensor_t *t, void *stream) {
    KO_REQUIRE(t != nullptr, KO_ERR_INVALID_ARG, "ko_tensor_device_to_host_async: NULL tensor");
    KO_CUDA(cudaMemcpyAsync(t->host, t->dev, t->bytes, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
    return KO_OK;
}

}  // extern "C"
