// CUDABackend, Tensor and top_k() over the C ABI (include/psx_b200.h).  Error behaviour follows
// the reference: contract violations throw std::invalid_argument (src/top_k.cpp:10-21), CUDA
// failures std::runtime_error with the PULSATRIX_CUDA_CHECK text.
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>
#include <utility>

#include "psx_b200.h"
#include "pulsatrix/device_backend.hpp"
#include "pulsatrix/top_k.hpp"

namespace pulsatrix {
namespace {

void check_cuda(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string("CUDA error: ") + cudaGetErrorString(e) + " in " + what);
}

void check_status(psx_status s) {
    if (s == PSX_OK) return;
    if (s == PSX_ERR_BAD_ARGUMENT) throw std::invalid_argument(psx_b200_last_error());
    throw std::runtime_error(psx_b200_last_error());
}

}  // namespace

CUDABackend::CUDABackend(int device_index) : device_index_(device_index) { check_status(psx_b200_ctx_create(device_index, &ctx_)); }

CUDABackend::~CUDABackend() { psx_b200_ctx_destroy(ctx_); }

void* CUDABackend::allocate(size_t bytes) {
    void* p = nullptr;
    check_cuda(cudaSetDevice(device_index_), "allocate");
    check_cuda(cudaMalloc(&p, bytes == 0 ? 1 : bytes), "allocate");
    return p;
}

void CUDABackend::free(void* ptr) noexcept {
    if (ptr) cudaFree(ptr);
}

void CUDABackend::copy(void* dst, const void* src, size_t bytes, CopyDirection dir) {
    if (bytes == 0) return;
    const cudaMemcpyKind kind = dir == CopyDirection::HostToDevice   ? cudaMemcpyHostToDevice
                                : dir == CopyDirection::DeviceToHost ? cudaMemcpyDeviceToHost
                                                                     : cudaMemcpyDeviceToDevice;
    cudaStream_t stream = static_cast<cudaStream_t>(psx_b200_ctx_stream(ctx_));
    check_cuda(cudaMemcpyAsync(dst, src, bytes, kind, stream), "copy");
    check_cuda(cudaStreamSynchronize(stream), "copy");
}

void CUDABackend::top_k_rows(const float* in, float* values, float* indices, size_t rows, size_t cols, size_t k,
                             bool largest) {
    if (rows == 0) return;
    void* stream = psx_b200_ctx_stream(ctx_);
    check_status(psx_b200_top_k_rows(ctx_, stream, in, values, indices, rows, cols, k, largest ? 1 : 0));
    check_status(psx_b200_sync(ctx_, stream));
}

void CUDABackend::softmax_rows(const float* in, float* out, size_t rows, size_t cols) {
    void* stream = psx_b200_ctx_stream(ctx_);
    check_status(psx_b200_softmax_rows(ctx_, stream, in, out, rows, cols));
    check_status(psx_b200_sync(ctx_, stream));
}

void CUDABackend::logsumexp_rows(const float* in, float* out, size_t rows, size_t cols) {
    void* stream = psx_b200_ctx_stream(ctx_);
    check_status(psx_b200_logsumexp_rows(ctx_, stream, in, out, rows, cols));
    check_status(psx_b200_sync(ctx_, stream));
}

void CUDABackend::gather_rows(const float* table, const float* indices, float* out, size_t count, size_t dim) {
    void* stream = psx_b200_ctx_stream(ctx_);
    check_status(psx_b200_gather_rows(ctx_, stream, table, indices, out, count, dim));
    check_status(psx_b200_sync(ctx_, stream));
}

Tensor::Tensor(Shape shape, DeviceBackend* backend) : shape_(std::move(shape)), backend_(backend) {
    data_ = static_cast<float*>(backend_->allocate(static_cast<size_t>(shape_.numel()) * sizeof(float)));
}

Tensor::Tensor(Shape shape, DeviceBackend* backend, const std::vector<float>& values) : Tensor(std::move(shape), backend) {
    if (static_cast<int64_t>(values.size()) != shape_.numel()) {
        throw std::invalid_argument("Tensor: " + std::to_string(values.size()) + " values for " +
                                    std::to_string(shape_.numel()) + " elements");
    }
    backend_->copy(data_, values.data(), values.size() * sizeof(float), CopyDirection::HostToDevice);
}

Tensor::~Tensor() {
    if (backend_ && data_) backend_->free(data_);
}

Tensor::Tensor(Tensor&& other) noexcept : shape_(std::move(other.shape_)), backend_(other.backend_), data_(other.data_) {
    other.data_ = nullptr;
}

Tensor& Tensor::operator=(Tensor&& other) noexcept {
    if (this != &other) {
        if (backend_ && data_) backend_->free(data_);
        shape_ = std::move(other.shape_);
        backend_ = other.backend_;
        data_ = other.data_;
        other.data_ = nullptr;
    }
    return *this;
}

std::vector<float> Tensor::to_host_vector() const {
    std::vector<float> host(static_cast<size_t>(numel()));
    backend_->copy(host.data(), data_, host.size() * sizeof(float), CopyDirection::DeviceToHost);
    return host;
}

TopKResult top_k(const Tensor& input, int64_t k, bool largest) {
    if (input.rank() < 1 || input.numel() <= 0) {
        throw std::invalid_argument("top_k: input must be non-empty with rank >= 1");
    }
    const int64_t cols = input.shape().dim(input.rank() - 1);
    if (k < 1 || k > cols) {
        throw std::invalid_argument("top_k: k must be in [1, " + std::to_string(cols) + "], got " + std::to_string(k));
    }
    if (cols > (int64_t{1} << 24)) {
        throw std::invalid_argument("top_k: last dimension exceeds 2^24, beyond exact float indices");
    }
    std::vector<int64_t> out_dims;
    for (int64_t d = 0; d + 1 < input.rank(); ++d) out_dims.push_back(input.shape().dim(d));
    out_dims.push_back(k);
    TopKResult result{Tensor(Shape(out_dims), input.backend()), Tensor(Shape(out_dims), input.backend())};
    input.backend()->top_k_rows(input.data(), result.values.data(), result.indices.data(),
                                static_cast<size_t>(input.numel() / cols), static_cast<size_t>(cols),
                                static_cast<size_t>(k), largest);
    return result;
}

}  // namespace pulsatrix
