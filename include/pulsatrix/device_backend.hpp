/** @file device_backend.hpp
 *  The part of the reference's DeviceBackend interface (include/pulsatrix/device_backend.hpp:248-838)
 *  that the selection path and its neighbours touch: memory, copies, top_k_rows (:828-837),
 *  softmax_rows (:456), logsumexp_rows (:465) and gather_rows (:596), plus the minimal Shape/Tensor
 *  that top_k() takes.  Same names and argument meaning; everything else of the reference's ~100
 *  virtuals belongs to the model side and is not rebuilt here, so this class is not
 *  layout-compatible with the reference's: a program written against these headers links against
 *  this library, one compiled against the reference's header does not.
 */
#pragma once

#include <cstddef>
#include <cstdint>
#include <initializer_list>
#include <vector>

#include "pulsatrix/export.hpp"

struct psx_ctx;

namespace pulsatrix {

enum class DeviceType { Cpu, Cuda };
enum class CopyDirection { HostToDevice, DeviceToHost, DeviceToDevice };

class PULSATRIX_API DeviceBackend {
public:
    virtual ~DeviceBackend() = default;
    [[nodiscard]] virtual DeviceType device() const noexcept = 0;
    /** Never null for a non-zero size; throws std::runtime_error on failure. */
    [[nodiscard]] virtual void* allocate(size_t bytes) = 0;
    virtual void free(void* ptr) noexcept = 0;
    virtual void copy(void* dst, const void* src, size_t bytes, CopyDirection dir) = 0;
    /** Per row of a row-major (rows, cols) matrix: the k largest (or smallest) values in rank order
     *  and their columns as whole-number floats.  NaN ranks above every number; equal values keep
     *  the lower column first.  Preconditions (checked by top_k()): 1 <= k <= cols <= 2^24. */
    virtual void top_k_rows(const float* in, float* values, float* indices, size_t rows, size_t cols, size_t k,
                            bool largest) = 0;
    /** Row-wise softmax of a (rows x cols) matrix, max-subtracted. out may alias in. */
    virtual void softmax_rows(const float* in, float* out, size_t rows, size_t cols) = 0;
    /** Per-row log-sum-exp, max-subtracted: out[i] = log sum_j exp(in[i][j]). */
    virtual void logsumexp_rows(const float* in, float* out, size_t rows, size_t cols) = 0;
    /** out[i][:] = table[indices[i]][:] for count rows of width dim. */
    virtual void gather_rows(const float* table, const float* indices, float* out, size_t count, size_t dim) = 0;
};

/** The B200 backend: owns a psx_ctx (stream + scratch); every call synchronises before returning,
 *  like the reference's CUDABackend (include/pulsatrix/cuda_backend.hpp:20-22). */
class PULSATRIX_API CUDABackend : public DeviceBackend {
public:
    explicit CUDABackend(int device_index = 0);
    ~CUDABackend() override;
    CUDABackend(const CUDABackend&) = delete;
    CUDABackend& operator=(const CUDABackend&) = delete;
    [[nodiscard]] DeviceType device() const noexcept override { return DeviceType::Cuda; }
    [[nodiscard]] void* allocate(size_t bytes) override;
    void free(void* ptr) noexcept override;
    void copy(void* dst, const void* src, size_t bytes, CopyDirection dir) override;
    void top_k_rows(const float* in, float* values, float* indices, size_t rows, size_t cols, size_t k,
                    bool largest) override;
    void softmax_rows(const float* in, float* out, size_t rows, size_t cols) override;
    void logsumexp_rows(const float* in, float* out, size_t rows, size_t cols) override;
    void gather_rows(const float* table, const float* indices, float* out, size_t count, size_t dim) override;
    /** The underlying C context, for the generation entry points. */
    [[nodiscard]] psx_ctx* context() const noexcept { return ctx_; }

private:
    psx_ctx* ctx_ = nullptr;
    int device_index_ = 0;
};

class PULSATRIX_API Shape {
public:
    Shape() = default;
    Shape(std::initializer_list<int64_t> dims) : dims_(dims) {}
    explicit Shape(std::vector<int64_t> dims) : dims_(std::move(dims)) {}
    [[nodiscard]] int64_t rank() const { return static_cast<int64_t>(dims_.size()); }
    [[nodiscard]] int64_t dim(int64_t i) const { return dims_.at(static_cast<size_t>(i)); }
    [[nodiscard]] int64_t numel() const {
        int64_t n = 1;
        for (int64_t d : dims_) n *= d;
        return n;
    }
    bool operator==(const Shape& other) const { return dims_ == other.dims_; }

private:
    std::vector<int64_t> dims_;
};

/** A float tensor owned through its backend; only what top_k() and its callers need. */
class PULSATRIX_API Tensor {
public:
    Tensor(Shape shape, DeviceBackend* backend);
    Tensor(Shape shape, DeviceBackend* backend, const std::vector<float>& values);
    ~Tensor();
    Tensor(Tensor&& other) noexcept;
    Tensor& operator=(Tensor&& other) noexcept;
    Tensor(const Tensor&) = delete;
    Tensor& operator=(const Tensor&) = delete;
    [[nodiscard]] const Shape& shape() const { return shape_; }
    [[nodiscard]] int64_t rank() const { return shape_.rank(); }
    [[nodiscard]] int64_t numel() const { return shape_.numel(); }
    [[nodiscard]] float* data() { return data_; }
    [[nodiscard]] const float* data() const { return data_; }
    [[nodiscard]] DeviceBackend* backend() const { return backend_; }
    [[nodiscard]] DeviceType device() const { return backend_->device(); }
    [[nodiscard]] std::vector<float> to_host_vector() const;

private:
    Shape shape_;
    DeviceBackend* backend_ = nullptr;
    float* data_ = nullptr;
};

}  // namespace pulsatrix
