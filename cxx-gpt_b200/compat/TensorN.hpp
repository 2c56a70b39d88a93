// Minimal stand-in for the TensorN library, which CXX-GPT builds against but does not ship
// (its TensorN/ directory is empty).  It provides exactly what the attention kernel headers and
// the kernel unit test touch: host Tensor<T>, device CudaTensor<T> with device_ptr / shape / size /
// memset_zero / fromTensor / toTensor / copyFromHost, and CHECK_CUDA_ERROR.  When the real TensorN
// is available this directory is simply left off the include path.
#pragma once
#define TENSORN_CUDA_AVAILABLE 1
#include <cuda_runtime.h>
#include <cstddef>
#include <initializer_list>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#define CHECK_CUDA_ERROR(expr)                                                                   \
    do {                                                                                         \
        cudaError_t tensorn_err_ = (expr);                                                       \
        if (tensorn_err_ != cudaSuccess)                                                         \
            throw std::runtime_error(std::string("CUDA error: ") + cudaGetErrorString(tensorn_err_) + \
                                     " at " + __FILE__ + ":" + std::to_string(__LINE__));        \
    } while (0)

namespace TensorN {

inline size_t shape_size(const std::vector<size_t>& s) {
    size_t n = 1;
    for (size_t d : s) n *= d;
    return s.empty() ? 0 : n;
}

template <typename T>
class Tensor {
public:
    std::shared_ptr<std::vector<T>> data;
    Tensor() : data(std::make_shared<std::vector<T>>()) {}
    explicit Tensor(std::vector<size_t> shape)
        : data(std::make_shared<std::vector<T>>(shape_size(shape))), shape_(std::move(shape)) {}
    Tensor(std::vector<size_t> shape, const std::vector<T>& values)
        : data(std::make_shared<std::vector<T>>(values)), shape_(std::move(shape)) {}
    const std::vector<size_t>& shape() const { return shape_; }
    size_t size() const { return data->size(); }
    T& operator[](size_t i) { return (*data)[i]; }
    const T& operator[](size_t i) const { return (*data)[i]; }

private:
    std::vector<size_t> shape_;
};

template <typename T>
class CudaTensor {
public:
    CudaTensor() = default;
    CudaTensor(std::initializer_list<size_t> shape) : CudaTensor(std::vector<size_t>(shape)) {}
    explicit CudaTensor(std::vector<size_t> shape) : shape_(std::move(shape)), n_(shape_size(shape_)) {
        if (n_) CHECK_CUDA_ERROR(cudaMalloc(reinterpret_cast<void**>(&ptr_), n_ * sizeof(T)));
    }
    CudaTensor(const CudaTensor& o) : CudaTensor(o.shape_) {
        if (n_) CHECK_CUDA_ERROR(cudaMemcpy(ptr_, o.ptr_, n_ * sizeof(T), cudaMemcpyDeviceToDevice));
    }
    CudaTensor(CudaTensor&& o) noexcept : shape_(std::move(o.shape_)), n_(o.n_), ptr_(o.ptr_), owns_(o.owns_) {
        o.ptr_ = nullptr;
        o.n_ = 0;
    }
    CudaTensor& operator=(CudaTensor o) noexcept {
        std::swap(shape_, o.shape_);
        std::swap(n_, o.n_);
        std::swap(ptr_, o.ptr_);
        std::swap(owns_, o.owns_);
        return *this;
    }
    ~CudaTensor() {
        if (ptr_ && owns_) cudaFree(ptr_);
    }
    // Not part of TensorN: wraps device memory owned by someone else (used by test harnesses that
    // hand raw pointers to functions taking CudaTensor references).
    static CudaTensor view(T* ptr, std::vector<size_t> shape) {
        CudaTensor c;
        c.shape_ = std::move(shape);
        c.n_ = shape_size(c.shape_);
        c.ptr_ = ptr;
        c.owns_ = false;
        return c;
    }
    T* device_ptr() { return ptr_; }
    const T* device_ptr() const { return ptr_; }
    const std::vector<size_t>& shape() const { return shape_; }
    size_t size() const { return n_; }
    void memset_zero() {
        if (n_) CHECK_CUDA_ERROR(cudaMemset(ptr_, 0, n_ * sizeof(T)));
    }
    void copyFromHost(const T* src, size_t n) {
        CHECK_CUDA_ERROR(cudaMemcpy(ptr_, src, n * sizeof(T), cudaMemcpyHostToDevice));
    }
    static CudaTensor fromTensor(const Tensor<T>& t) {
        CudaTensor c(t.shape());
        if (c.n_) c.copyFromHost(t.data->data(), c.n_);
        return c;
    }
    Tensor<T> toTensor() const {
        Tensor<T> t(shape_);
        if (n_) CHECK_CUDA_ERROR(cudaMemcpy(t.data->data(), ptr_, n_ * sizeof(T), cudaMemcpyDeviceToHost));
        return t;
    }

private:
    std::vector<size_t> shape_;
    size_t n_ = 0;
    T* ptr_ = nullptr;
    bool owns_ = true;
};

}  // namespace TensorN
