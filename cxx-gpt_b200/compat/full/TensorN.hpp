// Wider stand-in for the TensorN library (absent from the CXX-GPT tree), for compiling CXX-GPT's
// MODEL headers unmodified: src/GPT/gpt_gpt.hpp and src/TwoStage/two_stage_gpt.hpp.  On top of the
// tensor types of ../TensorN.hpp it declares the dense operations those headers call
// (gpt_gpt.hpp:84-114, 365-438; two_stage_gpt.hpp:143-199), implemented in tensorn_ops.cu with
// cuBLAS and plain CUDA kernels, a small device memory pool, and GGUF entry points that only throw: the checks that are built
// on this never read or write a checkpoint.  Semantics are taken from the call sites: row-major
// matrices, matmul(A[m,k], B[k,n], C[m,n]), transpose(A[m,n], At[n,m]), element-wise add and
// multiply, sum_axis(A, 0) -> column sums, softmax over the last axis, tanh-form GELU matching
// gpt_cuda::gelu_deriv (gpt_cuda_kernels.cu).
#pragma once
#include "../TensorN.hpp"

#include <cstdint>
#include <unordered_map>
#include <utility>
#include <variant>

namespace TensorN {

using GGUFMetadataValue = std::variant<uint64_t, int64_t, float, double, bool, std::string>;

inline void save_gguf_multi(const std::vector<std::pair<std::string, Tensor<float>>>&, const std::string&,
                            const std::unordered_map<std::string, GGUFMetadataValue>&) {
    throw std::runtime_error("GGUF output is not part of this TensorN stand-in");
}
inline std::unordered_map<std::string, GGUFMetadataValue> gguf_read_metadata(const std::string&) {
    throw std::runtime_error("GGUF input is not part of this TensorN stand-in");
}
template <typename T>
std::unordered_map<std::string, Tensor<T>> load_gguf_multi(const std::string&) {
    throw std::runtime_error("GGUF input is not part of this TensorN stand-in");
}

// Device allocations handed out and taken back by size (gpt_cuda_kernels.cu:382-397,
// two_stage_train.cpp:245-348): freed blocks are kept and reused for requests of the same size.
class CudaMemoryPool {
public:
    static CudaMemoryPool& instance() {
        static CudaMemoryPool pool;
        return pool;
    }
    void* acquire(size_t bytes) {
        auto& spare = free_[bytes];
        void* p = nullptr;
        if (!spare.empty()) {
            p = spare.back();
            spare.pop_back();
        } else {
            CHECK_CUDA_ERROR(cudaMalloc(&p, bytes ? bytes : 1));
        }
        size_[p] = bytes;
        return p;
    }
    void release(void* p) {
        auto it = size_.find(p);
        if (it == size_.end()) return;
        free_[it->second].push_back(p);
        size_.erase(it);
    }

private:
    std::unordered_map<size_t, std::vector<void*>> free_;
    std::unordered_map<void*, size_t> size_;
};

namespace cuda {
void set_tf32(bool on);
void matmul(const CudaTensor<float>& A, const CudaTensor<float>& B, CudaTensor<float>& C);
void transpose(const CudaTensor<float>& A, CudaTensor<float>& At);
void add(const CudaTensor<float>& A, const CudaTensor<float>& B, CudaTensor<float>& C);
void multiply(const CudaTensor<float>& A, const CudaTensor<float>& B, CudaTensor<float>& C);
void multiply_scalar(const CudaTensor<float>& A, float s, CudaTensor<float>& C);
CudaTensor<float> sum_axis(const CudaTensor<float>& A, int axis);
void softmax(const CudaTensor<float>& A, CudaTensor<float>& out, int axis);
void gelu(const CudaTensor<float>& A, CudaTensor<float>& out);
}  // namespace cuda

}  // namespace TensorN
