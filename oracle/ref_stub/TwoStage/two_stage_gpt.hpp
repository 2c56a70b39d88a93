// Host-only stand-in used ONLY to compile the reference's kernel_test.cpp (where it lies in the
// reference tree) into oracle/_ref/ so that its static CPU reference functions can be called.
// The reference file includes "TwoStage/two_stage_gpt.hpp", which needs the TensorN library that
// is not part of the reference tree; this directory is put first on the include path instead.
// main() of that file is renamed and never called, so the tensor types below only have to
// satisfy the compiler and the two_stage_cuda entry points are declared but never run.
#pragma once
#include <cstddef>
#include <initializer_list>
#include <memory>
#include <vector>

namespace TensorN {
template <typename T>
struct Tensor {
    std::shared_ptr<std::vector<T>> data;
    Tensor() : data(std::make_shared<std::vector<T>>()) {}
    Tensor(std::initializer_list<size_t>, const std::vector<T>& v)
        : data(std::make_shared<std::vector<T>>(v)) {}
};
template <typename T>
struct CudaTensor {
    CudaTensor() {}
    CudaTensor(std::initializer_list<size_t>) {}
    static CudaTensor fromTensor(const Tensor<T>&) { return CudaTensor(); }
    Tensor<T> toTensor() const { return Tensor<T>(); }
};
}  // namespace TensorN

namespace two_stage_cuda {
using TensorN::CudaTensor;
typedef const CudaTensor<float>& In;
typedef CudaTensor<float>& Out;
void fused_mha_fwd(In, In, In, Out, size_t, size_t, size_t, size_t);
void fused_mha_bwd(In, In, In, In, In, Out, Out, Out, size_t, size_t, size_t, size_t);
void kernel_attn_fwd(In, In, In, Out, Out, Out, Out, Out, size_t, size_t, size_t, size_t);
void kernel_attn_bwd_step1(In, In, In, Out, Out, size_t, size_t);
void kernel_attn_bwd_dQ(In, In, In, In, In, In, Out, Out, size_t, size_t, size_t, size_t);
void kernel_attn_bwd_dKdV(In, In, In, In, In, Out, Out, size_t, size_t, size_t, size_t);
void rope_fwd(Out, Out, size_t, size_t, size_t, size_t);
void rope_bwd(Out, Out, size_t, size_t, size_t, size_t);
}  // namespace two_stage_cuda
