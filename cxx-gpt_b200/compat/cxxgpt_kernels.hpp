// The C++ kernel entry points that CXX-GPT's models call, declared with the signatures of
// src/TwoStage/two_stage_cuda_kernels.cuh:18-85 and src/LinearAttention/linear_cuda_kernels.cuh:11-46
// and implemented in cxxgpt_kernels.cpp on top of the C-ABI of libcxxattn.so.  A CXX-GPT build keeps
// its own two headers and links cxxgpt_kernels.cpp + libcxxattn.so instead of its two .cu files;
// this header exists so that the adapter also compiles without the CXX-GPT tree.
#pragma once
#include "TensorN.hpp"

// Not in the reference: lets the kept fp32 softmax signatures run on the bf16 tensor-core kernels
// (head dimension 64; tolerance 2e-2 instead of 1e-5).  Default: off, or CXXATTN_COMPAT_PRECISION=tensorcore.
namespace cxxattn_compat {
void set_tensorcore(bool on);
// LinearGPT's mapped features carry zero columns from n_embd to the next power of two
// (linear_cuda_kernels.cu:316-323).  On (the default; CXXATTN_COMPAT_SKIP_PADDING=0 turns it off): the scan
// entry points skip those columns for tensors that this adapter's phi_elu_forward produced, with the
// same results.
void set_skip_padding(bool on);
// Stage-1 attention of TwoStageGPT with its rotary embedding folded in: what
//   rope_fwd(Q, K, ..., Dh); fused_mha_fwd(Q, K, V, O, ...)            (two_stage_gpt.hpp:102-106)
//   fused_mha_bwd(Q, K, V, O, dO, dQ, dK, dV, ...); rope_bwd(dQ, dK, ..., Dh)   (two_stage_gpt.hpp:171-174)
// compute, but Q and K are the projections BEFORE the rotation and are left untouched: the rotation
// runs in the same pass as the conversion the attention kernels need anyway, and the gradients come
// back already un-rotated.  Follows the precision switch above.
void rope_fused_mha_fwd(const TensorN::CudaTensor<float>& Q, const TensorN::CudaTensor<float>& K,
                        const TensorN::CudaTensor<float>& V, TensorN::CudaTensor<float>& O, size_t B, size_t S,
                        size_t H, size_t Dh);
void rope_fused_mha_bwd(const TensorN::CudaTensor<float>& Q, const TensorN::CudaTensor<float>& K,
                        const TensorN::CudaTensor<float>& V, const TensorN::CudaTensor<float>& O,
                        const TensorN::CudaTensor<float>& dO, TensorN::CudaTensor<float>& dQ,
                        TensorN::CudaTensor<float>& dK, TensorN::CudaTensor<float>& dV, size_t B, size_t S, size_t H,
                        size_t Dh);
}

namespace two_stage_cuda {
using TensorN::CudaTensor;
typedef const CudaTensor<float>& In;
typedef CudaTensor<float>& Out;
void fused_mha_fwd(In Q, In K, In V, Out O, size_t B, size_t S, size_t H, size_t Dh);
void fused_mha_bwd(In Q, In K, In V, In O, In dO, Out dQ, Out dK, Out dV, size_t B, size_t S, size_t H, size_t Dh);
void kernel_attn_fwd(In Q, In K, In V, Out O, Out den_cache, Out z_cache, Out S_buf, Out z_buf,
                     size_t B, size_t S, size_t D, size_t E);
void kernel_attn_bwd_step1(In O, In dO, In den_cache, Out dnum, Out dden, size_t N, size_t E);
void kernel_attn_bwd_dQ(In K, In V, In dnum, In dden, In z_cache, In Q, Out dQ, Out S_buf,
                        size_t B, size_t S, size_t D, size_t E);
void kernel_attn_bwd_dKdV(In Q, In K, In V, In dnum, In dden, Out dK, Out dV, size_t B, size_t S, size_t D, size_t E);
void rope_fwd(Out Q, Out K, size_t B, size_t S, size_t D, size_t head_dim);
void rope_bwd(Out dQ, Out dK, size_t B, size_t S, size_t D, size_t head_dim);
void gelu_exact(In A, Out C);
void gelu_exact_deriv(In A, Out C);
}  // namespace two_stage_cuda

namespace linear_cuda {
using TensorN::CudaTensor;
typedef const CudaTensor<float>& In;
typedef CudaTensor<float>& Out;
void causal_linear_attention_fwd(In Q_phi, In K_phi, In V, Out O, Out den_cache, Out z_cache, Out S_buf, Out z_buf,
                                 size_t B, size_t S, size_t D, size_t E);
void causal_linear_attention_bwd_step1(In O, In dO, In den_cache, Out dnum, Out dden, size_t N, size_t E);
void causal_linear_attention_bwd_dQ(In K_phi, In V, In dnum, In dden, In z_cache, Out dQ_phi, Out S_buf,
                                    size_t B, size_t S, size_t D, size_t E);
void causal_linear_attention_bwd_dKdV(In Q_phi, In K_phi, In V, In dnum, In dden, Out dK_phi, Out dV,
                                      size_t B, size_t S, size_t D, size_t E);
void phi_elu_forward(In x, Out phi, size_t D, size_t E);
void phi_elu_backward(In dphi, In x, Out dx, size_t D, size_t E);
}  // namespace linear_cuda
