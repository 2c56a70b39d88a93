// Builds the reference's own CUDA kernels into a shared object.  TEST / BASELINE INFRASTRUCTURE ONLY.
//
// The reference's src/TwoStage/two_stage_cuda_kernels.cu and src/LinearAttention/
// linear_cuda_kernels.cu are compiled UNMODIFIED, where they lie in the reference tree, for
// sm_100 against the TensorN stand-in (the reference ships no TensorN); this file only adds
// extern "C" callers that wrap raw device pointers in non-owning CudaTensor views.  The result,
// oracle/_ref/libref_cuda.so, is used to check this library's kernels against the reference's on
// the GPU and to time the reference's serial-scan kernels on the same box.
#include "TwoStage/two_stage_cuda_kernels.cuh"
#include "LinearAttention/linear_cuda_kernels.cuh"

namespace {
typedef CudaTensor<float> T;
T v(const float* p, std::vector<size_t> shape) { return T::view(const_cast<float*>(p), std::move(shape)); }
}  // namespace

extern "C" {

int refcuda_mha_fwd(const float* Q, const float* K, const float* V, float* O, size_t B, size_t S, size_t H, size_t Dh) {
    try {
        T q = v(Q, {B * S, H * Dh}), k = v(K, {B * S, H * Dh}), vv = v(V, {B * S, H * Dh}), o = v(O, {B * S, H * Dh});
        two_stage_cuda::fused_mha_fwd(q, k, vv, o, B, S, H, Dh);
        return 0;
    } catch (...) { return -1; }
}

int refcuda_mha_bwd(const float* Q, const float* K, const float* V, const float* O, const float* dO, float* dQ,
                    float* dK, float* dV, size_t B, size_t S, size_t H, size_t Dh) {
    try {
        std::vector<size_t> sh = {B * S, H * Dh};
        T q = v(Q, sh), k = v(K, sh), vv = v(V, sh), o = v(O, sh), g = v(dO, sh), dq = v(dQ, sh), dk = v(dK, sh),
          dv = v(dV, sh);
        two_stage_cuda::fused_mha_bwd(q, k, vv, o, g, dq, dk, dv, B, S, H, Dh);
        return 0;
    } catch (...) { return -1; }
}

// ELU+1 kernel attention, forward + the three backward steps, as StageBlock calls them
// (two_stage_gpt.hpp:121, 149-156).  Scratch tensors are allocated here, outside any timing the
// caller does around the individual steps being irrelevant: the caller times the whole call.
int refcuda_kernel_attn_fwd_bwd(const float* Q, const float* K, const float* V, const float* dO, float* O, float* den,
                                float* dQ, float* dK, float* dV, float* zc, float* Sbuf, float* zbuf, float* dnum,
                                float* dden, size_t B, size_t S, size_t D, size_t E, int do_bwd) {
    try {
        const size_t N = B * S;
        T q = v(Q, {N, D}), k = v(K, {N, D}), vv = v(V, {N, E}), g = v(dO, {N, E}), o = v(O, {N, E}), dn = v(den, {N}),
          z = v(zc, {N, D}), sb = v(Sbuf, {B * E, D}), zb = v(zbuf, {B, D}), nu = v(dnum, {N, E}), dd = v(dden, {N}),
          dq = v(dQ, {N, D}), dk = v(dK, {N, D}), dv = v(dV, {N, E});
        two_stage_cuda::kernel_attn_fwd(q, k, vv, o, dn, z, sb, zb, B, S, D, E);
        if (do_bwd) {
            two_stage_cuda::kernel_attn_bwd_step1(o, g, dn, nu, dd, N, E);
            two_stage_cuda::kernel_attn_bwd_dQ(k, vv, nu, dd, z, q, dq, sb, B, S, D, E);
            two_stage_cuda::kernel_attn_bwd_dKdV(q, k, vv, nu, dd, dk, dv, B, S, D, E);
        }
        return 0;
    } catch (...) { return -1; }
}

// LinearGPT scan on pre-mapped features, forward + backward steps (linear_gpt.hpp:109-112, 154-167).
int refcuda_linear_fwd_bwd(const float* Qp, const float* Kp, const float* V, const float* dO, float* O, float* den,
                           float* dQp, float* dKp, float* dV, float* zc, float* Sbuf, float* zbuf, float* dnum,
                           float* dden, size_t B, size_t S, size_t D, size_t E, int do_bwd) {
    try {
        const size_t N = B * S;
        T q = v(Qp, {N, D}), k = v(Kp, {N, D}), vv = v(V, {N, E}), g = v(dO, {N, E}), o = v(O, {N, E}), dn = v(den, {N}),
          z = v(zc, {N, D}), sb = v(Sbuf, {B * D, E}), zb = v(zbuf, {B, D}), nu = v(dnum, {N, E}), dd = v(dden, {N}),
          dq = v(dQp, {N, D}), dk = v(dKp, {N, D}), dv = v(dV, {N, E});
        linear_cuda::causal_linear_attention_fwd(q, k, vv, o, dn, z, sb, zb, B, S, D, E);
        if (do_bwd) {
            linear_cuda::causal_linear_attention_bwd_step1(o, g, dn, nu, dd, N, E);
            linear_cuda::causal_linear_attention_bwd_dQ(k, vv, nu, dd, z, dq, sb, B, S, D, E);
            linear_cuda::causal_linear_attention_bwd_dKdV(q, k, vv, nu, dd, dk, dv, B, S, D, E);
        }
        return 0;
    } catch (...) { return -1; }
}

}  // extern "C"
