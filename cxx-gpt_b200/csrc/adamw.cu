// The kernel that follows the gradient all-reduce of the data-parallel step: one pass over the flat
// fp32 parameter, gradient and moment buffers that
//   - turns the all-reduced SUM of the ranks' gradients into their mean (g * grad_scale, 1/world),
//   - applies AdamW exactly as the reference's optimiser does (src/GPT/gpt_cuda_kernels.cu:488-501 with
//     the host factors of src/GPT/gpt_gpt.hpp:273-278: alpha = lr*sqrt(1-beta2^t)/(1-beta1^t),
//     eps_hat = eps*sqrt(1-beta2^t), decoupled decay lr*wd*data taken from the value before the step),
//   - and accumulates the squared norm of the mean gradient (the reference does that in a separate
//     kernel per parameter with a cudaMalloc and a blocking copy each, gpt_cuda_kernels.cu:517-547).
// With a bf16 gradient (mixed precision) the same pass also writes the bf16 working copy of the parameters that
// the next forward pass reads.  HBM-bound: 16 bytes read and 12 written per parameter (14 and 14 mixed); 16-byte accesses, a grid of a few CTAs per SM
// striding over the buffer, one atomic per CTA for the norm.
#include "internal.cuh"
#include <algorithm>
#include <cmath>

namespace cxxattn {
namespace {

struct AdamArgs {
    float grad_scale, lr, beta1, beta2, wd, alpha, eps_hat;
};

__device__ __forceinline__ float adam_one(float& p, float g, float& m, float& v, const AdamArgs& a) {
    g *= a.grad_scale;
    const float nm = a.beta1 * m + (1.0f - a.beta1) * g;
    const float nv = a.beta2 * v + (1.0f - a.beta2) * g * g;
    m = nm;
    v = nv;
    p -= a.alpha * nm / (sqrtf(nv) + a.eps_hat) + a.lr * a.wd * p;
    return g * g;
}

// MIXED: the gradient is bf16 and a bf16 copy of the updated parameter is written beside the fp32 master
// (mixed-precision training: the forward and backward passes read the copy, the optimiser owns the master).
template <bool MIXED>
__global__ void __launch_bounds__(256) adamw_fused_kernel(float* __restrict__ param, const void* __restrict__ grad_,
                                                         float* __restrict__ m, float* __restrict__ v,
                                                         __nv_bfloat16* __restrict__ copy, size_t n, AdamArgs a,
                                                         float* __restrict__ norm_sq) {
    __shared__ float part[8];
    float acc = 0.f;
    const size_t n4 = n / 4;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const float* grad = static_cast<const float*>(grad_);
    const __nv_bfloat16* gradh = static_cast<const __nv_bfloat16*>(grad_);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 p = reinterpret_cast<float4*>(param)[i];
        float4 g;
        if (MIXED) {
            const uint2 h = reinterpret_cast<const uint2*>(gradh)[i];
            const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&h.x));
            const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&h.y));
            g = make_float4(lo.x, lo.y, hi.x, hi.y);
        } else {
            g = reinterpret_cast<const float4*>(grad)[i];
        }
        float4 mm = reinterpret_cast<float4*>(m)[i], vv = reinterpret_cast<float4*>(v)[i];
        acc += adam_one(p.x, g.x, mm.x, vv.x, a);
        acc += adam_one(p.y, g.y, mm.y, vv.y, a);
        acc += adam_one(p.z, g.z, mm.z, vv.z, a);
        acc += adam_one(p.w, g.w, mm.w, vv.w, a);
        reinterpret_cast<float4*>(param)[i] = p;
        reinterpret_cast<float4*>(m)[i] = mm;
        reinterpret_cast<float4*>(v)[i] = vv;
        if (MIXED) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(p.x, p.y), hi = __floats2bfloat162_rn(p.z, p.w);
            reinterpret_cast<uint2*>(copy)[i] = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        }
    }
    // the last n % 4 elements
    for (size_t i = n4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        acc += adam_one(param[i], MIXED ? __bfloat162float(gradh[i]) : grad[i], m[i], v[i], a);
        if (MIXED) copy[i] = __float2bfloat16_rn(param[i]);
    }
    if (norm_sq == nullptr) return;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (threadIdx.x % 32 == 0) part[threadIdx.x / 32] = acc;
    __syncthreads();
    if (threadIdx.x < 8) {
        acc = part[threadIdx.x];
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffu, acc, o);
        if (threadIdx.x == 0) atomicAdd(norm_sq, acc);
    }
}

}  // namespace

int adamw_fused(float* param, const void* grad, int grad_dtype, float* m, float* v, void* param_copy, size_t n,
                float grad_scale, float lr, float beta1, float beta2, float wd, float eps, int step, float* norm_sq,
                cudaStream_t st) {
    for (const void* q : {(const void*)param, grad, (const void*)m, (const void*)v})
        if (reinterpret_cast<uintptr_t>(q) % 16) return CXXATTN_ERR_ALIGNMENT;
    const bool mixed = grad_dtype == CXXATTN_BF16;
    if (mixed && (param_copy == nullptr || reinterpret_cast<uintptr_t>(param_copy) % 8)) return CXXATTN_ERR_ALIGNMENT;
    const float corr1 = 1.0f - powf(beta1, (float)step), corr2 = 1.0f - powf(beta2, (float)step);
    AdamArgs a;
    a.grad_scale = grad_scale; a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.wd = wd;
    a.alpha = lr * sqrtf(corr2) / corr1;
    a.eps_hat = eps * sqrtf(corr2);
    const size_t want = (n / 4 + 255) / 256;
    const unsigned grid = (unsigned)std::max<size_t>(1, std::min<size_t>(want, (size_t)sm_count() * 8));
    if (mixed)
        adamw_fused_kernel<true><<<grid, 256, 0, st>>>(param, grad, m, v, static_cast<__nv_bfloat16*>(param_copy), n, a,
                                                       norm_sq);
    else
        adamw_fused_kernel<false><<<grid, 256, 0, st>>>(param, grad, m, v, nullptr, n, a, norm_sq);
    return check_launch();
}

}  // namespace cxxattn
