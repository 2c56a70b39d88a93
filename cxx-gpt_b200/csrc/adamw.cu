// The kernel that follows the gradient all-reduce of the data-parallel step: one pass over the flat
// fp32 parameter, gradient and moment buffers that
//   - turns the all-reduced SUM of the ranks' gradients into their mean (g * grad_scale, 1/world),
//   - applies AdamW exactly as the reference's optimiser does (src/GPT/gpt_cuda_kernels.cu:488-501 with
//     the host factors of src/GPT/gpt_gpt.hpp:273-278: alpha = lr*sqrt(1-beta2^t)/(1-beta1^t),
//     eps_hat = eps*sqrt(1-beta2^t), decoupled decay lr*wd*data taken from the value before the step),
//   - and accumulates the squared norm of the mean gradient (the reference does that in a separate
//     kernel per parameter with a cudaMalloc and a blocking copy each, gpt_cuda_kernels.cu:517-547).
// HBM-bound: 16 bytes read and 12 written per parameter; 16-byte accesses, a grid of a few CTAs per SM
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

__global__ void __launch_bounds__(256) adamw_fused_kernel(float* __restrict__ param, const float* __restrict__ grad,
                                                         float* __restrict__ m, float* __restrict__ v, size_t n,
                                                         AdamArgs a, float* __restrict__ norm_sq) {
    __shared__ float part[8];
    float acc = 0.f;
    const size_t n4 = n / 4;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 p = reinterpret_cast<float4*>(param)[i];
        const float4 g = reinterpret_cast<const float4*>(grad)[i];
        float4 mm = reinterpret_cast<float4*>(m)[i], vv = reinterpret_cast<float4*>(v)[i];
        acc += adam_one(p.x, g.x, mm.x, vv.x, a);
        acc += adam_one(p.y, g.y, mm.y, vv.y, a);
        acc += adam_one(p.z, g.z, mm.z, vv.z, a);
        acc += adam_one(p.w, g.w, mm.w, vv.w, a);
        reinterpret_cast<float4*>(param)[i] = p;
        reinterpret_cast<float4*>(m)[i] = mm;
        reinterpret_cast<float4*>(v)[i] = vv;
    }
    // the last n % 4 elements
    for (size_t i = n4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        acc += adam_one(param[i], grad[i], m[i], v[i], a);
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

int adamw_fused(float* param, const float* grad, float* m, float* v, size_t n, float grad_scale, float lr, float beta1,
                float beta2, float wd, float eps, int step, float* norm_sq, cudaStream_t st) {
    for (const void* q : {(const void*)param, (const void*)grad, (const void*)m, (const void*)v})
        if (reinterpret_cast<uintptr_t>(q) % 16) return CXXATTN_ERR_ALIGNMENT;
    const float corr1 = 1.0f - powf(beta1, (float)step), corr2 = 1.0f - powf(beta2, (float)step);
    AdamArgs a;
    a.grad_scale = grad_scale; a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.wd = wd;
    a.alpha = lr * sqrtf(corr2) / corr1;
    a.eps_hat = eps * sqrtf(corr2);
    const size_t want = (n / 4 + 255) / 256;
    const unsigned grid = (unsigned)std::max<size_t>(1, std::min<size_t>(want, (size_t)sm_count() * 8));
    adamw_fused_kernel<<<grid, 256, 0, st>>>(param, grad, m, v, n, a, norm_sq);
    return check_launch();
}

}  // namespace cxxattn
