// The gradient exchange of the data-parallel step and the optimiser step as ONE kernel over peer
// memory (NVLink / NVSwitch loads and stores), instead of an all-reduce followed by the AdamW pass:
//
//   rank r owns the contiguous shard [lo, lo + count) of the flat parameter buffer.  For its shard it
//     - reads the gradient of every rank (its own from local memory, the others' through their
//       peer-mapped buffers) and sums them in fp32, in a fixed order,
//     - applies the mean and AdamW to its fp32 master parameters and moments (as adamw.cu does; the
//       moments exist for the shard only),
//     - writes the updated parameters, in the dtype the forward pass reads, into the parameter buffer of
//       EVERY rank (its own included).
//
// The link traffic is that of a reduce-scatter followed by an all-gather, i.e. of an all-reduce:
// (world-1)/world of the gradient bytes come into each GPU as load responses and the same amount of
// parameter bytes arrive as the peers' stores, and as much leaves it.  What the fusion removes is the
// full-size optimiser pass on every rank (each rank updates 1/world of the parameters and keeps 1/world of
// the master copy and moments), the gradient sum's round trip through memory, and all but one launch.
// The kernel does not wait for anything: the caller orders it after "every rank's gradients are final"
// and before "every rank may read its parameters" with two stream-ordered barriers (a one-element
// all-reduce each; the second one carries the partial squared gradient norms).  Plain loads and stores
// only: no TMA, no multicast.
//
// The buffers peers read and write are cudaMalloc allocations exported with CUDA IPC handles
// (cxxattn_peer_*): one process per GPU opens the other ranks' handles once at start-up.
#include "internal.cuh"
#include <algorithm>
#include <cmath>
#include <cstring>

namespace cxxattn {
namespace {

constexpr int kMaxPeers = 16;

struct ExchangeArgs {
    const void* grad[kMaxPeers];  // every rank's gradient buffer, whole length
    void* copy[kMaxPeers];        // every rank's parameter buffer as the forward pass reads it, whole length
    float grad_scale, lr, beta1, beta2, wd, alpha, eps_hat;
    int world, rank;
};

__device__ __forceinline__ float adam_one(float& p, float g, float& m, float& v, const ExchangeArgs& a) {
    g *= a.grad_scale;
    const float nm = a.beta1 * m + (1.0f - a.beta1) * g;
    const float nv = a.beta2 * v + (1.0f - a.beta2) * g * g;
    m = nm;
    v = nv;
    p -= a.alpha * nm / (sqrtf(nv) + a.eps_hat) + a.lr * a.wd * p;
    return g * g;
}

__device__ __forceinline__ void add_bf16x8(float (&acc)[8], const uint4 h) {
    const uint32_t w[4] = {h.x, h.y, h.z, h.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
    }
}

// BF16: gradients and parameter copies are bf16 (mixed precision), eight elements per thread and pass;
// otherwise fp32, four elements.  `lo` and `count` are multiples of the vector width.
template <bool BF16>
__global__ void __launch_bounds__(256) adamw_exchange_kernel(float* __restrict__ param, float* __restrict__ m,
                                                            float* __restrict__ v, ExchangeArgs a, size_t lo,
                                                            size_t count, float* __restrict__ norm_sq) {
    constexpr int VEC = BF16 ? 8 : 4;
    __shared__ float part[8];
    float accn = 0.f;
    const size_t nvec = count / VEC;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        const size_t e = lo + i * VEC;  // element index in the whole buffers
        // every load of the pass is issued before the first use: the local master and moments, then the
        // ranks' gradients in the order rank+1, rank+2, ..., rank (at any moment the ranks read from
        // different peers), eight ranks to a batch
        float p[VEC], mm[VEC], vv[VEC];
#pragma unroll
        for (int k = 0; k < VEC; k += 4) {
            *reinterpret_cast<float4*>(&p[k]) = reinterpret_cast<const float4*>(param + i * VEC)[k / 4];
            *reinterpret_cast<float4*>(&mm[k]) = reinterpret_cast<const float4*>(m + i * VEC)[k / 4];
            *reinterpret_cast<float4*>(&vv[k]) = reinterpret_cast<const float4*>(v + i * VEC)[k / 4];
        }
        float g[VEC];
#pragma unroll
        for (int k = 0; k < VEC; k++) g[k] = 0.f;
        for (int q0 = 0; q0 < a.world; q0 += 8) {
            uint4 raw[8];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int q = q0 + j;
                if (q < a.world) {
                    int src = a.rank + 1 + q;
                    if (src >= a.world) src -= a.world;
                    raw[j] = *reinterpret_cast<const uint4*>(static_cast<const char*>(a.grad[src]) + e * (BF16 ? 2 : 4));
                }
            }
#pragma unroll
            for (int j = 0; j < 8; j++) {
                if (q0 + j < a.world) {
                    if constexpr (BF16) {
                        add_bf16x8(g, raw[j]);
                    } else {
                        g[0] += __uint_as_float(raw[j].x);
                        g[1] += __uint_as_float(raw[j].y);
                        g[2] += __uint_as_float(raw[j].z);
                        g[3] += __uint_as_float(raw[j].w);
                    }
                }
            }
        }
#pragma unroll
        for (int k = 0; k < VEC; k++) accn += adam_one(p[k], g[k], mm[k], vv[k], a);
#pragma unroll
        for (int k = 0; k < VEC; k += 4) {
            reinterpret_cast<float4*>(param + i * VEC)[k / 4] = *reinterpret_cast<const float4*>(&p[k]);
            reinterpret_cast<float4*>(m + i * VEC)[k / 4] = *reinterpret_cast<const float4*>(&mm[k]);
            reinterpret_cast<float4*>(v + i * VEC)[k / 4] = *reinterpret_cast<const float4*>(&vv[k]);
        }
        uint4 out;
        if constexpr (BF16) {
            __nv_bfloat162 h[4];
#pragma unroll
            for (int k = 0; k < 4; k++) h[k] = __floats2bfloat162_rn(p[2 * k], p[2 * k + 1]);
            out = *reinterpret_cast<const uint4*>(h);
        } else {
            out = make_uint4(__float_as_uint(p[0]), __float_as_uint(p[1]), __float_as_uint(p[2]), __float_as_uint(p[3]));
        }
        for (int q = 0; q < a.world; q++) {
            int dst = a.rank + 1 + q;
            if (dst >= a.world) dst -= a.world;
            char* where = static_cast<char*>(a.copy[dst]) + e * (BF16 ? 2 : 4);
            // fp32: this rank's own copy may BE the master buffer just written
            if (BF16 || where != reinterpret_cast<char*>(param + i * VEC)) *reinterpret_cast<uint4*>(where) = out;
        }
    }
    if (norm_sq == nullptr) return;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) accn += __shfl_xor_sync(0xffffffffu, accn, o);
    if (threadIdx.x % 32 == 0) part[threadIdx.x / 32] = accn;
    __syncthreads();
    if (threadIdx.x < 8) {
        accn = part[threadIdx.x];
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) accn += __shfl_xor_sync(0xffu, accn, o);
        if (threadIdx.x == 0) atomicAdd(norm_sq, accn);
    }
}

}  // namespace

int adamw_exchange(float* param_shard, float* m_shard, float* v_shard, const void* const* grads, void* const* copies,
                   int dtype, int world, int rank, size_t lo, size_t count, float grad_scale, float lr, float beta1,
                   float beta2, float wd, float eps, int step, float* norm_sq, cudaStream_t st) {
    const bool bf16 = dtype == CXXATTN_BF16;
    const size_t vec = bf16 ? 8 : 4;
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || lo % vec || count % vec) return CXXATTN_ERR_INVALID;
    for (const void* q : {(const void*)param_shard, (const void*)m_shard, (const void*)v_shard})
        if (reinterpret_cast<uintptr_t>(q) % 16) return CXXATTN_ERR_ALIGNMENT;
    ExchangeArgs a;
    for (int r = 0; r < kMaxPeers; r++) {
        a.grad[r] = nullptr;
        a.copy[r] = nullptr;
    }
    for (int r = 0; r < world; r++) {
        if (grads[r] == nullptr || copies[r] == nullptr) return CXXATTN_ERR_INVALID;
        if (reinterpret_cast<uintptr_t>(grads[r]) % 16 || reinterpret_cast<uintptr_t>(copies[r]) % 16)
            return CXXATTN_ERR_ALIGNMENT;
        a.grad[r] = grads[r];
        a.copy[r] = copies[r];
    }
    const float corr1 = 1.0f - powf(beta1, (float)step), corr2 = 1.0f - powf(beta2, (float)step);
    a.grad_scale = grad_scale; a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.wd = wd;
    a.alpha = lr * sqrtf(corr2) / corr1;
    a.eps_hat = eps * sqrtf(corr2);
    a.world = world;
    a.rank = rank;
    if (count == 0) return CXXATTN_OK;  // more ranks than vectors: this rank owns nothing
    const size_t want = (count / vec + 255) / 256;
    const unsigned grid = (unsigned)std::max<size_t>(1, std::min<size_t>(want, (size_t)sm_count() * 8));
    if (bf16)
        adamw_exchange_kernel<true><<<grid, 256, 0, st>>>(param_shard, m_shard, v_shard, a, lo, count, norm_sq);
    else
        adamw_exchange_kernel<false><<<grid, 256, 0, st>>>(param_shard, m_shard, v_shard, a, lo, count, norm_sq);
    return check_launch();
}

// ---- peer-visible buffers (CUDA IPC) ------------------------------------------------------------
int peer_alloc(size_t bytes, void** ptr) {
    if (ptr == nullptr || bytes == 0) return CXXATTN_ERR_INVALID;
    *ptr = nullptr;
    if (cudaMalloc(ptr, bytes) != cudaSuccess) {
        cudaGetLastError();
        return CXXATTN_ERR_CUDA;
    }
    return CXXATTN_OK;
}
int peer_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? CXXATTN_OK : CXXATTN_ERR_CUDA; }
int peer_export(const void* ptr, unsigned char* handle) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the C-ABI fixes the handle at 64 bytes");
    cudaIpcMemHandle_t h;
    if (ptr == nullptr || handle == nullptr) return CXXATTN_ERR_INVALID;
    if (cudaIpcGetMemHandle(&h, const_cast<void*>(ptr)) != cudaSuccess) {
        cudaGetLastError();
        return CXXATTN_ERR_CUDA;
    }
    memcpy(handle, &h, sizeof(h));
    return CXXATTN_OK;
}
int peer_open(const unsigned char* handle, void** ptr) {
    if (ptr == nullptr || handle == nullptr) return CXXATTN_ERR_INVALID;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    *ptr = nullptr;
    if (cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        cudaGetLastError();
        return CXXATTN_ERR_CUDA;
    }
    return CXXATTN_OK;
}
int peer_close(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? CXXATTN_OK : CXXATTN_ERR_CUDA; }

}  // namespace cxxattn
