// LayerNorm backward for the data-parallel step: dx, dgamma, dbeta from dy, x, gamma and the row
// statistics the forward pass saved (the reference's gpt_cuda::layernorm_backward,
// src/GPT/gpt_cuda_kernels.cu:250-320, which runs one CTA per row and adds every element of dgamma and
// dbeta with its own atomic):
//   xhat = (x - mean) rstd,  g = dy gamma,  dx = rstd (g - (sum(g) + xhat sum(g xhat)) / D),
//   dgamma[c] = sum_r dy xhat,  dbeta[c] = sum_r dy.
// Two launches that each read dy and x once (a few MB, L2-resident between them): a warp per row for dx,
// and for the two column sums the tiling of colsum.cu (64 columns x a group of rows per CTA, fp32 partial
// sums added into a self-cleaning workspace, the last CTA of a column block writes the results).
#include "internal.cuh"
#include <algorithm>

namespace cxxattn {
namespace {

template <typename T>
struct Io;
template <>
struct Io<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
        const float4 q = *reinterpret_cast<const float4*>(p);
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
    static __device__ __forceinline__ float cvt(float x) { return x; }
};
template <>
struct Io<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
        const uint4 q = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
        __nv_bfloat162 h[4];
#pragma unroll
        for (int i = 0; i < 4; i++) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(h);
    }
    static __device__ __forceinline__ __nv_bfloat16 cvt(float x) { return __float2bfloat16_rn(x); }
};

// dx: a warp per row, two sweeps over the row (the second one finds it in the L1).
template <typename T>
__global__ void __launch_bounds__(256) ln_dx_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ gamma,
                                                   const float* __restrict__ mean, const float* __restrict__ rstd,
                                                   T* __restrict__ dx, size_t rows, size_t cols) {
    constexpr int VEC = Io<T>::N;
    const size_t r = (size_t)blockIdx.x * 8 + threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    if (r >= rows) return;
    const T* dyr = dy + r * cols;
    const T* xr = x + r * cols;
    const float m = mean[r], rs = rstd[r];
    float s1 = 0.f, s2 = 0.f;
    for (size_t c = (size_t)lane * VEC; c < cols; c += 32 * VEC) {
        float a[VEC], b[VEC], g[VEC];
        Io<T>::load(dyr + c, a);
        Io<T>::load(xr + c, b);
        Io<T>::load(gamma + c, g);
#pragma unroll
        for (int k = 0; k < VEC; k++) {
            const float gg = a[k] * g[k];
            s1 += gg;
            s2 += gg * ((b[k] - m) * rs);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
        s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    }
    const float inv = 1.0f / (float)cols;
    for (size_t c = (size_t)lane * VEC; c < cols; c += 32 * VEC) {
        float a[VEC], b[VEC], g[VEC], o[VEC];
        Io<T>::load(dyr + c, a);
        Io<T>::load(xr + c, b);
        Io<T>::load(gamma + c, g);
#pragma unroll
        for (int k = 0; k < VEC; k++) {
            const float xh = (b[k] - m) * rs;
            o[k] = rs * (a[k] * g[k] - (s2 * xh + s1) * inv);
        }
        Io<T>::store(dx + r * cols + c, o);
    }
}

constexpr int CB = 64;  // columns per CTA of the column-sum kernel

template <typename T>
__global__ void __launch_bounds__(256) ln_dgdb_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                     const float* __restrict__ mean, const float* __restrict__ rstd,
                                                     T* __restrict__ dgamma, T* __restrict__ dbeta, size_t rows, size_t cols,
                                                     size_t rows_per_group, float* ws, unsigned* counters, size_t ws_cols) {
    constexpr int VEC = Io<T>::N, CT = CB / VEC, RL = 256 / CT;
    __shared__ float part[2][RL][CB + 1];
    __shared__ bool last;
    const int tx = threadIdx.x % CT, ty = threadIdx.x / CT;
    const size_t col = (size_t)blockIdx.x * CB + tx * VEC;
    const size_t r0 = (size_t)blockIdx.y * rows_per_group, r1 = min(rows, r0 + rows_per_group);
    float ag[VEC], ab[VEC];
#pragma unroll
    for (int k = 0; k < VEC; k++) ag[k] = ab[k] = 0.f;
    if (col < cols) {
        for (size_t r = r0 + ty; r < r1; r += RL) {
            float a[VEC], b[VEC];
            Io<T>::load(dy + r * cols + col, a);
            Io<T>::load(x + r * cols + col, b);
            const float m = mean[r], rs = rstd[r];
#pragma unroll
            for (int k = 0; k < VEC; k++) {
                ag[k] += a[k] * ((b[k] - m) * rs);
                ab[k] += a[k];
            }
        }
    }
#pragma unroll
    for (int k = 0; k < VEC; k++) {
        part[0][ty][tx * VEC + k] = ag[k];
        part[1][ty][tx * VEC + k] = ab[k];
    }
    __syncthreads();
    if (threadIdx.x < 2 * CB) {
        const int which = threadIdx.x / CB, cc = threadIdx.x % CB;
        float s = 0.f;
#pragma unroll 8
        for (int j = 0; j < RL; j++) s += part[which][j][cc];
        const size_t c = (size_t)blockIdx.x * CB + cc;
        if (c < cols) atomicAdd(ws + which * ws_cols + c, s);
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(counters + blockIdx.x, 1u) == gridDim.y - 1;
    __syncthreads();
    if (!last) return;
    __threadfence();
    if (threadIdx.x < 2 * CB) {
        const int which = threadIdx.x / CB, cc = threadIdx.x % CB;
        const size_t c = (size_t)blockIdx.x * CB + cc;
        if (c < cols) {
            (which ? dbeta : dgamma)[c] = Io<T>::cvt(__ldcg(ws + which * ws_cols + c));
            ws[which * ws_cols + c] = 0.f;
        }
    }
    if (threadIdx.x == 0) counters[blockIdx.x] = 0u;
}

template <typename T>
int launch(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, void* dx, void* dgamma,
           void* dbeta, size_t rows, size_t cols, float* ws, unsigned* counters, size_t ws_cols, size_t blocks,
           cudaStream_t st) {
    ln_dx_kernel<T><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(static_cast<const T*>(dy), static_cast<const T*>(x),
                                                               static_cast<const T*>(gamma), mean, rstd, static_cast<T*>(dx),
                                                               rows, cols);
    const size_t want = std::max<size_t>(1, ((size_t)sm_count() * 4 + blocks - 1) / blocks);
    const size_t groups = std::max<size_t>(1, std::min<size_t>({want, (rows + 63) / 64, (size_t)65535}));
    const size_t per = (rows + groups - 1) / groups;
    const dim3 grid((unsigned)blocks, (unsigned)((rows + per - 1) / per));
    ln_dgdb_kernel<T><<<grid, 256, 0, st>>>(static_cast<const T*>(dy), static_cast<const T*>(x), mean, rstd,
                                           static_cast<T*>(dgamma), static_cast<T*>(dbeta), rows, cols, per, ws, counters,
                                           ws_cols);
    return check_launch();
}

}  // namespace

size_t layernorm_bwd_workspace(size_t cols) {
    const size_t blocks = (cols + CB - 1) / CB;
    return 2 * blocks * CB * sizeof(float) + blocks * sizeof(unsigned);
}

int layernorm_bwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, void* dx,
                  void* dgamma, void* dbeta, size_t rows, size_t cols, int dtype, void* ws, size_t ws_bytes, cudaStream_t st) {
    const size_t vec = dtype == CXXATTN_BF16 ? 8 : 4;
    if (cols % vec) return CXXATTN_ERR_UNSUPPORTED;
    for (const void* q : {dy, x, gamma, (const void*)dx, (const void*)ws})
        if (reinterpret_cast<uintptr_t>(q) % 16) return CXXATTN_ERR_ALIGNMENT;
    if (rows > 0x7fffffffull * 8) return CXXATTN_ERR_TOO_LARGE;
    if (ws == nullptr || ws_bytes < layernorm_bwd_workspace(cols)) return CXXATTN_ERR_WORKSPACE;
    const size_t blocks = (cols + CB - 1) / CB, ws_cols = blocks * CB;
    float* sums = static_cast<float*>(ws);
    unsigned* counters = reinterpret_cast<unsigned*>(sums + 2 * ws_cols);
    if (dtype == CXXATTN_BF16)
        return launch<__nv_bfloat16>(dy, x, gamma, mean, rstd, dx, dgamma, dbeta, rows, cols, sums, counters, ws_cols, blocks, st);
    return launch<float>(dy, x, gamma, mean, rstd, dx, dgamma, dbeta, rows, cols, sums, counters, ws_cols, blocks, st);
}

}  // namespace cxxattn
