// Column sums of a row-major matrix: out[c] = sum_r X[r][c], the bias gradient of a linear layer
// (the reference's TensorN::cuda::sum_axis(dout, 0) in Linear::backward, src/GPT/gpt_gpt.hpp:111).
// HBM-bound and small (a few MB per call in the data-parallel step), so what matters is that one launch
// reads the matrix once with every SM: CTAs take a block of 64 columns x a group of rows, add their
// partial sums into an fp32 workspace with atomics, and the last CTA of a column block (a counter per
// block) converts the totals to the output type and puts the workspace back to zero for the next call.
#include "internal.cuh"
#include <algorithm>

namespace cxxattn {
namespace {

constexpr int CB = 64;  // columns per CTA

template <typename T>
struct Vec16;
template <>
struct Vec16<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void add(float (&acc)[4], const uint4 v) {
        acc[0] += __uint_as_float(v.x); acc[1] += __uint_as_float(v.y);
        acc[2] += __uint_as_float(v.z); acc[3] += __uint_as_float(v.w);
    }
    static __device__ __forceinline__ float out(float x) { return x; }
};
template <>
struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void add(float (&acc)[8], const uint4 v) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            acc[2 * i] += __uint_as_float(w[i] << 16);
            acc[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ __nv_bfloat16 out(float x) { return __float2bfloat16_rn(x); }
};

template <typename T>
__global__ void __launch_bounds__(256) colsum_kernel(const T* __restrict__ X, T* __restrict__ out, size_t rows, size_t cols,
                                                    size_t rows_per_group, float* ws, unsigned* counters) {
    constexpr int VEC = Vec16<T>::N, CT = CB / VEC, RL = 256 / CT;  // column threads, row lanes
    __shared__ float part[RL][CB + 1];
    __shared__ bool last;
    const int tx = threadIdx.x % CT, ty = threadIdx.x / CT;
    const size_t col = (size_t)blockIdx.x * CB + tx * VEC;
    const size_t r0 = (size_t)blockIdx.y * rows_per_group, r1 = min(rows, r0 + rows_per_group);
    float acc[VEC];
#pragma unroll
    for (int k = 0; k < VEC; k++) acc[k] = 0.f;
    if (col < cols) {
        size_t r = r0 + ty;
        for (; r + 3 * RL < r1; r += 4 * RL) {  // four rows in flight
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; u++) v[u] = *reinterpret_cast<const uint4*>(X + (r + u * RL) * cols + col);
#pragma unroll
            for (int u = 0; u < 4; u++) Vec16<T>::add(acc, v[u]);
        }
        for (; r < r1; r += RL) Vec16<T>::add(acc, *reinterpret_cast<const uint4*>(X + r * cols + col));
    }
#pragma unroll
    for (int k = 0; k < VEC; k++) part[ty][tx * VEC + k] = acc[k];
    __syncthreads();
    if (threadIdx.x < CB) {
        float s = 0.f;
#pragma unroll 8
        for (int j = 0; j < RL; j++) s += part[j][threadIdx.x];
        const size_t c = (size_t)blockIdx.x * CB + threadIdx.x;
        if (c < cols) atomicAdd(ws + c, s);
    }
    // the CTA that arrives last at this column block finishes it
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(counters + blockIdx.x, 1u) == gridDim.y - 1;
    __syncthreads();
    if (!last) return;
    __threadfence();
    if (threadIdx.x < CB) {
        const size_t c = (size_t)blockIdx.x * CB + threadIdx.x;
        if (c < cols) {
            out[c] = Vec16<T>::out(__ldcg(ws + c));
            ws[c] = 0.f;
        }
    }
    if (threadIdx.x == 0) counters[blockIdx.x] = 0u;
}

}  // namespace

size_t colsum_workspace(size_t cols) {
    const size_t blocks = (cols + CB - 1) / CB;
    return blocks * CB * sizeof(float) + blocks * sizeof(unsigned);
}

int colsum(const void* X, int dtype, void* out, size_t rows, size_t cols, void* ws, size_t ws_bytes, cudaStream_t st) {
    const size_t vec = dtype == CXXATTN_BF16 ? 8 : 4;
    if (cols % vec) return CXXATTN_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(X) % 16 || reinterpret_cast<uintptr_t>(ws) % 16) return CXXATTN_ERR_ALIGNMENT;
    if (ws == nullptr || ws_bytes < colsum_workspace(cols)) return CXXATTN_ERR_WORKSPACE;
    const size_t blocks = (cols + CB - 1) / CB;
    if (blocks > 0x7fffffffu) return CXXATTN_ERR_TOO_LARGE;
    // row groups: enough CTAs for a few per SM, at least 128 rows each
    const size_t want = std::max<size_t>(1, ((size_t)sm_count() * 4 + blocks - 1) / blocks);
    const size_t groups = std::max<size_t>(1, std::min<size_t>({want, (rows + 127) / 128, (size_t)65535}));
    const size_t per = (rows + groups - 1) / groups;
    float* sums = static_cast<float*>(ws);
    unsigned* counters = reinterpret_cast<unsigned*>(sums + blocks * CB);
    const dim3 grid((unsigned)blocks, (unsigned)((rows + per - 1) / per));
    if (dtype == CXXATTN_BF16)
        colsum_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(X), static_cast<__nv_bfloat16*>(out),
                                                          rows, cols, per, sums, counters);
    else
        colsum_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(X), static_cast<float*>(out), rows, cols, per,
                                                  sums, counters);
    return check_launch();
}

}  // namespace cxxattn
