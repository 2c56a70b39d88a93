// Elementwise neighbours of the attention kernels that share the reference's kernel headers:
// step 1 of the linear-attention backward, the ELU+1 feature map of LinearGPT, rotary embedding
// and erf-GELU.  All are HBM-bound single-pass kernels: one warp per row for the row-wise ones,
// grid-stride for the flat ones.
#include "internal.cuh"

namespace cxxattn {
namespace {

// dnum = dO / den, dden = -(dO . O) / den  (ts.cu:1190-1219, lin.cu:101-134).  One warp per row.
__global__ void step1_kernel(const float* __restrict__ O, const float* __restrict__ dO,
                             const float* __restrict__ den, float* __restrict__ dnum,
                             float* __restrict__ dden, size_t N, size_t E) {
    const size_t row = (size_t)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    if (row >= N) return;
    const float inv = 1.0f / den[row];
    float sum = 0.f;
    for (size_t e = lane; e < E; e += 32) {
        const float g = dO[row * E + e];
        dnum[row * E + e] = g * inv;
        sum = fmaf(g, O[row * E + e], sum);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) dden[row] = -sum * inv;
}

// phi[n,d] = ELU(x[n,d]) + 1 for d < E, 0 for E <= d < D  (lin.cu:305-325).
__global__ void phi_fwd_kernel(const float* __restrict__ x, float* __restrict__ phi, size_t total,
                               size_t D, size_t E) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t n = i / D, d = i % D;
        float v = 0.f;
        if (d < E) {
            const float xv = x[n * E + d];
            v = (xv > 0.f ? xv : expf(xv) - 1.0f) + 1.0f;
        }
        phi[i] = v;
    }
}

// dx[n,e] = dphi[n,e] * (x > 0 ? 1 : exp(x))  (lin.cu:347-364); dphi has D columns, x and dx have E.
__global__ void phi_bwd_kernel(const float* __restrict__ dphi, const float* __restrict__ x,
                               float* __restrict__ dx, size_t total, size_t D, size_t E) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t n = i / E, e = i % E;
        const float xv = x[i];
        dx[i] = dphi[n * D + e] * (xv > 0.f ? 1.0f : expf(xv));
    }
}

// Rotary embedding, in place, one thread per (row, pair)  (ts.cu:1820-1857).  The frequency is
// 10000^(-2i/head_dim) and the position is row % S.  Q and K are rotated one after the other by
// the same thread, so passing the same pointer twice rotates twice, as in the reference.
__global__ void rope_kernel(float* Q, float* K, size_t total, size_t S, size_t D, size_t hd, float sign) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t npairs = D / 2, pph = hd / 2;
    const size_t row = idx / npairs, pair = idx % npairs, i = pair % pph;
    const size_t off = row * D + (pair / pph) * hd + 2 * i;
    const float ang = sign * (float)(row % S) * expf(-2.0f * (float)i / (float)hd * 9.210340371976184f);
    float s, c;
    sincosf(ang, &s, &c);
    if (Q) {
        const float x0 = Q[off], x1 = Q[off + 1];
        Q[off] = x0 * c - x1 * s;
        Q[off + 1] = x0 * s + x1 * c;
    }
    if (K) {
        const float x0 = K[off], x1 = K[off + 1];
        K[off] = x0 * c - x1 * s;
        K[off + 1] = x0 * s + x1 * c;
    }
}

// erf-GELU and its derivative  (ts.cu:1888-1915).
__global__ void gelu_kernel(const float* __restrict__ A, float* __restrict__ C, size_t n, int deriv) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x) {
        const float x = A[i];
        const float cdf = 0.5f * (1.0f + erff(x * 0.7071067811865476f));
        C[i] = deriv ? cdf + x * expf(-0.5f * x * x) * 0.3989422804014327f : x * cdf;
    }
}

inline unsigned flat_grid(size_t n) {
    const size_t blocks = (n + 255) / 256;
    return (unsigned)(blocks < 148 * 16 ? (blocks ? blocks : 1) : 148 * 16);  // 148 SMs x 16 resident CTAs
}

}  // namespace

int step1_f32(const float* O, const float* dO, const float* den, float* dnum, float* dden,
              size_t N, size_t E, cudaStream_t st) {
    step1_kernel<<<(unsigned)((N + 7) / 8), 256, 0, st>>>(O, dO, den, dnum, dden, N, E);
    return check_launch();
}

int phi_elu_fwd(const float* x, float* phi, size_t N, size_t D, size_t E, cudaStream_t st) {
    phi_fwd_kernel<<<flat_grid(N * D), 256, 0, st>>>(x, phi, N * D, D, E);
    return check_launch();
}

int phi_elu_bwd(const float* dphi, const float* x, float* dx, size_t N, size_t D, size_t E, cudaStream_t st) {
    phi_bwd_kernel<<<flat_grid(N * E), 256, 0, st>>>(dphi, x, dx, N * E, D, E);
    return check_launch();
}

int rope(float* Q, float* K, size_t B, size_t S, size_t D, size_t hd, float sign, cudaStream_t st) {
    const size_t total = B * S * (D / 2);
    rope_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(Q, K, total, S, D, hd, sign);
    return check_launch();
}

// fp32 <-> bf16, four elements per thread where the count allows
__global__ void cast_f32_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n / 4; i += stride) {
        const float4 v = reinterpret_cast<const float4*>(src)[i];
        __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        reinterpret_cast<uint2*>(dst)[i] = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
    for (size_t i = n / 4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        dst[i] = __float2bfloat16_rn(src[i]);
}
__global__ void cast_bf16_f32_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n / 4; i += stride) {
        const uint2 v = reinterpret_cast<const uint2*>(src)[i];
        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
        const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
        reinterpret_cast<float4*>(dst)[i] = make_float4(lo.x, lo.y, hi.x, hi.y);
    }
    for (size_t i = n / 4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        dst[i] = __bfloat162float(src[i]);
}

int cast(const void* src, int src_dtype, void* dst, int dst_dtype, size_t n, cudaStream_t st) {
    if (reinterpret_cast<uintptr_t>(src) % 16 || reinterpret_cast<uintptr_t>(dst) % 16) return CXXATTN_ERR_ALIGNMENT;
    if (src_dtype == CXXATTN_F32 && dst_dtype == CXXATTN_BF16)
        cast_f32_bf16_kernel<<<flat_grid(n / 4 + 1), 256, 0, st>>>(static_cast<const float*>(src),
                                                                  static_cast<__nv_bfloat16*>(dst), n);
    else if (src_dtype == CXXATTN_BF16 && dst_dtype == CXXATTN_F32)
        cast_bf16_f32_kernel<<<flat_grid(n / 4 + 1), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(src),
                                                                  static_cast<float*>(dst), n);
    else
        return CXXATTN_ERR_UNSUPPORTED;
    return check_launch();
}

// Rotary embedding out of place with a type conversion in the same pass: dst = rope(src), where
// src and dst are fp32 or bf16.  This replaces "rotate fp32 in place, then convert" (three passes
// over the tensor) by one read and one write when fp32 activations feed the bf16 tensor-core
// kernels, and the reverse (bf16 gradients -> inverse rotation -> fp32) on the way back.  The
// angle depends on the position and the pair only, so one thread owns four columns of one
// position, forms its two sine/cosine pairs once and walks over the batch.  Same angle formula
// as rope_kernel (ts.cu:1820-1857).
template <typename TI, typename TO>
__global__ void rope_cast_kernel(const TI* __restrict__ src0, TO* __restrict__ dst0, const TI* __restrict__ src1,
                                 TO* __restrict__ dst1, size_t B, size_t S, size_t D, size_t hd, float sign) {
    // blockIdx.y picks the tensor: the reference rotates Q and K in one call, and so can this
    const TI* __restrict__ src = blockIdx.y ? src1 : src0;
    TO* __restrict__ dst = blockIdx.y ? dst1 : dst0;
    const size_t qpr = D / 4;  // quads per row
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= S * qpr) return;
    const size_t pos = idx / qpr, col = (idx % qpr) * 4;
    const size_t i0 = (col % hd) / 2;  // first pair index inside its head (hd % 4 == 0: i0 + 1 is in it too)
    float s0, c0, s1, c1;
    sincosf(sign * (float)pos * expf(-2.0f * (float)i0 / (float)hd * 9.210340371976184f), &s0, &c0);
    sincosf(sign * (float)pos * expf(-2.0f * (float)(i0 + 1) / (float)hd * 9.210340371976184f), &s1, &c1);
#pragma unroll 4  // the batch items of a position are independent: their loads go out together
    for (size_t b = 0; b < B; b++) {
        const size_t off = (b * S + pos) * D + col;
        float x0, x1, x2, x3;
        if constexpr (sizeof(TI) == 4) {
            const float4 v = *reinterpret_cast<const float4*>(src + off);
            x0 = v.x, x1 = v.y, x2 = v.z, x3 = v.w;
        } else {
            const uint2 v = *reinterpret_cast<const uint2*>(src + off);
            const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
            const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
            x0 = lo.x, x1 = lo.y, x2 = hi.x, x3 = hi.y;
        }
        const float y0 = x0 * c0 - x1 * s0, y1 = x0 * s0 + x1 * c0;
        const float y2 = x2 * c1 - x3 * s1, y3 = x2 * s1 + x3 * c1;
        if constexpr (sizeof(TO) == 4) {
            *reinterpret_cast<float4*>(dst + off) = make_float4(y0, y1, y2, y3);
        } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(y0, y1), hi = __floats2bfloat162_rn(y2, y3);
            *reinterpret_cast<uint2*>(dst + off) =
                make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        }
    }
}

int rope_cast_pair(const void* src0, const void* src1, int src_dtype, void* dst0, void* dst1, int dst_dtype, size_t B,
                   size_t S, size_t D, size_t hd, float sign, cudaStream_t st) {
    for (const void* q : {src0, src1, (const void*)dst0, (const void*)dst1})
        if (reinterpret_cast<uintptr_t>(q) % 16) return CXXATTN_ERR_ALIGNMENT;
    const size_t threads = S * (D / 4);
    const dim3 grid((unsigned)((threads + 255) / 256), src1 != nullptr ? 2u : 1u);
    const bool si = src_dtype == CXXATTN_F32, so = dst_dtype == CXXATTN_F32;
    if ((!si && src_dtype != CXXATTN_BF16) || (!so && dst_dtype != CXXATTN_BF16)) return CXXATTN_ERR_UNSUPPORTED;
    if (si && so)
        rope_cast_kernel<float, float><<<grid, 256, 0, st>>>(static_cast<const float*>(src0), static_cast<float*>(dst0),
                                                            static_cast<const float*>(src1), static_cast<float*>(dst1),
                                                            B, S, D, hd, sign);
    else if (si)
        rope_cast_kernel<float, __nv_bfloat16><<<grid, 256, 0, st>>>(
            static_cast<const float*>(src0), static_cast<__nv_bfloat16*>(dst0), static_cast<const float*>(src1),
            static_cast<__nv_bfloat16*>(dst1), B, S, D, hd, sign);
    else if (so)
        rope_cast_kernel<__nv_bfloat16, float><<<grid, 256, 0, st>>>(
            static_cast<const __nv_bfloat16*>(src0), static_cast<float*>(dst0), static_cast<const __nv_bfloat16*>(src1),
            static_cast<float*>(dst1), B, S, D, hd, sign);
    else
        rope_cast_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, st>>>(
            static_cast<const __nv_bfloat16*>(src0), static_cast<__nv_bfloat16*>(dst0),
            static_cast<const __nv_bfloat16*>(src1), static_cast<__nv_bfloat16*>(dst1), B, S, D, hd, sign);
    return check_launch();
}

int rope_cast(const void* src, int src_dtype, void* dst, int dst_dtype, size_t B, size_t S, size_t D, size_t hd,
              float sign, cudaStream_t st) {
    return rope_cast_pair(src, nullptr, src_dtype, dst, nullptr, dst_dtype, B, S, D, hd, sign, st);
}

int gelu_exact(const float* A, float* C, size_t n, int deriv, cudaStream_t st) {
    gelu_kernel<<<flat_grid(n), 256, 0, st>>>(A, C, n, deriv);
    return check_launch();
}

}  // namespace cxxattn
