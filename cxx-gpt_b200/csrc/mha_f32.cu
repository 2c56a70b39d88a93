// Exact fp32 causal softmax multi-head attention, forward and backward, on the CUDA cores.
//
// This is the validation-grade path behind cxxattn_mha_fwd / cxxattn_mha_bwd for dtype F32:
// fp32 operands, fp32 FMA accumulation, accurate expf/logf, no atomics (results are
// deterministic).  It computes what two_stage_cuda::fused_mha_fwd / fused_mha_bwd compute
// (reference: src/TwoStage/two_stage_cuda_kernels.cu:54-125, 334-491) but is organised the
// FlashAttention way: a CTA owns a tile of query rows (forward, dQ) or of key rows (dK/dV),
// streams the other side through shared memory in tiles, skips tiles above the causal
// diagonal, and keeps O(S) state (the row log-sum-exp) instead of the reference's S x S
// P/dP matrices.  Any S, any Dh <= 256 and any element strides are accepted.
//
// Thread layout: 256 threads as a 16 x 16 grid; thread (ty, tx) owns score rows
// ty*TM .. ty*TM+TM-1 and score columns tx, tx+16, ... of a BM x BN tile, and output columns
// tx, tx+16, ... of the Dh-wide accumulators.
#include "internal.cuh"

namespace cxxattn {
namespace {

constexpr int NT = 256;
constexpr int PAD = 4;  // floats added to every shared-memory row: keeps 16-byte alignment, staggers banks

template <int DHP, int BM_, int BN_>
struct Tile {
    static constexpr int BM = BM_, BN = BN_;
    static constexpr int LD = DHP + PAD;   // row pitch of a [rows][Dh] tile
    static constexpr int LDP = BN + PAD;   // row pitch of a [BM][BN] tile
    static constexpr int TM = BM / 16, TN = BN / 16, TD = DHP / 16;
};

// Copies rows [row0, row0+ROWS) x [0, Dh) of one (batch, head) slice into a [ROWS][LD] tile,
// zero-filling rows >= S and columns >= Dh.  `base` points at element (b, 0, h, 0).
template <int ROWS, int LD, int DHP>
__device__ __forceinline__ void load_tile(float* dst, const float* __restrict__ base, int64_t ss,
                                          int row0, int S, int Dh, bool vec) {
    if (vec) {
        constexpr int C4 = DHP / 4;
        for (int i = threadIdx.x; i < ROWS * C4; i += NT) {
            int r = i / C4, c = (i % C4) * 4, row = row0 + r;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (row < S && c < Dh) v = *reinterpret_cast<const float4*>(base + (int64_t)row * ss + c);
            *reinterpret_cast<float4*>(dst + r * LD + c) = v;
        }
    } else {
        for (int i = threadIdx.x; i < ROWS * DHP; i += NT) {
            int r = i / DHP, c = i % DHP, row = row0 + r;
            dst[r * LD + c] = (row < S && c < Dh) ? base[(int64_t)row * ss + c] : 0.f;
        }
    }
}

// acc[i][j] += sum_d A[(ty*TM+i)][d] * B[(tx+16j)][d]   (both tiles [rows][LD], d contiguous)
template <int TM, int TN, int LD, int DHP>
__device__ __forceinline__ void dot_nt(float (&acc)[TM][TN], const float* A, const float* B,
                                       int ty, int tx) {
#pragma unroll 4
    for (int d = 0; d < DHP; d += 4) {
        float4 a[TM], b[TN];
#pragma unroll
        for (int i = 0; i < TM; i++) a[i] = *reinterpret_cast<const float4*>(A + (ty * TM + i) * LD + d);
#pragma unroll
        for (int j = 0; j < TN; j++) b[j] = *reinterpret_cast<const float4*>(B + (tx + 16 * j) * LD + d);
#pragma unroll
        for (int i = 0; i < TM; i++)
#pragma unroll
            for (int j = 0; j < TN; j++) {
                acc[i][j] = fmaf(a[i].x, b[j].x, acc[i][j]);
                acc[i][j] = fmaf(a[i].y, b[j].y, acc[i][j]);
                acc[i][j] = fmaf(a[i].z, b[j].z, acc[i][j]);
                acc[i][j] = fmaf(a[i].w, b[j].w, acc[i][j]);
            }
    }
}

// acc[i][j] += sum_k P[(ty*TM+i)][k] * V[k][tx+16j]   (P is [BM][LDP], V is [BN][LD])
template <int TM, int TD, int BN, int LDP, int LD>
__device__ __forceinline__ void dot_nn(float (&acc)[TM][TD], const float* P, const float* V,
                                       int ty, int tx) {
#pragma unroll 2
    for (int k = 0; k < BN; k += 4) {
        float4 a[TM];
#pragma unroll
        for (int i = 0; i < TM; i++) a[i] = *reinterpret_cast<const float4*>(P + (ty * TM + i) * LDP + k);
#pragma unroll
        for (int kk = 0; kk < 4; kk++) {
            float v[TD];
#pragma unroll
            for (int j = 0; j < TD; j++) v[j] = V[(k + kk) * LD + tx + 16 * j];
#pragma unroll
            for (int i = 0; i < TM; i++) {
                float pv = kk == 0 ? a[i].x : kk == 1 ? a[i].y : kk == 2 ? a[i].z : a[i].w;
#pragma unroll
                for (int j = 0; j < TD; j++) acc[i][j] = fmaf(pv, v[j], acc[i][j]);
            }
        }
    }
}

__device__ __forceinline__ float half_warp_max(float v) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Forward.  One CTA per (batch, head, tile of BM query rows).  WRITE_O = false turns the kernel
// into the statistics pre-pass of the backward (lse only).
template <int DHP, int BM, int BN, bool WRITE_O>
__global__ void __launch_bounds__(NT) mha_fwd_kernel(MhaShape p, const float* __restrict__ Q,
                                                     const float* __restrict__ K,
                                                     const float* __restrict__ V, float* __restrict__ O,
                                                     float* __restrict__ lse, bool vec) {
    using T = Tile<DHP, BM, BN>;
    extern __shared__ __align__(16) float smem[];
    float* Qs = smem;
    float* Ks = Qs + BM * T::LD;
    float* Vs = Ks + BN * T::LD;
    float* Ps = Vs + BN * T::LD;

    const int nqt = (p.S + BM - 1) / BM;
    const int qt = nqt - 1 - (int)(blockIdx.x % nqt);  // longest rows are scheduled first
    const int bh = blockIdx.x / nqt;
    const int b = bh / p.H, h = bh % p.H;
    const int64_t off = (int64_t)b * p.sb + (int64_t)h * p.sh;
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
    const int q0 = qt * BM;

    load_tile<BM, T::LD, DHP>(Qs, Q + off, p.ss, q0, p.S, p.Dh, vec);

    float m[T::TM], l[T::TM], o[T::TM][T::TD];
#pragma unroll
    for (int i = 0; i < T::TM; i++) {
        m[i] = -1e30f;
        l[i] = 0.f;
#pragma unroll
        for (int j = 0; j < T::TD; j++) o[i][j] = 0.f;
    }

    const int kend = min(p.S, q0 + BM);
    for (int k0 = 0; k0 < kend; k0 += BN) {
        __syncthreads();
        load_tile<BN, T::LD, DHP>(Ks, K + off, p.ss, k0, p.S, p.Dh, vec);
        if (WRITE_O) load_tile<BN, T::LD, DHP>(Vs, V + off, p.ss, k0, p.S, p.Dh, vec);
        __syncthreads();

        float s[T::TM][T::TN];
#pragma unroll
        for (int i = 0; i < T::TM; i++)
#pragma unroll
            for (int j = 0; j < T::TN; j++) s[i][j] = 0.f;
        dot_nt<T::TM, T::TN, T::LD, DHP>(s, Qs, Ks, ty, tx);

#pragma unroll
        for (int i = 0; i < T::TM; i++) {
            const int qr = q0 + ty * T::TM + i;
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < T::TN; j++) {
                const int kc = k0 + tx + 16 * j;
                s[i][j] = (kc <= qr && kc < p.S) ? s[i][j] * p.scale : -INFINITY;
                mx = fmaxf(mx, s[i][j]);
            }
            mx = half_warp_max(mx);
            const float m_new = fmaxf(m[i], mx);
            const float alpha = expf(m[i] - m_new);
            float rs = 0.f;
#pragma unroll
            for (int j = 0; j < T::TN; j++) {
                const float pj = expf(s[i][j] - m_new);
                if (WRITE_O) Ps[(ty * T::TM + i) * T::LDP + tx + 16 * j] = pj;
                rs += pj;
            }
            rs = half_warp_sum(rs);
            l[i] = l[i] * alpha + rs;
            m[i] = m_new;
#pragma unroll
            for (int j = 0; j < T::TD; j++) o[i][j] *= alpha;
        }
        if (WRITE_O) {
            __syncthreads();
            dot_nn<T::TM, T::TD, BN, T::LDP, T::LD>(o, Ps, Vs, ty, tx);
        }
    }

#pragma unroll
    for (int i = 0; i < T::TM; i++) {
        const int qr = q0 + ty * T::TM + i;
        if (qr >= p.S) continue;
        if (WRITE_O) {
            const float inv = 1.f / l[i];
#pragma unroll
            for (int j = 0; j < T::TD; j++) {
                const int c = tx + 16 * j;
                if (c < p.Dh) O[off + (int64_t)qr * p.ss + c] = o[i][j] * inv;
            }
        }
        if (lse != nullptr && tx == 0) lse[(int64_t)bh * p.S + qr] = m[i] + logf(l[i]);
    }
}

// delta[b,h,s] = dO[b,s,h,:] . O[b,s,h,:]; one warp per row.
__global__ void mha_delta_kernel(MhaShape p, const float* __restrict__ O, const float* __restrict__ dO,
                                 float* __restrict__ delta) {
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    if (row >= (int64_t)p.B * p.H * p.S) return;
    const int s = row % p.S;
    const int bh = row / p.S;
    const int64_t off = (int64_t)(bh / p.H) * p.sb + (int64_t)(bh % p.H) * p.sh + (int64_t)s * p.ss;
    float acc = 0.f;
    for (int c = lane; c < p.Dh; c += 32) acc = fmaf(dO[off + c], O[off + c], acc);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) delta[row] = acc;
}

// Recomputes, for one BM x BN tile, P = exp(scale*QK^T - lse) and dS = P o (dO V^T - delta), and
// leaves them in shared memory ([BM][LDP] each; Ps may be null when only dS is wanted).
template <int DHP, int BM, int BN>
__device__ __forceinline__ void recompute_p_ds(const MhaShape& p, const float* Qs, const float* Ks,
                                               const float* Gs, const float* Vs, const float* Ls,
                                               const float* Dl, float* Ps, float* Ds, int q0, int k0,
                                               int ty, int tx) {
    using T = Tile<DHP, BM, BN>;
    float s[T::TM][T::TN], dp[T::TM][T::TN];
#pragma unroll
    for (int i = 0; i < T::TM; i++)
#pragma unroll
        for (int j = 0; j < T::TN; j++) s[i][j] = dp[i][j] = 0.f;
    dot_nt<T::TM, T::TN, T::LD, DHP>(s, Qs, Ks, ty, tx);
    dot_nt<T::TM, T::TN, T::LD, DHP>(dp, Gs, Vs, ty, tx);
#pragma unroll
    for (int i = 0; i < T::TM; i++) {
        const int r = ty * T::TM + i, qr = q0 + r;
        const float lr = Ls[r], dr = Dl[r];
#pragma unroll
        for (int j = 0; j < T::TN; j++) {
            const int c = tx + 16 * j, kc = k0 + c;
            const bool valid = kc <= qr && qr < p.S && kc < p.S;
            const float pij = valid ? expf(s[i][j] * p.scale - lr) : 0.f;
            if (Ps) Ps[r * T::LDP + c] = pij;
            Ds[r * T::LDP + c] = pij * (dp[i][j] - dr);
        }
    }
}

// dK, dV.  One CTA per (batch, head, tile of BN key rows); loops over the query tiles at or
// below the diagonal.  dV = P^T dO, dK = scale * dS^T Q.
template <int DHP, int BM, int BN>
__global__ void __launch_bounds__(NT) mha_bwd_dkdv_kernel(MhaShape p, const float* __restrict__ Q,
                                                          const float* __restrict__ K,
                                                          const float* __restrict__ V,
                                                          const float* __restrict__ dO,
                                                          const float* __restrict__ lse,
                                                          const float* __restrict__ delta,
                                                          float* __restrict__ dK, float* __restrict__ dV,
                                                          bool vec) {
    using T = Tile<DHP, BM, BN>;
    extern __shared__ __align__(16) float smem[];
    float* Ks = smem;
    float* Vs = Ks + BN * T::LD;
    float* Qs = Vs + BN * T::LD;
    float* Gs = Qs + BM * T::LD;
    float* Ps = Gs + BM * T::LD;
    float* Ds = Ps + BM * T::LDP;
    float* Ls = Ds + BM * T::LDP;
    float* Dl = Ls + BM;

    const int nkt = (p.S + BN - 1) / BN;
    const int kt = blockIdx.x % nkt;  // early key tiles see the most queries: scheduled first
    const int bh = blockIdx.x / nkt;
    const int b = bh / p.H, h = bh % p.H;
    const int64_t off = (int64_t)b * p.sb + (int64_t)h * p.sh;
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
    const int k0 = kt * BN;

    load_tile<BN, T::LD, DHP>(Ks, K + off, p.ss, k0, p.S, p.Dh, vec);
    load_tile<BN, T::LD, DHP>(Vs, V + off, p.ss, k0, p.S, p.Dh, vec);

    float dk[T::TN][T::TD], dv[T::TN][T::TD];
#pragma unroll
    for (int i = 0; i < T::TN; i++)
#pragma unroll
        for (int j = 0; j < T::TD; j++) dk[i][j] = dv[i][j] = 0.f;

    for (int q0 = (k0 / BM) * BM; q0 < p.S; q0 += BM) {
        __syncthreads();
        load_tile<BM, T::LD, DHP>(Qs, Q + off, p.ss, q0, p.S, p.Dh, vec);
        load_tile<BM, T::LD, DHP>(Gs, dO + off, p.ss, q0, p.S, p.Dh, vec);
        for (int r = threadIdx.x; r < BM; r += NT) {
            const bool ok = q0 + r < p.S;
            Ls[r] = ok ? lse[(int64_t)bh * p.S + q0 + r] : 0.f;
            Dl[r] = ok ? delta[(int64_t)bh * p.S + q0 + r] : 0.f;
        }
        __syncthreads();
        recompute_p_ds<DHP, BM, BN>(p, Qs, Ks, Gs, Vs, Ls, Dl, Ps, Ds, q0, k0, ty, tx);
        __syncthreads();
        // thread (ty, tx): key rows ty*TN+i, feature columns tx+16j
#pragma unroll 2
        for (int r = 0; r < BM; r++) {
            float pk[T::TN], dsk[T::TN], g[T::TD], q[T::TD];
#pragma unroll
            for (int i = 0; i < T::TN; i++) {
                pk[i] = Ps[r * T::LDP + ty * T::TN + i];
                dsk[i] = Ds[r * T::LDP + ty * T::TN + i];
            }
#pragma unroll
            for (int j = 0; j < T::TD; j++) {
                g[j] = Gs[r * T::LD + tx + 16 * j];
                q[j] = Qs[r * T::LD + tx + 16 * j];
            }
#pragma unroll
            for (int i = 0; i < T::TN; i++)
#pragma unroll
                for (int j = 0; j < T::TD; j++) {
                    dv[i][j] = fmaf(pk[i], g[j], dv[i][j]);
                    dk[i][j] = fmaf(dsk[i], q[j], dk[i][j]);
                }
        }
    }
#pragma unroll
    for (int i = 0; i < T::TN; i++) {
        const int kr = k0 + ty * T::TN + i;
        if (kr >= p.S) continue;
#pragma unroll
        for (int j = 0; j < T::TD; j++) {
            const int c = tx + 16 * j;
            if (c < p.Dh) {
                dK[off + (int64_t)kr * p.ss + c] = dk[i][j] * p.scale;
                dV[off + (int64_t)kr * p.ss + c] = dv[i][j];
            }
        }
    }
}

// dQ = scale * dS K.  One CTA per (batch, head, tile of BM query rows).
template <int DHP, int BM, int BN>
__global__ void __launch_bounds__(NT) mha_bwd_dq_kernel(MhaShape p, const float* __restrict__ Q,
                                                        const float* __restrict__ K,
                                                        const float* __restrict__ V,
                                                        const float* __restrict__ dO,
                                                        const float* __restrict__ lse,
                                                        const float* __restrict__ delta,
                                                        float* __restrict__ dQ, bool vec) {
    using T = Tile<DHP, BM, BN>;
    extern __shared__ __align__(16) float smem[];
    float* Qs = smem;
    float* Gs = Qs + BM * T::LD;
    float* Ks = Gs + BM * T::LD;
    float* Vs = Ks + BN * T::LD;
    float* Ds = Vs + BN * T::LD;
    float* Ls = Ds + BM * T::LDP;
    float* Dl = Ls + BM;

    const int nqt = (p.S + BM - 1) / BM;
    const int qt = nqt - 1 - (int)(blockIdx.x % nqt);
    const int bh = blockIdx.x / nqt;
    const int b = bh / p.H, h = bh % p.H;
    const int64_t off = (int64_t)b * p.sb + (int64_t)h * p.sh;
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
    const int q0 = qt * BM;

    load_tile<BM, T::LD, DHP>(Qs, Q + off, p.ss, q0, p.S, p.Dh, vec);
    load_tile<BM, T::LD, DHP>(Gs, dO + off, p.ss, q0, p.S, p.Dh, vec);
    for (int r = threadIdx.x; r < BM; r += NT) {
        const bool ok = q0 + r < p.S;
        Ls[r] = ok ? lse[(int64_t)bh * p.S + q0 + r] : 0.f;
        Dl[r] = ok ? delta[(int64_t)bh * p.S + q0 + r] : 0.f;
    }

    float dq[T::TM][T::TD];
#pragma unroll
    for (int i = 0; i < T::TM; i++)
#pragma unroll
        for (int j = 0; j < T::TD; j++) dq[i][j] = 0.f;

    const int kend = min(p.S, q0 + BM);
    for (int k0 = 0; k0 < kend; k0 += BN) {
        __syncthreads();
        load_tile<BN, T::LD, DHP>(Ks, K + off, p.ss, k0, p.S, p.Dh, vec);
        load_tile<BN, T::LD, DHP>(Vs, V + off, p.ss, k0, p.S, p.Dh, vec);
        __syncthreads();
        recompute_p_ds<DHP, BM, BN>(p, Qs, Ks, Gs, Vs, Ls, Dl, nullptr, Ds, q0, k0, ty, tx);
        __syncthreads();
        dot_nn<T::TM, T::TD, BN, T::LDP, T::LD>(dq, Ds, Ks, ty, tx);
    }
#pragma unroll
    for (int i = 0; i < T::TM; i++) {
        const int qr = q0 + ty * T::TM + i;
        if (qr >= p.S) continue;
#pragma unroll
        for (int j = 0; j < T::TD; j++) {
            const int c = tx + 16 * j;
            if (c < p.Dh) dQ[off + (int64_t)qr * p.ss + c] = dq[i][j] * p.scale;
        }
    }
}

bool vec_ok(const MhaShape& p, std::initializer_list<const void*> ptrs) {
    if (p.Dh % 4 || p.sb % 4 || p.ss % 4 || p.sh % 4) return false;
    for (const void* q : ptrs)
        if (reinterpret_cast<uintptr_t>(q) % 16) return false;
    return true;
}

template <int DHP, int BM, int BN, bool WRITE_O>
int launch_fwd(const MhaShape& p, const float* Q, const float* K, const float* V, float* O,
               float* lse, cudaStream_t st) {
    using T = Tile<DHP, BM, BN>;
    const size_t smem = sizeof(float) * ((BM + 2 * BN) * T::LD + BM * T::LDP);
    auto kern = mha_fwd_kernel<DHP, BM, BN, WRITE_O>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return CXXATTN_ERR_CUDA;
    const int64_t grid = (int64_t)((p.S + BM - 1) / BM) * p.B * p.H;
    kern<<<(unsigned)grid, NT, smem, st>>>(p, Q, K, V, O, lse, WRITE_O ? vec_ok(p, {Q, K, V}) : vec_ok(p, {Q, K}));
    return check_launch();
}

template <int DHP, int BM, int BN>
int launch_bwd(const MhaShape& p, const float* Q, const float* K, const float* V, const float* dO,
               const float* lse, const float* delta, float* dQ, float* dK, float* dV, cudaStream_t st) {
    using T = Tile<DHP, BM, BN>;
    const bool vec = vec_ok(p, {Q, K, V, dO});
    {
        const size_t smem = sizeof(float) * ((2 * BN + 2 * BM) * T::LD + 2 * BM * T::LDP + 2 * BM);
        auto kern = mha_bwd_dkdv_kernel<DHP, BM, BN>;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return CXXATTN_ERR_CUDA;
        const int64_t grid = (int64_t)((p.S + BN - 1) / BN) * p.B * p.H;
        kern<<<(unsigned)grid, NT, smem, st>>>(p, Q, K, V, dO, lse, delta, dK, dV, vec);
        if (check_launch() != CXXATTN_OK) return CXXATTN_ERR_CUDA;
    }
    {
        const size_t smem = sizeof(float) * ((2 * BN + 2 * BM) * T::LD + BM * T::LDP + 2 * BM);
        auto kern = mha_bwd_dq_kernel<DHP, BM, BN>;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return CXXATTN_ERR_CUDA;
        const int64_t grid = (int64_t)((p.S + BM - 1) / BM) * p.B * p.H;
        kern<<<(unsigned)grid, NT, smem, st>>>(p, Q, K, V, dO, lse, delta, dQ, vec);
    }
    return check_launch();
}

template <bool WRITE_O>
int dispatch_fwd(const MhaShape& p, const float* Q, const float* K, const float* V, float* O,
                 float* lse, cudaStream_t st) {
    if (p.Dh <= 32) return launch_fwd<32, 64, 64, WRITE_O>(p, Q, K, V, O, lse, st);
    if (p.Dh <= 64) return launch_fwd<64, 64, 64, WRITE_O>(p, Q, K, V, O, lse, st);
    if (p.Dh <= 128) return launch_fwd<128, 64, 64, WRITE_O>(p, Q, K, V, O, lse, st);
    if (p.Dh <= 256) return launch_fwd<256, 32, 32, WRITE_O>(p, Q, K, V, O, lse, st);
    return CXXATTN_ERR_UNSUPPORTED;  // the reference rejects Dh > 256 as well (ts.cu:316-321)
}

}  // namespace

int mha_f32_fwd(const MhaShape& p, const float* Q, const float* K, const float* V, float* O,
                float* lse, cudaStream_t st) {
    return dispatch_fwd<true>(p, Q, K, V, O, lse, st);
}

size_t mha_f32_bwd_workspace(const MhaShape& p, bool have_lse) {
    const size_t rows = align_up((size_t)p.B * p.H * p.S * sizeof(float), 256);
    return have_lse ? rows : 2 * rows;
}

int mha_f32_bwd(const MhaShape& p, const float* Q, const float* K, const float* V, const float* O,
                const float* dO, const float* lse, float* dQ, float* dK, float* dV,
                void* ws, size_t ws_bytes, cudaStream_t st) {
    if (p.Dh > 256) return CXXATTN_ERR_UNSUPPORTED;
    if (ws == nullptr || ws_bytes < mha_f32_bwd_workspace(p, lse != nullptr)) return CXXATTN_ERR_WORKSPACE;
    const size_t rows = align_up((size_t)p.B * p.H * p.S * sizeof(float), 256);
    float* delta = static_cast<float*>(ws);
    if (lse == nullptr) {
        float* my_lse = reinterpret_cast<float*>(static_cast<char*>(ws) + rows);
        int rc = dispatch_fwd<false>(p, Q, K, nullptr, nullptr, my_lse, st);
        if (rc != CXXATTN_OK) return rc;
        lse = my_lse;
    }
    const int64_t nrows = (int64_t)p.B * p.H * p.S;
    mha_delta_kernel<<<(unsigned)((nrows + 7) / 8), 256, 0, st>>>(p, O, dO, delta);
    if (check_launch() != CXXATTN_OK) return CXXATTN_ERR_CUDA;
    if (p.Dh <= 32) return launch_bwd<32, 64, 64>(p, Q, K, V, dO, lse, delta, dQ, dK, dV, st);
    if (p.Dh <= 64) return launch_bwd<64, 64, 64>(p, Q, K, V, dO, lse, delta, dQ, dK, dV, st);
    if (p.Dh <= 128) return launch_bwd<128, 64, 64>(p, Q, K, V, dO, lse, delta, dQ, dK, dV, st);
    return launch_bwd<256, 32, 32>(p, Q, K, V, dO, lse, delta, dQ, dK, dV, st);
}

}  // namespace cxxattn
