// Token-by-token decoding with carried state, exact fp32.  The reference's generate() re-runs the
// whole context through both attention stages for every new token (two_stage_gpt.hpp:458-474);
// these two steps compute the same last row from what the earlier steps left behind:
//
//   linear stage  (ts.cu:889-976 row t; lin.cu:10-79 for the pre-mapped flavour)
//       z += phi(k);  S += phi(k) (x) v;  den = phi(q).z;  o = phi(q)^T S / (den + 1e-8)
//       state per unit: S[D][E] and z[D] in fp32.  HBM-bound: the state is read and written once,
//       2 * D * (E + 1) * 4 bytes per unit and step.
//   softmax stage (ts.cu:54-125 row t)
//       K[pos] = k, V[pos] = v;  o = softmax(scale * q.K[0..pos]) V[0..pos]
//       cache per batch item: K, V [capacity][H*Dh] in fp32.  HBM-bound: 2 * (pos+1) * Dh * 4
//       bytes per (batch, head) and step.  Few (batch, head) units are cut along the keys
//       (partial maxima, sums and outputs in the workspace, merged by a second small kernel).
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>

#include "internal.cuh"

namespace cxxattn {
namespace {

__device__ __forceinline__ float phi_f(float x) { return x > 0.f ? x + 1.f : expf(x); }

// z += phi(k) for every unit: the first of two launches when a unit's state is cut over several
// CTAs (they all need the updated z and must not race with its writer).
__global__ void lin_decode_z_kernel(const float* __restrict__ k, float* __restrict__ z, size_t n, int map) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) z[i] += map ? phi_f(k[i]) : k[i];
}

// One CTA of 256 threads per (unit, group of 32-column tiles): thread (ty, tx) walks rows
// d = ty, ty+8, ... of the tile that holds column e0 + tx, so a warp touches 128 contiguous bytes
// of S per row, and eight rows are in flight per thread.  With gridDim.y == 1 the CTA also owns
// z (Z_DONE = false); otherwise z was updated by lin_decode_z_kernel before.
template <bool Z_DONE>
__global__ void __launch_bounds__(256)
lin_decode_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                  float* __restrict__ S, float* __restrict__ z, float* __restrict__ o, float* __restrict__ den,
                  int D, int E, int map, int eps_in_den, int tiles_per_cta) {
    extern __shared__ float sm[];
    float* pq = sm;            // phi(q) [D]
    float* pk = sm + D;        // phi(k) [D]
    float* part = sm + 2 * D;  // [8][32] partial numerators of one column tile
    const int b = blockIdx.x, t = threadIdx.x, tx = t & 31, ty = t >> 5;
    const float* qb = q + (size_t)b * D;
    const float* kb = k + (size_t)b * D;
    float* zb = z + (size_t)b * D;
    float dpart = 0.f;
    for (int d = t; d < D; d += 256) {
        const float a = map ? phi_f(qb[d]) : qb[d], c = map ? phi_f(kb[d]) : kb[d];
        pq[d] = a;
        pk[d] = c;
        float zn = zb[d];
        if (!Z_DONE) {
            zn += c;
            zb[d] = zn;
        }
        dpart += a * zn;
    }
    for (int off = 16; off; off >>= 1) dpart += __shfl_xor_sync(0xffffffffu, dpart, off);
    __shared__ float dsum[8];
    if (tx == 0) dsum[ty] = dpart;
    __syncthreads();
    float dn = 0.f;
    for (int i = 0; i < 8; i++) dn += dsum[i];
    if (t == 0 && blockIdx.y == 0 && den != nullptr) den[b] = eps_in_den ? dn + 1e-8f : dn;
    const float inv = 1.0f / (dn + 1e-8f);
    float* Sb = S + (size_t)b * D * E;
    const float* vb = v + (size_t)b * E;
    const int e_begin = blockIdx.y * tiles_per_cta * 32;
    const int e_end = min(E, e_begin + tiles_per_cta * 32);
    for (int e0 = e_begin; e0 < e_end; e0 += 32) {
        const int e = e0 + tx;
        float acc = 0.f;
        if (e < E) {
            const float ve = vb[e];
            int d = ty;
            for (; d + 56 < D; d += 64) {  // eight independent rows per thread in flight
                float sv[8];
#pragma unroll
                for (int u = 0; u < 8; u++) sv[u] = Sb[(size_t)(d + 8 * u) * E + e];
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    sv[u] += pk[d + 8 * u] * ve;
                    Sb[(size_t)(d + 8 * u) * E + e] = sv[u];
                    acc += pq[d + 8 * u] * sv[u];
                }
            }
            for (; d < D; d += 8) {
                const float s = Sb[(size_t)d * E + e] + pk[d] * ve;
                Sb[(size_t)d * E + e] = s;
                acc += pq[d] * s;
            }
        }
        part[ty * 32 + tx] = acc;
        __syncthreads();
        if (ty == 0 && e < E) {
            float n = 0.f;
            for (int i = 0; i < 8; i++) n += part[i * 32 + tx];
            o[(size_t)b * E + e] = n * inv;
        }
        __syncthreads();
    }
}

// Softmax decoding, one CTA of 4 warps per (batch*head, key split).  A warp takes blocks of four
// consecutive keys of its split (eight rows of 4*NV*32 bytes in flight per warp); its lanes share
// the head dimension (NV values per lane, Dh <= 32*NV <= 256), the dot products are reduced with
// shuffles and the running maximum / sum / output are kept per warp, then merged over the 4
// warps.  With nsplit > 1 the CTA leaves (m, l, o[Dh]) in the workspace.
constexpr int DEC_WARPS = 4;
constexpr int DEC_KEYS = 4;  // keys per warp and iteration

struct DecParams {
    const float* q;
    const float* knew;
    const float* vnew;
    float* Kc;
    float* Vc;
    float* o;
    float* part;  // [B*H][nsplit][Dh + 2]
    int H, Dh, cap, pos, nsplit;
    float scale;
};

// NV floats of one row for this lane.  VEC (Dh == 32*NV): lane owns columns lane*NV .. lane*NV+NV-1
// and fetches them with one 4/8/16-byte load (two for NV = 8); otherwise columns lane + 32*i.
template <int NV, bool VEC>
__device__ __forceinline__ void load_row(const float* __restrict__ row, int lane, int Dh, bool live, float (&x)[NV]) {
    if constexpr (VEC) {
        if (!live) {
#pragma unroll
            for (int i = 0; i < NV; i++) x[i] = 0.f;
        } else if constexpr (NV == 1) {
            x[0] = row[lane];
        } else if constexpr (NV == 2) {
            const float2 v = reinterpret_cast<const float2*>(row)[lane];
            x[0] = v.x, x[1] = v.y;
        } else {
#pragma unroll
            for (int j = 0; j < NV / 4; j++) {
                const float4 v = reinterpret_cast<const float4*>(row)[lane * (NV / 4) + j];
                x[4 * j] = v.x, x[4 * j + 1] = v.y, x[4 * j + 2] = v.z, x[4 * j + 3] = v.w;
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < NV; i++) {
            const int d = lane + 32 * i;
            x[i] = live && d < Dh ? row[d] : 0.f;
        }
    }
}
template <int NV, bool VEC>
__device__ __forceinline__ int col_of(int lane, int i) {
    return VEC ? lane * NV + i : lane + 32 * i;
}

template <int NV, bool VEC>
__global__ void __launch_bounds__(DEC_WARPS * 32) mha_decode_kernel(DecParams p) {
    const int bh = blockIdx.x, split = blockIdx.y, b = bh / p.H, h = bh % p.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int HD = p.H * p.Dh;
    const size_t row0 = (size_t)b * p.cap * HD + (size_t)h * p.Dh;
    float* Krow = p.Kc + row0;
    float* Vrow = p.Vc + row0;
    const float* knew = p.knew + (size_t)b * HD + h * p.Dh;
    const float* vnew = p.vnew + (size_t)b * HD + h * p.Dh;
    // The new token's key and value are taken from k, v and appended to the cache by the one warp
    // whose turn key `pos` is; no other CTA reads that cache row in this step.
    const int nkeys = p.pos + 1;
    const int per = (nkeys + p.nsplit - 1) / p.nsplit;
    const int t0 = split * per, t1 = min(nkeys, t0 + per);
    float qv[NV], acc[NV];
    load_row<NV, VEC>(p.q + (size_t)b * HD + h * p.Dh, lane, p.Dh, true, qv);
#pragma unroll
    for (int i = 0; i < NV; i++) {
        qv[i] *= p.scale;
        acc[i] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    for (int tb = t0 + warp * DEC_KEYS; tb < t1; tb += DEC_WARPS * DEC_KEYS) {
        float kv[DEC_KEYS][NV], vv[DEC_KEYS][NV], s[DEC_KEYS];
#pragma unroll
        for (int u = 0; u < DEC_KEYS; u++) {
            const int t = tb + u;
            const bool fresh = t == p.pos;
            const float* kr = fresh ? knew : Krow + (size_t)t * HD;
            const float* vr = fresh ? vnew : Vrow + (size_t)t * HD;
            load_row<NV, VEC>(kr, lane, p.Dh, t < t1, kv[u]);
            load_row<NV, VEC>(vr, lane, p.Dh, t < t1, vv[u]);
        }
        if (tb <= p.pos && p.pos < tb + DEC_KEYS && p.pos < t1) {  // append the new token's rows to the cache
            const int u = p.pos - tb;
#pragma unroll
            for (int uu = 0; uu < DEC_KEYS; uu++) {
                if (uu != u) continue;
#pragma unroll
                for (int i = 0; i < NV; i++) {
                    const int d = col_of<NV, VEC>(lane, i);
                    if (d < p.Dh) {
                        Krow[(size_t)p.pos * HD + d] = kv[uu][i];
                        Vrow[(size_t)p.pos * HD + d] = vv[uu][i];
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < DEC_KEYS; u++) {
            float x = 0.f;
#pragma unroll
            for (int i = 0; i < NV; i++) x += qv[i] * kv[u][i];
            s[u] = x;
        }
#pragma unroll
        for (int off = 16; off; off >>= 1)
#pragma unroll
            for (int u = 0; u < DEC_KEYS; u++) s[u] += __shfl_xor_sync(0xffffffffu, s[u], off);
        float mn = m;
#pragma unroll
        for (int u = 0; u < DEC_KEYS; u++)
            if (tb + u < t1) mn = fmaxf(mn, s[u]);
        const float a = expf(m - mn);  // m = -inf on the first block: a = 0
        l *= a;
#pragma unroll
        for (int i = 0; i < NV; i++) acc[i] *= a;
#pragma unroll
        for (int u = 0; u < DEC_KEYS; u++) {
            const float e = tb + u < t1 ? expf(s[u] - mn) : 0.f;
            l += e;
#pragma unroll
            for (int i = 0; i < NV; i++) acc[i] += e * vv[u][i];
        }
        m = mn;
    }
    // merge the warps
    __shared__ float sm_m[DEC_WARPS], sm_l[DEC_WARPS], sm_o[DEC_WARPS][32 * NV];
    if (lane == 0) {
        sm_m[warp] = m;
        sm_l[warp] = l;
    }
#pragma unroll
    for (int i = 0; i < NV; i++) sm_o[warp][col_of<NV, VEC>(lane, i)] = acc[i];
    __syncthreads();
    float M = -INFINITY;
    for (int w = 0; w < DEC_WARPS; w++) M = fmaxf(M, sm_m[w]);
    float L = 0.f;
    for (int w = 0; w < DEC_WARPS; w++) L += sm_m[w] == -INFINITY ? 0.f : sm_l[w] * expf(sm_m[w] - M);
    for (int d = threadIdx.x; d < p.Dh; d += DEC_WARPS * 32) {
        float n = 0.f;
        for (int w = 0; w < DEC_WARPS; w++) n += sm_m[w] == -INFINITY ? 0.f : sm_o[w][d] * expf(sm_m[w] - M);
        if (p.nsplit == 1) p.o[(size_t)b * HD + h * p.Dh + d] = n / L;
        else p.part[((size_t)bh * p.nsplit + split) * (p.Dh + 2) + 2 + d] = n;
    }
    if (p.nsplit > 1 && threadIdx.x == 0) {
        float* pp = p.part + ((size_t)bh * p.nsplit + split) * (p.Dh + 2);
        pp[0] = M;  // -inf for an empty split
        pp[1] = L;
    }
}

__global__ void mha_decode_merge_kernel(DecParams p) {
    const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
    const float* base = p.part + (size_t)bh * p.nsplit * (p.Dh + 2);
    float M = -INFINITY;
    for (int s = 0; s < p.nsplit; s++) M = fmaxf(M, base[(size_t)s * (p.Dh + 2)]);
    float L = 0.f;
    for (int s = 0; s < p.nsplit; s++) {
        const float ms = base[(size_t)s * (p.Dh + 2)];
        if (ms != -INFINITY) L += base[(size_t)s * (p.Dh + 2) + 1] * expf(ms - M);
    }
    for (int d = threadIdx.x; d < p.Dh; d += blockDim.x) {
        float n = 0.f;
        for (int s = 0; s < p.nsplit; s++) {
            const float ms = base[(size_t)s * (p.Dh + 2)];
            if (ms != -INFINITY) n += base[(size_t)s * (p.Dh + 2) + 2 + d] * expf(ms - M);
        }
        p.o[(size_t)b * p.H * p.Dh + h * p.Dh + d] = n / L;
    }
}

}  // namespace

// The same step with 16-byte accesses, for E % 4 == 0: the CTA's columns [e_begin, e_end) are nq
// quads; thread (ty, tq) owns quad tq of rows d = ty, ty + R, ... (R = 256 / nq row lanes), four rows
// in flight, and the R partial numerators of a quad meet in shared memory.
template <bool Z_DONE>
__global__ void __launch_bounds__(256)
lin_decode_vec_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                      float* __restrict__ S, float* __restrict__ z, float* __restrict__ o, float* __restrict__ den,
                      int D, int E, int map, int eps_in_den, int cols_per_cta) {
    extern __shared__ float sm[];
    float* pq = sm;            // phi(q) [D]
    float* pk = sm + D;        // phi(k) [D]
    float* part = sm + 2 * D;  // [R][nq * 4] partial numerators (at most 256 * 4 floats)
    const int b = blockIdx.x, t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const float* qb = q + (size_t)b * D;
    const float* kb = k + (size_t)b * D;
    float* zb = z + (size_t)b * D;
    float dpart = 0.f;
    for (int d = t; d < D; d += 256) {
        const float a = map ? phi_f(qb[d]) : qb[d], c = map ? phi_f(kb[d]) : kb[d];
        pq[d] = a;
        pk[d] = c;
        float zn = zb[d];
        if (!Z_DONE) {
            zn += c;
            zb[d] = zn;
        }
        dpart += a * zn;
    }
    for (int off = 16; off; off >>= 1) dpart += __shfl_xor_sync(0xffffffffu, dpart, off);
    __shared__ float dsum[8];
    if (lane == 0) dsum[warp] = dpart;
    __syncthreads();
    float dn = 0.f;
    for (int i = 0; i < 8; i++) dn += dsum[i];
    if (t == 0 && blockIdx.y == 0 && den != nullptr) den[b] = eps_in_den ? dn + 1e-8f : dn;
    const float inv = 1.0f / (dn + 1e-8f);

    const int e_begin = blockIdx.y * cols_per_cta;
    const int e_end = min(E, e_begin + cols_per_cta);
    const int nq = (e_end - e_begin) / 4;  // <= 256
    const int R = 256 / nq;
    const int tq = t % nq, ty = t / nq;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (ty < R) {
        float4* Sq = reinterpret_cast<float4*>(S + (size_t)b * D * E + e_begin) + tq;  // row stride E/4 quads
        const size_t rs = (size_t)E / 4;
        const float4 ve = reinterpret_cast<const float4*>(v + (size_t)b * E + e_begin)[tq];
        int d = ty;
        for (; d + 3 * R < D; d += 4 * R) {
            float4 sv[4];
#pragma unroll
            for (int u = 0; u < 4; u++) sv[u] = Sq[(size_t)(d + u * R) * rs];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const float c = pk[d + u * R], a = pq[d + u * R];
                sv[u].x += c * ve.x, sv[u].y += c * ve.y, sv[u].z += c * ve.z, sv[u].w += c * ve.w;
                Sq[(size_t)(d + u * R) * rs] = sv[u];
                acc.x += a * sv[u].x, acc.y += a * sv[u].y, acc.z += a * sv[u].z, acc.w += a * sv[u].w;
            }
        }
        for (; d < D; d += R) {
            float4 x = Sq[(size_t)d * rs];
            const float c = pk[d], a = pq[d];
            x.x += c * ve.x, x.y += c * ve.y, x.z += c * ve.z, x.w += c * ve.w;
            Sq[(size_t)d * rs] = x;
            acc.x += a * x.x, acc.y += a * x.y, acc.z += a * x.z, acc.w += a * x.w;
        }
        reinterpret_cast<float4*>(part)[ty * nq + tq] = acc;
    }
    __syncthreads();
    for (int c = t; c < nq * 4; c += 256) {
        float n = 0.f;
        for (int r = 0; r < R; r++) n += part[r * nq * 4 + c];
        o[(size_t)b * E + e_begin + c] = n * inv;
    }
}

int linattn_decode_step(const cxxattn_lin_desc& d, const float* q, const float* k, const float* v, float* S, float* z,
                        float* o, float* den, cudaStream_t st) {
    const size_t smem = (2 * (size_t)d.D + 8 * 32) * sizeof(float);
    if (smem > 48 * 1024) return CXXATTN_ERR_TOO_LARGE;
    const int map = d.feature_map == CXXATTN_MAP_ELU1;
    // Column groups per unit: about four CTAs per SM when the units alone are fewer; a unit whose
    // state is a few KB stays in one CTA (one launch).
    const int64_t tiles = (d.E + 31) / 32;
    int64_t groups = (4 * 148 + d.B - 1) / d.B;
    if (groups > tiles) groups = tiles;
    if (d.D * d.E <= 64 * 64 || groups < 1) groups = 1;
    int per = (int)((tiles + groups - 1) / groups);
    // 16-byte accesses when the rows allow it; a CTA then takes at most 1024 columns (256 quads)
    const uintptr_t all = reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(S);
    const bool vec = d.E % 4 == 0 && all % 16 == 0;
    if (vec && per > 32) per = 32;
    groups = (tiles + per - 1) / per;
    const dim3 grid((unsigned)d.B, (unsigned)groups);
    if (groups > 1) {
        const size_t n = (size_t)d.B * d.D;
        lin_decode_z_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(k, z, n, map);
    }
    if (vec) {
        const size_t smem_v = (2 * (size_t)d.D + 256 * 4) * sizeof(float);
        if (smem_v > 48 * 1024) return CXXATTN_ERR_TOO_LARGE;
        if (groups == 1)
            lin_decode_vec_kernel<false><<<grid, 256, smem_v, st>>>(q, k, v, S, z, o, den, (int)d.D, (int)d.E, map,
                                                                  d.eps_in_den, per * 32);
        else
            lin_decode_vec_kernel<true><<<grid, 256, smem_v, st>>>(q, k, v, S, z, o, den, (int)d.D, (int)d.E, map,
                                                                 d.eps_in_den, per * 32);
    } else if (groups == 1) {
        lin_decode_kernel<false><<<grid, 256, smem, st>>>(q, k, v, S, z, o, den, (int)d.D, (int)d.E, map, d.eps_in_den, per);
    } else {
        lin_decode_kernel<true><<<grid, 256, smem, st>>>(q, k, v, S, z, o, den, (int)d.D, (int)d.E, map, d.eps_in_den, per);
    }
    return check_launch();
}

// Key splits: enough CTAs (of four warps) for about sixteen per SM, which is what keeps enough rows
// in flight to cover the DRAM latency; at least 256 keys per split.
int mha_decode_splits(int64_t BH, int64_t nkeys) {
    int64_t want = (16 * 148 + BH - 1) / BH, most = (nkeys + 255) / 256;
    int64_t n = want < most ? want : most;
    return (int)(n < 1 ? 1 : n > 64 ? 64 : n);
}

size_t mha_decode_workspace(const cxxattn_mha_desc& d) {
    // sized for the largest split count any position of this cache can ask for
    const int ns = mha_decode_splits(d.B * d.H, d.S);
    return ns > 1 ? (size_t)d.B * d.H * ns * (d.Dh + 2) * sizeof(float) : 0;
}

int mha_decode_step(const cxxattn_mha_desc& d, const float* q, const float* k, const float* v, float* Kc, float* Vc,
                    int64_t pos, float* o, void* ws, size_t ws_bytes, cudaStream_t st) {
    DecParams p;
    p.q = q, p.knew = k, p.vnew = v, p.Kc = Kc, p.Vc = Vc, p.o = o;
    p.H = (int)d.H, p.Dh = (int)d.Dh, p.cap = (int)d.S, p.pos = (int)pos;
    p.scale = 1.0f / sqrtf((float)d.Dh);
    p.nsplit = mha_decode_splits(d.B * d.H, pos + 1);
    p.part = static_cast<float*>(ws);
    if (p.nsplit > 1 && (!ws || ws_bytes < (size_t)d.B * d.H * p.nsplit * (d.Dh + 2) * sizeof(float)))
        return CXXATTN_ERR_WORKSPACE;
    const dim3 grid((unsigned)(d.B * d.H), (unsigned)p.nsplit);
    // vector loads: whole rows of 32*NV floats, and every tensor on a 16-byte boundary
    const uintptr_t all = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                          reinterpret_cast<uintptr_t>(Kc) | reinterpret_cast<uintptr_t>(Vc);
    const bool vec = (d.Dh == 32 || d.Dh == 64 || d.Dh == 128 || d.Dh == 256) && all % 16 == 0;
    if (vec) {
        if (d.Dh == 32) mha_decode_kernel<1, true><<<grid, DEC_WARPS * 32, 0, st>>>(p);
        else if (d.Dh == 64) mha_decode_kernel<2, true><<<grid, DEC_WARPS * 32, 0, st>>>(p);
        else if (d.Dh == 128) mha_decode_kernel<4, true><<<grid, DEC_WARPS * 32, 0, st>>>(p);
        else mha_decode_kernel<8, true><<<grid, DEC_WARPS * 32, 0, st>>>(p);
    } else if (d.Dh <= 32) mha_decode_kernel<1, false><<<grid, DEC_WARPS * 32, 0, st>>>(p);
    else if (d.Dh <= 64) mha_decode_kernel<2, false><<<grid, DEC_WARPS * 32, 0, st>>>(p);
    else if (d.Dh <= 128) mha_decode_kernel<4, false><<<grid, DEC_WARPS * 32, 0, st>>>(p);
    else mha_decode_kernel<8, false><<<grid, DEC_WARPS * 32, 0, st>>>(p);
    if (p.nsplit > 1) mha_decode_merge_kernel<<<(unsigned)(d.B * d.H), 64, 0, st>>>(p);
    return check_launch();
}

}  // namespace cxxattn
