// Causal linear attention with ONE wide head on the tensor cores (tcgen05 + TMEM + TMA), bf16 operands,
// fp32 accumulation: the shapes the models call.  TwoStageGPT's second stage is a single head of
// width n_embd (two_stage_gpt.hpp:113-122: kernel_attn_fwd(..., B, S, E, E)), LinearGPT uses
// D = next_pow2(n_embd), E = n_embd (linear_gpt.hpp:103-112, 232), and both train on sequences of at
// most block_size = 256 tokens.  For such shapes (S of the order of D or below) the scan's state
// products, 4*S*D*E flops per unit, cost more than the masked quadratic form
//     num = ((phiQ phiK^T) o M) V,   den = ((phiQ phiK^T) o M) 1,   O = num / (den + eps)
// with its 2*S^2*(D+E)/2, so this file evaluates the quadratic form and keeps no state at all.  The
// reference walks the tokens one by one with a D x E state in global memory
// (src/TwoStage/two_stage_cuda_kernels.cu:889-976, src/LinearAttention/linear_cuda_kernels.cu:10-79).
//
// Forward and the three gradients are the same computation with the operands exchanged:
//     X_r[128 x G] = sum over partner tiles t of  mask( L_r R_t^T (+ rank-one term) ) Z_t[:, G]
//   mode   rows      L      R      K-loop   rank-one     Z      partners   result
//   FWD    queries   phiQ   phiK   D        -            V      t <= r     O (scaled by 1/(den+eps)), den = row sums
//   DQ     queries   dnum   V      E        dden[row]    phiK   t <= r     dphiQ
//   DV     keys      phiK   phiQ   D        -            dnum   t >= r     dV
//   DK     keys      V      dnum   E        dden[col]    phiQ   t >= r     dphiK
// (dnum = dO/den, dden = -(dO.O)/den: step 1 of the reference backward, ts.cu:1190-1219.)  One kernel
// template covers the four.  A CTA owns one tile of 128 rows of one batch unit and one group of up to
// 256 result columns; per partner tile it forms the 128 x 128 product in TMEM with a K-loop over 64-wide
// blocks streamed by TMA (SS MMA, both operands K-major), its four compute warps (thread = row = TMEM
// lane) add the rank-one term, mask the diagonal tile, sum rows (FWD) and write the tile back to TMEM
// as bf16, and a TS MMA multiplies it with the partner's Z blocks into the result accumulator.
// The feature map (ELU+1) and its derivative are applied by small element-wise passes either side
// (phi of Q and K into bf16 copies; dQ = dphiQ o phi'(Q)), so the kernel itself is map-agnostic, as
// the reference's linear_cuda kernels are.
#include <algorithm>

#include "internal.cuh"
#include "tc_common.cuh"

namespace cxxattn {
namespace {

using namespace tc;

constexpr int BT = 128;                  // rows per tile
constexpr int KB = 64;                   // K-loop block = one 128-byte TMA row
constexpr int TILE_BYTES = BT * KB * 2;  // 16 KB
constexpr int NST = 5;                   // ring stages of two tiles each
constexpr int GW = 256;                  // result columns per CTA
constexpr int NTHREADS = 192;            // warps 0-3 compute, 4 TMA producer, 5 MMA issuer
constexpr int W_PROD = 4, W_MMA = 5;
constexpr uint32_t TMEM_COLS = 512, COL_ACC = 0, COL_P = 128, COL_OUT = 192;  // 128 + 64 + 256
constexpr size_t SMEM_BYTES = (size_t)NST * 2 * TILE_BYTES + 1024;

enum { FWD = 0, DQ = 1, DV = 2, DK = 3 };

struct WideParams {
    __nv_bfloat16* out;  // [B*S, WO]
    float* den;          // FWD: row sums out
    const float* dden;   // DQ: per row, DK: per column
    int* status;
    int B, S, WL, WO;    // WL = width of L and R (the K-loop), WO = width of Z and of the result
    int ldo;             // row stride of the result (>= WO)
    int eps_in_den;
};

template <int MODE>
__global__ void __launch_bounds__(NTHREADS, 1)
linattn_wide_kernel(const __grid_constant__ CUtensorMap tmL, const __grid_constant__ CUtensorMap tmR,
                    const __grid_constant__ CUtensorMap tmZ, WideParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full[NST], empty[NST], acc_full, acc_free, p_full, p_free, out_full;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    constexpr bool LOWER = MODE == FWD || MODE == DQ;  // partners at or before the row tile
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int ntile = (p.S + BT - 1) / BT;
    const int ngroup = (p.WO + GW - 1) / GW;
    const int g = blockIdx.x % ngroup;
    const int r = (blockIdx.x / ngroup) % ntile;
    const int b = blockIdx.x / (ngroup * ntile);
    const int nw = p.WL / KB;                                    // K-loop blocks
    const int ncb = min(GW, p.WO - g * GW) / KB;                 // result column blocks of this CTA
    const int t0 = LOWER ? 0 : r, t1 = LOWER ? r : ntile - 1;    // partner tiles t0 .. t1
    const Guard guard{&abort_flag, p.status};

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < NST; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(&acc_full, 1);
        mbar_init(&acc_free, 4);  // one arrival per compute warp
        mbar_init(&p_full, 4);
        mbar_init(&p_free, 1);
        mbar_init(&out_full, 1);
        fence_barrier_init();
    }
    if (warp == W_MMA) tmem_alloc(&tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;

    if (warp == W_PROD) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            prefetch_tmap(&tmL);
            prefetch_tmap(&tmR);
            prefetch_tmap(&tmZ);
            int n = 0;  // stages filled so far
            auto stage = [&](uint32_t bytes) {
                const int s = n % NST;
                if (n >= NST) mbar_wait(&empty[s], ((n / NST) - 1) & 1, guard, 801);
                mbar_expect_tx(&full[s], bytes);
                n++;
                return s;
            };
            for (int t = t0; t <= t1; t++) {
                for (int wb = 0; wb < nw; wb++) {  // operands of the 128 x 128 product, one K block at a time
                    const int s = stage(2 * TILE_BYTES);
                    tma_load_4d(smem + s * 2 * TILE_BYTES, &tmL, &full[s], 0, wb, r * BT, b);
                    tma_load_4d(smem + s * 2 * TILE_BYTES + TILE_BYTES, &tmR, &full[s], 0, wb, t * BT, b);
                }
                for (int zb = 0; zb < ncb; zb += 2) {  // the partner's Z blocks, two per stage
                    const int nb = min(2, ncb - zb);
                    const int s = stage(nb * TILE_BYTES);
                    for (int i = 0; i < nb; i++)
                        tma_load_4d(smem + s * 2 * TILE_BYTES + i * TILE_BYTES, &tmZ, &full[s], 0, g * (GW / KB) + zb + i,
                                    t * BT, b);
                }
            }
        }
    } else if (warp == W_MMA) {
        // ---------------- MMA issuer ----------------
        // the whole warp runs the loop (uniform control flow and operands); one elected lane issues
        const uint32_t el = elect_one();
        constexpr uint32_t IDESC_A = idesc_bf16(BT, BT, 0, 0);  // L, R both K-major
        constexpr uint32_t IDESC_O = idesc_bf16(BT, KB, 0, 1);  // tile from TMEM, Z MN-major
        const uint64_t d0 = smem_desc_sw128(smem_u32(smem), 16);  // stage 0, first tile (K-major form)
        const uint64_t z0 = smem_desc_sw128(smem_u32(smem), 0);   // the same bits; read as an MN-major operand
        constexpr uint64_t TILE16 = TILE_BYTES >> 4;
        int n = 0;
        for (int t = t0, ti = 0; t <= t1; t++, ti++) {
            // the compute warps have read the product of the tile before out of TMEM
            if (ti > 0) mbar_wait_poll(&acc_free, (ti - 1) & 1, guard, 811);
            for (int wb = 0; wb < nw; wb++, n++) {
                const int s = n % NST;
                mbar_wait_poll(&full[s], (n / NST) & 1, guard, 812);
                tc_fence_after();
                const uint64_t l = d0 + s * 2 * TILE16, rr = l + TILE16;
#pragma unroll
                for (int kk = 0; kk < KB / 16; kk++)
                    umma_ss_e(el, tmem + COL_ACC, l + 2 * kk, rr + 2 * kk, IDESC_A, wb > 0 || kk > 0);
                umma_commit_e(el, &empty[s]);
            }
            umma_commit_e(el, &acc_full);
            mbar_wait_poll(&p_full, ti & 1, guard, 813);
            tc_fence_after();
            for (int zb = 0; zb < ncb; zb += 2, n++) {
                const int s = n % NST;
                mbar_wait_poll(&full[s], (n / NST) & 1, guard, 814);
                tc_fence_after();
                const int nb = min(2, ncb - zb);
                for (int i = 0; i < nb; i++) {
                    const uint64_t z = z0 + (s * 2 + i) * TILE16;
                    const uint32_t d = tmem + COL_OUT + (zb + i) * KB;
#pragma unroll
                    for (int kk = 0; kk < BT / 16; kk++)
                        umma_ts_e(el, d, tmem + COL_P + 8 * kk, z + 128 * kk, IDESC_O, ti > 0 || kk > 0);
                }
                umma_commit_e(el, &empty[s]);
            }
            umma_commit_e(el, &p_free);  // the bf16 tile has been read by every product of this partner
        }
        umma_commit_e(el, &out_full);
    } else {
        // ---------------- compute warps ----------------
        const int row = warp * 32 + lane;   // row inside the tile == TMEM lane
        const int grow = r * BT + row;      // row inside the sequence
        const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
        const uint32_t tA = lane_base + COL_ACC, tP = lane_base + COL_P, tO = lane_base + COL_OUT;
        const float* dden_b = (MODE == DQ || MODE == DK) ? p.dden + (int64_t)b * p.S : nullptr;
        const float rank_row = (MODE == DQ && grow < p.S) ? dden_b[grow] : 0.f;
        float rs = 0.f;  // FWD: this row's sum of the masked products = den
        for (int t = t0, ti = 0; t <= t1; t++, ti++) {
            mbar_wait(&acc_full, ti & 1, guard, 821);
            tc_fence_after();
            const bool diag = t == r;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                uint32_t v[32];
                tmem_ld32(tA + 32 * c, v);
                tmem_ld_wait();
                if (c == 3) {  // the whole row is in registers: the next product may overwrite the columns
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_free);
                }
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float x[2];
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const int col = 32 * c + i + e;
                        float a = __uint_as_float(v[i + e]);
                        if (MODE == DQ) a += rank_row;
                        if (MODE == DK) {  // every lane reads the same address: one broadcast transaction
                            const int q = t * BT + col;
                            a += q < p.S ? __ldg(dden_b + q) : 0.f;
                        }
                        // rows are queries and columns keys (LOWER), or the other way round: a key is visible
                        // to the queries at or after it
                        if (diag && (LOWER ? col > row : row > col)) a = 0.f;
                        if (MODE == FWD) rs += a;
                        x[e] = a;
                    }
                    pk[i / 2] = pack_bf16(x[0], x[1]);
                }
                if (c == 0 && ti > 0) {  // the products of the partner before have read the bf16 tile
                    mbar_wait(&p_free, (ti - 1) & 1, guard, 822);
                    tc_fence_after();
                }
                tmem_st16(tP + 16 * c, pk);
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full);
        }
        // epilogue: result rows out of TMEM, 32 columns at a time
        mbar_wait(&out_full, 0, guard, 823);
        tc_fence_after();
        float scale = 1.0f;
        if (MODE == FWD) {
            scale = 1.0f / (rs + 1e-8f);
            if (g == 0 && grow < p.S) p.den[(int64_t)b * p.S + grow] = p.eps_in_den ? rs + 1e-8f : rs;
        }
        for (int cb = 0; cb < 2 * ncb; cb++) {
            uint32_t o[32];
            tmem_ld32(tO + 32 * cb, o);
            tmem_ld_wait();
            if (grow < p.S) {
                uint4* dst = reinterpret_cast<uint4*>(p.out + ((int64_t)b * p.S + grow) * p.ldo + g * GW + 32 * cb);
#pragma unroll
                for (int i = 0; i < 32; i += 8)
                    dst[i / 8] = make_uint4(
                        pack_bf16(__uint_as_float(o[i]) * scale, __uint_as_float(o[i + 1]) * scale),
                        pack_bf16(__uint_as_float(o[i + 2]) * scale, __uint_as_float(o[i + 3]) * scale),
                        pack_bf16(__uint_as_float(o[i + 4]) * scale, __uint_as_float(o[i + 5]) * scale),
                        pack_bf16(__uint_as_float(o[i + 6]) * scale, __uint_as_float(o[i + 7]) * scale));
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == W_MMA) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

// ---- element-wise passes either side of the kernel (HBM-bound, 16-byte accesses) ----
__device__ __forceinline__ float bf_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ float phi(float a) { return a > 0.f ? a + 1.f : expf(a); }
__device__ __forceinline__ float dphi(float a) { return a > 0.f ? 1.f : expf(a); }

// y = phi(x), bf16 -> bf16, n8 groups of eight elements
// (blockIdx.y = 1: the second tensor of a pair, so that Q and K take one launch)
__global__ void wide_phi_kernel(const uint4* __restrict__ x0, uint4* __restrict__ y0, const uint4* __restrict__ x1,
                                uint4* __restrict__ y1, size_t n8) {
    const uint4* __restrict__ x = blockIdx.y ? x1 : x0;
    uint4* __restrict__ y = blockIdx.y ? y1 : y0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
        const uint4 v = x[i];
        y[i] = make_uint4(pack_bf16(phi(bf_lo(v.x)), phi(bf_hi(v.x))), pack_bf16(phi(bf_lo(v.y)), phi(bf_hi(v.y))),
                          pack_bf16(phi(bf_lo(v.z)), phi(bf_hi(v.z))), pack_bf16(phi(bf_lo(v.w)), phi(bf_hi(v.w))));
    }
}
// dx = dy o phi'(x), bf16
__global__ void wide_dphi_kernel(const uint4* __restrict__ dy0, const uint4* __restrict__ x0, uint4* __restrict__ dx0,
                                 const uint4* __restrict__ dy1, const uint4* __restrict__ x1, uint4* __restrict__ dx1,
                                 size_t n8) {
    const uint4* __restrict__ dy = blockIdx.y ? dy1 : dy0;
    const uint4* __restrict__ x = blockIdx.y ? x1 : x0;
    uint4* __restrict__ dx = blockIdx.y ? dx1 : dx0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
        const uint4 v = x[i], d = dy[i];
        dx[i] = make_uint4(pack_bf16(bf_lo(d.x) * dphi(bf_lo(v.x)), bf_hi(d.x) * dphi(bf_hi(v.x))),
                           pack_bf16(bf_lo(d.y) * dphi(bf_lo(v.y)), bf_hi(d.y) * dphi(bf_hi(v.y))),
                           pack_bf16(bf_lo(d.z) * dphi(bf_lo(v.z)), bf_hi(d.z) * dphi(bf_hi(v.z))),
                           pack_bf16(bf_lo(d.w) * dphi(bf_lo(v.w)), bf_hi(d.w) * dphi(bf_hi(v.w))));
    }
}
// step 1: dnum = dO / den (bf16), dden = -(dO . O) / den (float); one warp per row, E % 8 == 0
__global__ void wide_step1_kernel(const uint4* __restrict__ O, const uint4* __restrict__ dO, const float* __restrict__ den,
                                  uint4* __restrict__ dnum, float* __restrict__ dden, size_t N, int E8) {
    const size_t row = (size_t)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    if (row >= N) return;
    const float inv = 1.0f / den[row];
    float dot = 0.f;
    for (int e = lane; e < E8; e += 32) {
        const uint4 a = dO[row * E8 + e], c = O[row * E8 + e];
        dot += bf_lo(a.x) * bf_lo(c.x) + bf_hi(a.x) * bf_hi(c.x) + bf_lo(a.y) * bf_lo(c.y) + bf_hi(a.y) * bf_hi(c.y) +
               bf_lo(a.z) * bf_lo(c.z) + bf_hi(a.z) * bf_hi(c.z) + bf_lo(a.w) * bf_lo(c.w) + bf_hi(a.w) * bf_hi(c.w);
        dnum[row * E8 + e] =
            make_uint4(pack_bf16(bf_lo(a.x) * inv, bf_hi(a.x) * inv), pack_bf16(bf_lo(a.y) * inv, bf_hi(a.y) * inv),
                       pack_bf16(bf_lo(a.z) * inv, bf_hi(a.z) * inv), pack_bf16(bf_lo(a.w) * inv, bf_hi(a.w) * inv));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (lane == 0) dden[row] = -dot * inv;
}

// z_cache[t][d] = sum over s <= t of phiK[s][d] (float), one thread per (unit, d) walking the sequence; the
// threads of a warp read consecutive d.  Only for callers of the kept reference signature, which hands
// z_cache to its backward; this library's wide backward does not read it.
__global__ void wide_zcache_kernel(const __nv_bfloat16* __restrict__ pk, float* __restrict__ zc, int B, int S, int D,
                                   int ldk, int ldz) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)B * D) return;
    const int b = (int)(i / D), d = (int)(i % D);
    float run = 0.f;
    for (int t = 0; t < S; t++) {
        const int64_t row = (int64_t)b * S + t;
        run += __bfloat162float(pk[row * ldk + d]);
        zc[row * ldz + d] = run;
    }
}

unsigned flat_grid8(size_t n8) { return (unsigned)std::max<size_t>(1, std::min<size_t>((n8 + 255) / 256, (size_t)sm_count() * 8)); }

// Carves the workspace: phiQ | phiK | dnum | dden | dphiQ | dphiK
struct WideWs {
    __nv_bfloat16 *pq, *pk, *dnum, *dpq, *dpk;
    float* dden;
    size_t bytes;
};
WideWs carve(const cxxattn_lin_desc& d, void* base) {
    const size_t N = (size_t)d.B * d.S;
    char* p = static_cast<char*>(base);
    WideWs w;
    size_t off = 0;
    auto take = [&](size_t n) { char* q = p ? p + off : nullptr; off += align_up(n, 256); return q; };
    w.pq = reinterpret_cast<__nv_bfloat16*>(take(N * d.D * 2));
    w.pk = reinterpret_cast<__nv_bfloat16*>(take(N * d.D * 2));
    w.dnum = reinterpret_cast<__nv_bfloat16*>(take(N * d.E * 2));
    w.dden = reinterpret_cast<float*>(take(N * 4));
    w.dpq = reinterpret_cast<__nv_bfloat16*>(take(N * d.D * 2));
    w.dpk = reinterpret_cast<__nv_bfloat16*>(take(N * d.D * 2));
    w.bytes = off;
    return w;
}

// ldw: row stride of the D-wide tensors among L, R, Z and the result (the E-wide ones are dense)
template <int MODE>
int launch(const cxxattn_lin_desc& d, const void* L, const void* R, const void* Z, int WL, int WO, void* out, float* den,
           const float* dden, int ldw, cudaStream_t st) {
    const int B = (int)d.B, S = (int)d.S;
    constexpr bool LR_WIDE = MODE == FWD || MODE == DV;  // L and R are Q/K-like; otherwise Z and the result are
    const int ldL = LR_WIDE ? ldw : WL, ldZ = LR_WIDE ? WO : ldw;
    CUtensorMap tmL, tmR, tmZ;
    if (!make_tmap_bhsd(&tmL, L, B, S, WL / KB, KB, (int64_t)S * ldL, ldL, KB, BT) ||
        !make_tmap_bhsd(&tmR, R, B, S, WL / KB, KB, (int64_t)S * ldL, ldL, KB, BT) ||
        !make_tmap_bhsd(&tmZ, Z, B, S, WO / KB, KB, (int64_t)S * ldZ, ldZ, KB, BT))
        return CXXATTN_ERR_CUDA;
    WideParams p;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.den = den;
    p.dden = dden;
    p.status = status_word();
    if (p.status == nullptr) return CXXATTN_ERR_CUDA;
    p.B = B; p.S = S; p.WL = WL; p.WO = WO;
    p.ldo = ldZ;
    p.eps_in_den = d.eps_in_den;
    static OncePerDevice attr;
    const int dev = current_device();
    if (attr.pending(dev)) {
        if (cudaFuncSetAttribute(linattn_wide_kernel<FWD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES) != cudaSuccess ||
            cudaFuncSetAttribute(linattn_wide_kernel<DQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES) != cudaSuccess ||
            cudaFuncSetAttribute(linattn_wide_kernel<DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES) != cudaSuccess ||
            cudaFuncSetAttribute(linattn_wide_kernel<DK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES) != cudaSuccess)
            return CXXATTN_ERR_CUDA;
        attr.done(dev);
    }
    const int64_t grid = (int64_t)B * ((S + BT - 1) / BT) * ((WO + GW - 1) / GW);
    if (grid > INT32_MAX) return CXXATTN_ERR_TOO_LARGE;
    linattn_wide_kernel<MODE><<<(unsigned)grid, NTHREADS, SMEM_BYTES, st>>>(tmL, tmR, tmZ, p);
    return check_launch();
}

// Row stride of the D-wide operands of a launch: the mapped copies in the workspace are dense
int ldw(const cxxattn_lin_desc& d, bool map) { return (map || d.ld_qk == 0) ? (int)d.D : (int)d.ld_qk; }

}  // namespace

// bf16, widths that are multiples of the 64-wide K block; D = E = 64 has kernels of its own
bool linattn_wide_supported(const cxxattn_lin_desc& d) {
    const bool dense = d.ld_qk == 0 || d.ld_qk == d.D;
    // rows wider than D (the first D columns of padded features) only without the fused feature map, and
    // on a stride TMA can take (a multiple of 16 bytes)
    return d.dtype == CXXATTN_BF16 && d.D % KB == 0 && d.E % KB == 0 && d.D <= 8192 && d.E <= 8192 &&
           (dense ? !(d.D == 64 && d.E == 64) : (d.feature_map == CXXATTN_MAP_NONE && d.ld_qk % 8 == 0));
}

size_t linattn_wide_workspace(const cxxattn_lin_desc& d) { return linattn_wide_supported(d) ? carve(d, nullptr).bytes : 0; }

namespace {
// phi of one tensor, or of two of the same size in one launch (x1 == nullptr: one)
int phi_pass(const void* x0, void* y0, const void* x1, void* y1, size_t n8, cudaStream_t st) {
    const dim3 grid(flat_grid8(n8), x1 != nullptr ? 2u : 1u);
    wide_phi_kernel<<<grid, 256, 0, st>>>(static_cast<const uint4*>(x0), static_cast<uint4*>(y0),
                                         static_cast<const uint4*>(x1), static_cast<uint4*>(y1), n8);
    return check_launch();
}
// dx = dy o phi'(x), likewise
int dphi_pass(const void* dy0, const void* x0, void* dx0, const void* dy1, const void* x1, void* dx1, size_t n8,
              cudaStream_t st) {
    const dim3 grid(flat_grid8(n8), dy1 != nullptr ? 2u : 1u);
    wide_dphi_kernel<<<grid, 256, 0, st>>>(static_cast<const uint4*>(dy0), static_cast<const uint4*>(x0), static_cast<uint4*>(dx0),
                                          static_cast<const uint4*>(dy1), static_cast<const uint4*>(x1), static_cast<uint4*>(dx1),
                                          n8);
    return check_launch();
}
}  // namespace

int linattn_wide_fwd(const cxxattn_lin_desc& d, const void* Q, const void* K, const void* V, void* O, float* den,
                     float* z_cache, void* ws, size_t ws_bytes, cudaStream_t st) {
    if (!linattn_wide_supported(d)) return CXXATTN_ERR_UNSUPPORTED;
    for (const void* q : {Q, K, V, (const void*)O})
        if (reinterpret_cast<uintptr_t>(q) % 16) return CXXATTN_ERR_ALIGNMENT;
    if (ws == nullptr || ws_bytes < carve(d, nullptr).bytes) return CXXATTN_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(ws) % 256) return CXXATTN_ERR_ALIGNMENT;
    const WideWs w = carve(d, ws);
    const void *q = Q, *k = K;
    const bool map = d.feature_map == CXXATTN_MAP_ELU1;
    if (map) {
        const size_t n8 = (size_t)d.B * d.S * d.D / 8;
        if (phi_pass(Q, w.pq, K, w.pk, n8, st) != CXXATTN_OK) return CXXATTN_ERR_CUDA;
        q = w.pq;
        k = w.pk;
    }
    if (z_cache != nullptr) {
        const int64_t n = d.B * d.D;
        wide_zcache_kernel<<<(unsigned)((n + 127) / 128), 128, 0, st>>>(static_cast<const __nv_bfloat16*>(k), z_cache, (int)d.B,
                                                                      (int)d.S, (int)d.D, ldw(d, map), ldw(d, false));
        if (check_launch() != CXXATTN_OK) return CXXATTN_ERR_CUDA;
    }
    return launch<FWD>(d, q, k, V, (int)d.D, (int)d.E, O, den, nullptr, ldw(d, map), st);
}

// The two halves of the backward as the reference's interface cuts it (kernel_attn_bwd_dQ / _dKdV,
// causal_linear_attention_bwd_dQ / _dKdV): dnum (bf16) and dden (float) come from step 1.
int linattn_wide_bwd_dq(const cxxattn_lin_desc& d, const void* K, const void* V, const void* dnum, const float* dden,
                        const void* Q, void* dQ, void* ws, size_t ws_bytes, cudaStream_t st) {
    if (!linattn_wide_supported(d)) return CXXATTN_ERR_UNSUPPORTED;
    const bool map = d.feature_map == CXXATTN_MAP_ELU1;
    if (map && Q == nullptr) return CXXATTN_ERR_INVALID;
    for (const void* q : {K, V, dnum, Q, (const void*)dQ})
        if (reinterpret_cast<uintptr_t>(q) % 16) return CXXATTN_ERR_ALIGNMENT;
    if (ws == nullptr || ws_bytes < carve(d, nullptr).bytes) return CXXATTN_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(ws) % 256) return CXXATTN_ERR_ALIGNMENT;
    const WideWs w = carve(d, ws);
    const size_t n8 = (size_t)d.B * d.S * d.D / 8;
    const void* k = K;
    if (map) {  // the mapped copies are rebuilt: the workspace need not survive from an earlier call
        if (phi_pass(K, w.pk, nullptr, nullptr, n8, st) != CXXATTN_OK) return CXXATTN_ERR_CUDA;
        k = w.pk;
    }
    int rc = launch<DQ>(d, dnum, V, k, (int)d.E, (int)d.D, map ? (void*)w.dpq : dQ, nullptr, dden, ldw(d, map), st);
    if (rc != CXXATTN_OK || !map) return rc;
    return dphi_pass(w.dpq, Q, dQ, nullptr, nullptr, nullptr, n8, st);
}

int linattn_wide_bwd_dkdv(const cxxattn_lin_desc& d, const void* Q, const void* K, const void* V, const void* dnum,
                          const float* dden, void* dK, void* dV, void* ws, size_t ws_bytes, cudaStream_t st) {
    if (!linattn_wide_supported(d)) return CXXATTN_ERR_UNSUPPORTED;
    for (const void* q : {Q, K, V, dnum, (const void*)dK, (const void*)dV})
        if (reinterpret_cast<uintptr_t>(q) % 16) return CXXATTN_ERR_ALIGNMENT;
    if (ws == nullptr || ws_bytes < carve(d, nullptr).bytes) return CXXATTN_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(ws) % 256) return CXXATTN_ERR_ALIGNMENT;
    const WideWs w = carve(d, ws);
    const bool map = d.feature_map == CXXATTN_MAP_ELU1;
    const size_t n8 = (size_t)d.B * d.S * d.D / 8;
    const void *q = Q, *k = K;
    if (map) {
        if (phi_pass(Q, w.pq, K, w.pk, n8, st) != CXXATTN_OK) return CXXATTN_ERR_CUDA;
        q = w.pq;
        k = w.pk;
    }
    int rc = launch<DV>(d, k, q, dnum, (int)d.D, (int)d.E, dV, nullptr, nullptr, ldw(d, map), st);
    if (rc != CXXATTN_OK) return rc;
    rc = launch<DK>(d, V, dnum, q, (int)d.E, (int)d.D, map ? (void*)w.dpk : dK, nullptr, dden, ldw(d, map), st);
    if (rc != CXXATTN_OK || !map) return rc;
    return dphi_pass(w.dpk, K, dK, nullptr, nullptr, nullptr, n8, st);
}

// The whole backward: step 1, then the two halves.
int linattn_wide_bwd(const cxxattn_lin_desc& d, const void* Q, const void* K, const void* V, const void* O, const void* dO,
                     const float* den, void* dQ, void* dK, void* dV, void* ws, size_t ws_bytes, cudaStream_t st) {
    if (!linattn_wide_supported(d)) return CXXATTN_ERR_UNSUPPORTED;
    for (const void* q : {O, dO})
        if (reinterpret_cast<uintptr_t>(q) % 16) return CXXATTN_ERR_ALIGNMENT;
    if (ws == nullptr || ws_bytes < carve(d, nullptr).bytes) return CXXATTN_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(ws) % 256) return CXXATTN_ERR_ALIGNMENT;
    const WideWs w = carve(d, ws);
    const size_t N = (size_t)d.B * d.S;
    wide_step1_kernel<<<(unsigned)((N + 7) / 8), 256, 0, st>>>(static_cast<const uint4*>(O), static_cast<const uint4*>(dO), den,
                                                              reinterpret_cast<uint4*>(w.dnum), w.dden, N, (int)(d.E / 8));
    if (check_launch() != CXXATTN_OK) return CXXATTN_ERR_CUDA;
    // the two halves in one go: phi(Q) and phi(K) are built once and together, and so are the two phi' passes
    for (const void* q : {Q, K, V, (const void*)dQ, (const void*)dK, (const void*)dV})
        if (reinterpret_cast<uintptr_t>(q) % 16) return CXXATTN_ERR_ALIGNMENT;
    const bool map = d.feature_map == CXXATTN_MAP_ELU1;
    const size_t n8 = (size_t)d.B * d.S * d.D / 8;
    const void *q = Q, *k = K;
    if (map) {
        if (phi_pass(Q, w.pq, K, w.pk, n8, st) != CXXATTN_OK) return CXXATTN_ERR_CUDA;
        q = w.pq;
        k = w.pk;
    }
    int rc = launch<DQ>(d, w.dnum, V, k, (int)d.E, (int)d.D, map ? (void*)w.dpq : dQ, nullptr, w.dden, ldw(d, map), st);
    if (rc != CXXATTN_OK) return rc;
    rc = launch<DV>(d, k, q, w.dnum, (int)d.D, (int)d.E, dV, nullptr, nullptr, ldw(d, map), st);
    if (rc != CXXATTN_OK) return rc;
    rc = launch<DK>(d, V, w.dnum, q, (int)d.E, (int)d.D, map ? (void*)w.dpk : dK, nullptr, w.dden, ldw(d, map), st);
    if (rc != CXXATTN_OK || !map) return rc;
    return dphi_pass(w.dpq, Q, dQ, w.dpk, K, dK, n8, st);
}

}  // namespace cxxattn
