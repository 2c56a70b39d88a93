// Group states for the bf16 tensor-core linear attention: the pre-pass that lets several CTAs share
// one batch unit's sequence.
//
// The reference scans a sequence serially (two_stage_cuda::kernel_attn_fwd and the three backward
// scans, src/TwoStage/two_stage_cuda_kernels.cu:889-1809; linear_cuda::*,
// src/LinearAttention/linear_cuda_kernels.cu:10-298).  The chunked kernels here keep a running state
// per batch unit, so with fewer units than SMs most of the GPU would idle.  The sequence is therefore
// cut into G groups of chunks; this kernel computes, for one (unit, group), the state contribution of
// the group alone,
//
//   mode 0 (prefix states, forward and dQ pass):   sum_t phi(K_t) (x) [V_t | 1]
//   mode 1 (suffix states, dK/dV pass):            sum_t phi(Q_t) (x) [dnum_t | dden_t]   (step 1 fused)
//
// as one SS MMA per chunk (64 state rows issued as M = 128 with the operand block repeated, N = 80:
// the 65th column is z), accumulated in TMEM over the group and written as fp32 to global memory.
// The main kernels start a group from the sum of the states of the groups before (after) it.
#include <algorithm>

#include "linattn_tc_common.cuh"

namespace cxxattn {
namespace {

using namespace tc;
using namespace lintc;

constexpr int NSTAGE = 2;
constexpr int NTHREADS = 320;  // 8 preparation warps, TMA producer, MMA issuer
constexpr int W_PROD = 8, W_MMA = 9;
constexpr uint32_t TMEM_COLS = 128;
// per stage A | B | side tile, then the constant ones tile
constexpr size_t SMEM_BYTES = (NSTAGE * 3 + 1) * TILE_BYTES + 1024;

struct LinStateParams {
    const __nv_bfloat16* O;  // mode 1: rows of O for dden
    const float* den;        // mode 1
    float* gstate;           // [B][G][64][GS_ROW]
    int* status;
    int B, S, G, gc;
    int map_elu;
};

template <int MODE>
__global__ void __launch_bounds__(NTHREADS, 1)
linattn_tc_state_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        LinStateParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full[NSTAGE], stage_free[NSTAGE], mapped[NSTAGE], done;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    auto sA = [&](int st) { return smem + (st * 3 + 0) * TILE_BYTES; };     // K (mode 0) or Q (mode 1), mapped in place
    auto sB = [&](int st) { return smem + (st * 3 + 1) * TILE_BYTES; };     // V, or dO rescaled to dnum in place
    auto sSide = [&](int st) { return smem + (st * 3 + 2) * TILE_BYTES; };  // mode 1: column 0 = dden_t
    uint8_t* sOnes = smem + NSTAGE * 3 * TILE_BYTES;                        // mode 0: column 0 = 1

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int b = blockIdx.x / (p.G - 1);
    const int g = blockIdx.x % (p.G - 1) + (MODE == 0 ? 0 : 1);
    const int nc = (p.S + CH - 1) / CH;
    const int c0 = g * p.gc;
    const int ng = min(nc, c0 + p.gc) - c0;  // chunks of this group (>= 1 by construction of the plan)
    const Guard guard{&abort_flag, p.status};

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < NSTAGE; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&stage_free[s], 1);
        }
        // one barrier per stage, so that a warp that runs a chunk ahead cannot complete an earlier phase
        for (int s = 0; s < NSTAGE; s++) mbar_init(&mapped[s], 8);
        mbar_init(&done, 1);
        fence_barrier_init();
    }
    if (warp == W_MMA) tmem_alloc(&tmem_slot, TMEM_COLS);
    // side tiles and the ones tile start as zero; only column 0 is ever written
    for (int st = 0; st < NSTAGE; st++)
        for (int i = threadIdx.x; i < TILE_BYTES / 16; i += NTHREADS)
            reinterpret_cast<uint4*>(sSide(st))[i] = make_uint4(0u, 0u, 0u, 0u);
    for (int i = threadIdx.x; i < TILE_BYTES / 16; i += NTHREADS)
        reinterpret_cast<uint4*>(sOnes)[i] = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
    if (threadIdx.x < CH)  // element (row, 0) of the swizzled tile sits in 16-byte chunk (row & 7)
        *reinterpret_cast<uint16_t*>(sOnes + threadIdx.x * 128 + (threadIdx.x & 7) * 16) = 0x3f80;  // bf16 1.0
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;

    if (warp == W_PROD) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            prefetch_tmap(&tmA);
            prefetch_tmap(&tmB);
            for (int c = 0; c < ng; c++) {
                const int st = c % NSTAGE;
                if (c >= NSTAGE) mbar_wait(&stage_free[st], ((c / NSTAGE) - 1) & 1, guard, 1001);
                mbar_expect_tx(&full[st], 2 * TILE_BYTES);
                tma_load_4d(sA(st), &tmA, &full[st], 0, 0, (c0 + c) * CH, b);
                tma_load_4d(sB(st), &tmB, &full[st], 0, 0, (c0 + c) * CH, b);
            }
        }
    } else if (warp == W_MMA) {
        // ---------------- MMA issuer (warp-uniform; one elected lane issues) ----------------
        const uint32_t el = elect_one();
        constexpr uint32_t IDESC_S = idesc_bf16(CH, 80, 1, 1);  // both operands MN-major
        for (int c = 0; c < ng; c++) {
            const int st = c % NSTAGE;
            // A: 64 state rows; the second block of 64 rows (offset 0) repeats the first, its output
            // lanes are never read.  B: [V | 1] or [dnum | dden]: the second block of 64 columns is
            // the ones tile or this stage's side tile.
            const uint64_t dAm = smem_desc_sw128(smem_u32(sA(st)), 0);
            const uint32_t second = MODE == 0 ? smem_u32(sOnes) : smem_u32(sSide(st));
            const uint64_t dB1 = smem_desc_sw128(smem_u32(sB(st)), second - smem_u32(sB(st)));
            mbar_wait_poll(&mapped[st], (c / NSTAGE) & 1, guard, 1011);
            tc_fence_after();
#pragma unroll
            for (int k = 0; k < CH / 16; k++) umma_ss_e(el, tmem, dAm + 128 * k, dB1 + 128 * k, IDESC_S, c > 0 || k > 0);
            umma_commit_e(el, &stage_free[st]);
        }
        umma_commit_e(el, &done);
    } else {
        // ---------------- preparation warps: two threads per token row of the chunk ----------------
        // mode 0: each maps half a row of K; mode 1: warps 0-3 do step 1 on the dO tile, warps 4-7 map Q
        // (a lone warp per scheduler doing everything would set the pace of the kernel)
        const int r = (warp % 4) * 32 + lane;
        const int second = warp / 4;
        for (int c = 0; c < ng; c++) {
            const int st = c % NSTAGE;
            const int tok = (c0 + c) * CH + r;
            const bool ok = tok < p.S;
            const int64_t row = (int64_t)b * p.S + tok;
            float den = 1.f;
            if (MODE == 1 && !second && ok) {
                den = p.den[row];
                if (tok + 2 * CH < p.S) prefetch_row(p.O + (row + 2 * CH) * DE);
            }
            mbar_wait(&full[st], (c / NSTAGE) & 1, guard, 1021);
            if (MODE == 1) {
                if (!second)
                    step1_row(sB(st) + r * 128, p.O + row * DE, den, ok, r & 7, sSide(st) + r * 128 + (r & 7) * 16);
                else if (p.map_elu)
                    map_row(sA(st) + r * 128, ok, true, r & 7);
            } else if (p.map_elu) {
                map_half_row(sA(st) + r * 128, ok, r & 7, second);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&mapped[st]);
        }
        // the group's state: TMEM lanes 0..63, 64 columns + z in column 64 -> global fp32
        mbar_wait(&done, 0, guard, 1022);
        tc_fence_after();
        if (warp < 2) {
            const uint32_t taddr = tmem + (static_cast<uint32_t>(warp * 32) << 16);
            uint32_t s0[32], s1[32], s2[32];
            tmem_ld32(taddr, s0);
            tmem_ld32(taddr + 32, s1);
            tmem_ld32(taddr + 64, s2);
            tmem_ld_wait();
            float4* dst = reinterpret_cast<float4*>(p.gstate + (((int64_t)b * p.G + g) * DE + r) * GS_ROW);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                dst[i] = make_float4(__uint_as_float(s0[4 * i]), __uint_as_float(s0[4 * i + 1]),
                                     __uint_as_float(s0[4 * i + 2]), __uint_as_float(s0[4 * i + 3]));
                dst[8 + i] = make_float4(__uint_as_float(s1[4 * i]), __uint_as_float(s1[4 * i + 1]),
                                         __uint_as_float(s1[4 * i + 2]), __uint_as_float(s1[4 * i + 3]));
            }
            dst[16] = make_float4(__uint_as_float(s2[0]), 0.f, 0.f, 0.f);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == W_MMA) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

}  // namespace

// Groups are worth it when the batch units leave SMs idle.  The cost model counts chunk-times: a main
// CTA costs its chunks plus a fixed fill/drain of about two, a pre-pass CTA about a quarter of that
// per chunk; CTAs run in waves of one per SM.
LinGroupPlan linattn_tc_plan(int B, int S) {
    const int nsm = sm_count();
    const int nc = (S + lintc::CH - 1) / lintc::CH;
    auto waves = [&](int64_t ctas) { return (double)((ctas + nsm - 1) / nsm); };
    LinGroupPlan best{1, nc, 0};
    double best_cost = waves(B) * (nc + 2.0);
    // CXXATTN_OPT_LIN_GROUPS = G > 0 forces the number of groups (rounded to one without empty groups)
    const int forced = option(CXXATTN_OPT_LIN_GROUPS);
    if (forced > 0) {
        const int gc = (nc + std::min(forced, nc) - 1) / std::min(forced, nc);
        const int G = (nc + gc - 1) / gc;
        if (G < 2) return best;
        return LinGroupPlan{G, gc, (size_t)B * G * lintc::DE * lintc::GS_ROW * sizeof(float)};
    }
    for (int G = 2; G <= 16 && G <= nc; G++) {
        const int gc = (nc + G - 1) / G;
        if ((nc + gc - 1) / gc != G) continue;  // this G leaves an empty last group: a smaller G covers it
        const double cost = waves((int64_t)B * G) * (gc + 2.0) + waves((int64_t)B * (G - 1)) * (0.25 * gc + 1.0);
        if (cost < 0.95 * best_cost) {
            best_cost = cost;
            best = LinGroupPlan{G, gc, (size_t)B * G * lintc::DE * lintc::GS_ROW * sizeof(float)};
        }
    }
    return best;
}

int linattn_tc_group_states(int mode, const LinGroupPlan& plan, int B, int S, int map_elu, const void* A, const void* Bm,
                            const void* O, const float* den, float* gstate, cudaStream_t st) {
    using namespace lintc;
    if (plan.G < 2) return CXXATTN_OK;
    CUtensorMap tmA, tmB;
    if (!make_tmap_bhsd(&tmA, A, B, S, 1, DE, (int64_t)S * DE, DE, DE, CH) ||
        !make_tmap_bhsd(&tmB, Bm, B, S, 1, DE, (int64_t)S * DE, DE, DE, CH))
        return CXXATTN_ERR_CUDA;
    LinStateParams p;
    p.O = static_cast<const __nv_bfloat16*>(O);
    p.den = den;
    p.gstate = gstate;
    p.status = status_word();
    if (p.status == nullptr) return CXXATTN_ERR_CUDA;
    p.B = B; p.S = S; p.G = plan.G; p.gc = plan.gc;
    p.map_elu = map_elu;
    static OncePerDevice attr;
    const int dev = current_device();
    if (attr.pending(dev)) {
        if (cudaFuncSetAttribute(linattn_tc_state_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)SMEM_BYTES) != cudaSuccess ||
            cudaFuncSetAttribute(linattn_tc_state_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)SMEM_BYTES) != cudaSuccess)
            return CXXATTN_ERR_CUDA;
        attr.done(dev);
    }
    const unsigned grid = (unsigned)(B * (plan.G - 1));
    if (mode == 0) linattn_tc_state_kernel<0><<<grid, NTHREADS, SMEM_BYTES, st>>>(tmA, tmB, p);
    else linattn_tc_state_kernel<1><<<grid, NTHREADS, SMEM_BYTES, st>>>(tmA, tmB, p);
    return check_launch();
}

}  // namespace cxxattn
