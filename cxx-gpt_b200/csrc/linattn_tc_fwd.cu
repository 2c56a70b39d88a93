// Causal linear attention forward on the tensor cores (tcgen05 + TMEM + TMA), bf16 tensors with
// fp32 accumulation and fp32 running state, D = E = 64.
//
// Replaces the serial per-timestep scan of two_stage_cuda::kernel_attn_fwd
// (src/TwoStage/two_stage_cuda_kernels.cu:889-976) and linear_cuda::causal_linear_attention_fwd
// (src/LinearAttention/linear_cuda_kernels.cu:10-79) for dtype BF16.  One CTA owns one batch unit
// and walks its sequence in chunks of 128 tokens; Q, K and V are read from HBM exactly once (TMA),
// O and den are written once, and the running state never leaves the SM:
//
//   phi            the feature map (ELU+1 or none) is applied in place on the Q and K tiles in shared
//                  memory by four dedicated warps, rows past the end of the sequence are zeroed
//   A   = phiQ phiK^T                       (SS MMA 128x128x64)   -> TMEM, masked to s <= t by the
//                                            compute warps, row sums taken, bf16 back to TMEM (P)
//   O'  = phiQ [S_prev | z_prev]            (SS MMA 128x80x64: the state of all earlier chunks as a
//                                            bf16 operand, its 65th column is z and yields phiQ.z)
//   O' += P V                               (TS MMA 128x64x128)
//   S  += phiK^T [V | 1]                    (SS MMA, 64 state rows (issued as M=128 with the operand
//                                            block repeated), N=80: the constant column of ones makes
//                                            column 64 the running z = sum phiK)
//   O   = O'[:, :64] / (den + 1e-8),  den = rowsum(A masked) + O'[:, 64]
//
// The state S (fp32, 64 x 65) lives in TMEM for the whole sequence; after each chunk it is copied
// as bf16 into shared memory to serve as the operand of the next chunk's inter-chunk product.
#include "linattn_tc_common.cuh"

namespace cxxattn {
namespace {

using namespace tc;
using namespace lintc;

constexpr int NSTAGE = 3;  // the feature-map warps work up to two chunks ahead of the products
constexpr int NTHREADS = 512;  // 4 compute warps, TMA producer, MMA issuer, 8 feature-map warps (4 for Q, 4 for K), 2 idle
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t COL_A = 0, COL_P = 128, COL_O = 192, COL_SX = 288;
// per stage Q | K | V, then the ones tile, then the bf16 state operand (2 blocks of 64 rows x 128 B)
constexpr size_t SMEM_BYTES = NSTAGE * 3 * TILE_BYTES + TILE_BYTES + 2 * 8192 + 1024;

struct LinFwdParams {
    __nv_bfloat16* O;
    float* den;
    int* status;
    int B, S;
    int map_elu;     // 1: phi(x) = x > 0 ? x + 1 : exp(x) applied to Q and K; 0: inputs pre-mapped
    int eps_in_den;  // 1: den stored with the 1e-8 added
    SeqGroups sg;    // sequence groups (G = 1: one CTA per unit)
};

__global__ void __launch_bounds__(NTHREADS, 1)
linattn_tc_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, LinFwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full[NSTAGE], stage_free[NSTAGE], mapped[NSTAGE], a_full, p_ready, o_full, o_free, s_done, sprev_ready;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ float s_rowsum[2][CH];  // row sums of the masked A, from the compute warps to the output warps

    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    auto sQ = [&](int st) { return smem + (st * 3 + 0) * TILE_BYTES; };
    auto sK = [&](int st) { return smem + (st * 3 + 1) * TILE_BYTES; };
    auto sV = [&](int st) { return smem + (st * 3 + 2) * TILE_BYTES; };
    uint8_t* sOnes = smem + NSTAGE * 3 * TILE_BYTES;  // [128 tokens][64] bf16, column 0 = 1
    uint8_t* sPrev = sOnes + TILE_BYTES;              // block 0: S_prev [64 d][64 e]; block 1: column 0 = z_prev

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int b = blockIdx.x / p.sg.G, g = blockIdx.x % p.sg.G;  // batch unit, sequence group
    const int c0 = g * p.sg.gc;                                   // first chunk of the group
    const int nc = min((p.S + CH - 1) / CH, c0 + p.sg.gc) - c0;   // chunks of the group
    const Guard guard{&abort_flag, p.status};

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < NSTAGE; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&stage_free[s], 1);
        }
        mbar_init(&a_full, 1);
        mbar_init(&o_full, 1);
        mbar_init(&s_done, 1);
        for (int s = 0; s < NSTAGE; s++) mbar_init(&mapped[s], 8);  // one arrival per feature-map warp
        mbar_init(&p_ready, 4);
        mbar_init(&o_free, 8);  // the eight output (feature-map) warps
        mbar_init(&sprev_ready, 4);
        fence_barrier_init();
    }
    if (warp == 5) tmem_alloc(&tmem_slot, TMEM_COLS);
    // constant tiles: ones column, and an all-zero state operand for the first chunk
    for (int i = threadIdx.x; i < (TILE_BYTES + 2 * 8192) / 16; i += NTHREADS)
        reinterpret_cast<uint4*>(sOnes)[i] = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
    if (threadIdx.x < CH)  // element (row, 0) of the swizzled tile sits in 16-byte chunk (row & 7)
        *reinterpret_cast<uint16_t*>(sOnes + threadIdx.x * 128 + (threadIdx.x & 7) * 16) = 0x3f80;  // bf16 1.0
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;

    // Register budget (512 threads x 128 at launch): the compute warps hold whole score rows, every
    // other warp group gives registers back.  The increase blocks until they are there:
    // 4 x 32 x (208 - 128) <= 12 x 32 x (128 - 96).
    if (warp >= 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");

    if (warp == 4) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            prefetch_tmap(&tmQ);
            prefetch_tmap(&tmK);
            prefetch_tmap(&tmV);
            for (int c = 0; c < nc; c++) {
                const int st = c % NSTAGE;
                if (c >= NSTAGE) mbar_wait(&stage_free[st], ((c / NSTAGE) - 1) & 1, guard, 701);
                mbar_expect_tx(&full[st], 3 * TILE_BYTES);
                tma_load_4d(sQ(st), &tmQ, &full[st], 0, 0, (c0 + c) * CH, b);
                tma_load_4d(sK(st), &tmK, &full[st], 0, 0, (c0 + c) * CH, b);
                tma_load_4d(sV(st), &tmV, &full[st], 0, 0, (c0 + c) * CH, b);
            }
        }
    } else if (warp == 5) {
        // ---------------- MMA issuer ----------------
        // the whole warp runs the loop (uniform control flow and operands); one elected lane issues
        {
            const uint32_t el = elect_one();
            constexpr uint32_t IDESC_A = idesc_bf16(CH, CH, 0, 0);  // phiQ phiK^T: both K-major
            constexpr uint32_t IDESC_I = idesc_bf16(CH, 80, 0, 1);  // phiQ [S_prev | z]: B MN-major
            constexpr uint32_t IDESC_P = idesc_bf16(CH, DE, 0, 1);  // P V: A in TMEM, B MN-major
            constexpr uint32_t IDESC_S = idesc_bf16(CH, 80, 1, 1);  // phiK^T [V | 1]: both MN-major
            const uint64_t dPrev = smem_desc_sw128(smem_u32(sPrev), 8192);
            for (int c = 0; c < nc; c++) {
                const int st = c % NSTAGE;
                const uint64_t dQ = smem_desc_sw128(smem_u32(sQ(st)), 16);
                const uint64_t dK = smem_desc_sw128(smem_u32(sK(st)), 16);
                // phiK as an MN-major A operand: 64 state rows; the second block of 64 rows (offset 0)
                // repeats the first, its output lanes are never read
                const uint64_t dKm = smem_desc_sw128(smem_u32(sK(st)), 0);
                const uint64_t dV = smem_desc_sw128(smem_u32(sV(st)), 0);
                // [V | 1]: the second block of 64 columns is the ones tile
                const uint64_t dV1 = smem_desc_sw128(smem_u32(sV(st)), smem_u32(sOnes) - smem_u32(sV(st)));
                mbar_wait_poll(&mapped[st], (c / NSTAGE) & 1, guard, 711);
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < DE / 16; k++) umma_ss_e(el, tmem + COL_A, dQ + 2 * k, dK + 2 * k, IDESC_A, k > 0);
                umma_commit_e(el, &a_full);
                mbar_wait_poll(&sprev_ready, c & 1, guard, 712);
                if (c > 0) mbar_wait_poll(&o_free, (c - 1) & 1, guard, 713);
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < DE / 16; k++) umma_ss_e(el, tmem + COL_O, dQ + 2 * k, dPrev + 128 * k, IDESC_I, k > 0);
#pragma unroll
                for (int k = 0; k < CH / 16; k++)
                    umma_ss_e(el, tmem + COL_SX, dKm + 128 * k, dV1 + 128 * k, IDESC_S, g > 0 || c > 0 || k > 0);
                umma_commit_e(el, &s_done);
                mbar_wait_poll(&p_ready, c & 1, guard, 714);
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < CH / 16; k++)
                    umma_ts_e(el, tmem + COL_O, tmem + COL_P + 8 * k, dV + 128 * k, IDESC_P, true);
                umma_commit_e(el, &o_full);
                umma_commit_e(el, &stage_free[st]);
            }
        }
    } else if (warp >= 14) {
        // idle warps: they only take part in the register hand-over
    } else if (warp >= 6) {
        // ---------------- feature-map warps: thread r = row r of the Q and K tiles ----------------
        // The map is applied in place as soon as a chunk has landed (with no map there is nothing to
        // do: rows past the end are already zero, TMA fills them), independently of the compute
        // warps, which are still busy with the previous chunk.
        // Warps 6-9 take the Q tile, warps 10-13 the K tile: one warp per scheduler alone is too slow
        // (a row is ~450 dependent instructions) and would set the pace of the whole kernel.
        // The same warps write the outputs, one chunk behind: O = O'[:, :64] / (den + 1e-8), den = rowsum
        // + O'[:, 64]; a warp owns the 32 rows of its TMEM lane quarter and one half of the 64 columns.
        const int r = ((warp - 6) % 4) * 32 + lane;  // warps 6..13 sit on lane quarters 2,3,0,1,2,3,0,1
        const bool k_tile = warp >= 10;
        const int rq = (warp % 4) * 32 + lane;  // row of this thread's TMEM lane
        const uint32_t lane_q = tmem + (static_cast<uint32_t>((warp % 4) * 32) << 16);
        const int half = k_tile ? 1 : 0;
        auto write_output = [&](int c) {
            mbar_wait(&o_full, c & 1, guard, 724);
            tc_fence_after();
            uint32_t o0[32], o2[32];
            tmem_ld32(lane_q + COL_O + 32 * half, o0);
            tmem_ld32(lane_q + COL_O + 64, o2);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&o_free);
            const int tok = (c0 + c) * CH + rq;
            if (tok < p.S) {
                const float den = s_rowsum[c & 1][rq] + __uint_as_float(o2[0]);
                const float inv = 1.0f / (den + 1e-8f);
                const int64_t row = (int64_t)b * p.S + tok;
                if (half == 0) p.den[row] = p.eps_in_den ? den + 1e-8f : den;
                uint4* dst = reinterpret_cast<uint4*>(p.O + row * DE + 32 * half);
#pragma unroll
                for (int i = 0; i < 32; i += 8)
                    dst[i / 8] = make_uint4(pack_bf16(__uint_as_float(o0[i]) * inv, __uint_as_float(o0[i + 1]) * inv),
                                            pack_bf16(__uint_as_float(o0[i + 2]) * inv, __uint_as_float(o0[i + 3]) * inv),
                                            pack_bf16(__uint_as_float(o0[i + 4]) * inv, __uint_as_float(o0[i + 5]) * inv),
                                            pack_bf16(__uint_as_float(o0[i + 6]) * inv, __uint_as_float(o0[i + 7]) * inv));
            }
        };
        for (int c = 0; c < nc; c++) {
            const int st = c % NSTAGE;
            mbar_wait(&full[st], (c / NSTAGE) & 1, guard, 721);
            if (p.map_elu) {
                const bool ok = (c0 + c) * CH + r < p.S;
                map_row((k_tile ? sK(st) : sQ(st)) + r * 128, ok, true, r & 7);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&mapped[st]);
            if (c > 0) write_output(c - 1);
        }
        write_output(nc - 1);
    } else {
        // ---------------- compute warps: thread r = token row r of the chunk = TMEM lane r ----------------
        asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
        const int r = warp * 32 + lane;
        const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
        // the state operand of the first chunk is the zero tile written at start-up, or, for a later
        // sequence group, the sum of the states of the groups before it (which also seeds TMEM)
        if (g > 0) init_state_row(p.sg, b, 0, g, r, lane_base + COL_SX, sPrev);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sprev_ready);
        for (int c = 0; c < nc; c++) {
            // A -> causal mask inside the chunk (key column s visible iff s <= r), row sum, bf16 P
            mbar_wait(&a_full, c & 1, guard, 722);
            tc_fence_after();
            float rowsum = 0.f;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                uint32_t v0[32], v1[32], pk[32];
                // columns of a 32-wide block beyond this warp's last row are all masked: not even loaded
                const bool need0 = 64 * h <= warp * 32 + 31, need1 = 64 * h + 32 <= warp * 32 + 31;
                if (need0) tmem_ld32(lane_base + COL_A + 64 * h, v0);
                if (need1) tmem_ld32(lane_base + COL_A + 64 * h + 32, v1);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const float a0 = (need0 && 64 * h + i <= r) ? __uint_as_float(v0[i]) : 0.f;
                    const float a1 = (need0 && 64 * h + i + 1 <= r) ? __uint_as_float(v0[i + 1]) : 0.f;
                    const float b0 = (need1 && 64 * h + 32 + i <= r) ? __uint_as_float(v1[i]) : 0.f;
                    const float b1 = (need1 && 64 * h + 32 + i + 1 <= r) ? __uint_as_float(v1[i + 1]) : 0.f;
                    rowsum += (a0 + a1) + (b0 + b1);
                    pk[i / 2] = pack_bf16(a0, a1);
                    pk[16 + i / 2] = pack_bf16(b0, b1);
                }
                tmem_st32(lane_base + COL_P + 32 * h, pk);
            }
            tmem_st_wait();
            s_rowsum[c & 1][r] = rowsum;  // read by the output warps after o_full(c), which follows p_ready(c)
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready);

            // state after this chunk -> bf16 operand of the next chunk's inter-chunk product
            mbar_wait(&s_done, c & 1, guard, 723);
            tc_fence_after();
            if (c + 1 < nc) {
                state_to_smem(lane_base + COL_SX, sPrev, r);  // shared by the four warps
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sprev_ready);
            }

        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

}  // namespace

bool linattn_tc_supported(const cxxattn_lin_desc& d) { return d.D == DE && d.E == DE && (d.ld_qk == 0 || d.ld_qk == DE); }

size_t linattn_tc_workspace(const cxxattn_lin_desc& d) {
    if (!linattn_tc_supported(d)) return 0;
    return 2 * linattn_tc_plan((int)d.B, (int)d.S).state_bytes;  // prefix and suffix group states
}

int linattn_tc_fwd(const cxxattn_lin_desc& d, const void* Q, const void* K, const void* V, void* O, float* den,
                   void* ws, size_t ws_bytes, cudaStream_t st) {
    if (!linattn_tc_supported(d)) return CXXATTN_ERR_UNSUPPORTED;
    for (const void* q : {Q, K, V, (const void*)O})
        if (reinterpret_cast<uintptr_t>(q) % 16) return CXXATTN_ERR_ALIGNMENT;
    CUtensorMap tmQ, tmK, tmV;
    const int B = (int)d.B, S = (int)d.S;
    if (!make_tmap_bhsd(&tmQ, Q, B, S, 1, DE, (int64_t)S * DE, DE, DE, CH) ||
        !make_tmap_bhsd(&tmK, K, B, S, 1, DE, (int64_t)S * DE, DE, DE, CH) ||
        !make_tmap_bhsd(&tmV, V, B, S, 1, DE, (int64_t)S * DE, DE, DE, CH))
        return CXXATTN_ERR_CUDA;
    LinFwdParams p;
    p.O = static_cast<__nv_bfloat16*>(O);
    p.den = den;
    p.status = status_word();
    if (p.status == nullptr) return CXXATTN_ERR_CUDA;
    p.B = B;
    p.S = S;
    p.map_elu = d.feature_map == CXXATTN_MAP_ELU1;
    p.eps_in_den = d.eps_in_den;
    // sequence groups when the units alone would leave SMs idle and the caller brought the workspace
    LinGroupPlan plan = linattn_tc_plan(B, S);
    if (plan.G > 1 && (ws == nullptr || ws_bytes < plan.state_bytes || reinterpret_cast<uintptr_t>(ws) % 16))
        plan = LinGroupPlan{1, (S + CH - 1) / CH, 0};
    p.sg = SeqGroups{static_cast<const float*>(ws), plan.G, plan.gc};
    if (plan.G > 1) {
        const int rc = linattn_tc_group_states(0, plan, B, S, p.map_elu, K, V, nullptr, nullptr, static_cast<float*>(ws), st);
        if (rc != CXXATTN_OK) return rc;
    }
    static OncePerDevice attr;
    const int dev = current_device();
    if (attr.pending(dev)) {
        if (cudaFuncSetAttribute(linattn_tc_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES) !=
            cudaSuccess)
            return CXXATTN_ERR_CUDA;
        attr.done(dev);
    }
    linattn_tc_fwd_kernel<<<(unsigned)(B * plan.G), NTHREADS, SMEM_BYTES, st>>>(tmQ, tmK, tmV, p);
    return check_launch();
}

}  // namespace cxxattn
