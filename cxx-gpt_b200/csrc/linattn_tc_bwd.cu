// Causal linear attention backward on the tensor cores (tcgen05 + TMEM + TMA), bf16 tensors with
// fp32 accumulation and fp32 running states, D = E = 64.
//
// Replaces, for dtype BF16, the three serial scans of the reference backward
// (two_stage_cuda::kernel_attn_bwd_step1 / _dQ / _dKdV, src/TwoStage/two_stage_cuda_kernels.cu:
// 1190-1809, and the linear_cuda:: counterparts, src/LinearAttention/linear_cuda_kernels.cu:
// 101-298) with two chunked passes over the sequence, one CTA per batch unit, 128 tokens per chunk.
// Step 1 (dnum = dO/den, dden = -(dO.O)/den) is fused into both passes: the dO tile is rescaled in
// place in shared memory and dden goes into column 0 of a small side tile, so that a bias or a
// rank-one term becomes one more K step of a matrix product:
//
//   pass 1 (chunks ascending, prefix state S = sum phiK (x) [V | 1], as in the forward):
//     W    = dnum V^T + dden 1^T                      masked to s <= t, bf16 -> TMEM (P)
//     dQ'  = [dnum | dden] [S_prev | z_prev]^T + P phiK
//     dQ   = dQ' o phi'(Q)
//   pass 2 (chunks descending, suffix state S* = sum phiQ (x) [dnum | dden]):
//     A^T  = phiK phiQ^T,   W2 = V dnum^T + 1 dden^T   both masked to s >= t, bf16 -> TMEM (P1, P2)
//     dV   = phiK S*_next + P1 dnum
//     dK   = (V S*_next^T + z*_next + P2 phiQ) o phi'(K)
//
// As in the forward, the states stay in TMEM (fp32) for the whole sequence and are copied as bf16
// into shared memory once per chunk to serve as matrix operands.
#include "linattn_tc_common.cuh"
#include <mutex>

namespace cxxattn {
namespace {

using namespace tc;
using namespace lintc;

constexpr int NSTAGE = 2;
constexpr int NTHREADS = 512;  // 4 compute warps, TMA producer, MMA issuer, 8 preparation warps (step 1, maps), 2 idle
constexpr uint32_t TMEM_COLS = 512;

struct LinBwdParams {
    const __nv_bfloat16* Q;  // raw inputs, read row-wise for phi'
    const __nv_bfloat16* K;
    const __nv_bfloat16* O;
    const float* den;
    __nv_bfloat16* dQ;
    __nv_bfloat16* dK;
    __nv_bfloat16* dV;
    int* status;
    int B, S;
    int map_elu;
    SeqGroups sgp;  // prefix group states (dQ pass); G = 1: one CTA per unit
    SeqGroups sgs;  // suffix group states (dK/dV pass)
};

// One gradient row: (acc + bias) * phi'(raw) -> bf16 -> global (128 bytes).  raw == nullptr: no
// phi' factor (pre-mapped features); bias == nullptr: none.
__device__ __forceinline__ void store_grad_row(__nv_bfloat16* dst, const __nv_bfloat16* raw, const uint32_t (&o0)[32],
                                               const uint32_t (&o1)[32], const float* bias) {
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    const uint4* r4 = reinterpret_cast<const uint4*>(raw);
#pragma unroll
    for (int half = 0; half < 2; half++) {
        // the four raw chunks of this half are requested together: one round trip, not four
        uint4 x[4];
        if (raw != nullptr) {
#pragma unroll
            for (int c4 = 0; c4 < 4; c4++) x[c4] = r4[4 * half + c4];
        }
#pragma unroll
        for (int c4 = 0; c4 < 4; c4++) {
            const int ch = 4 * half + c4;
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int col = 8 * ch + i;
                v[i] = __uint_as_float(col < 32 ? o0[col] : o1[col - 32]);
            }
            if (bias != nullptr) {
                const float4 b0 = reinterpret_cast<const float4*>(bias)[2 * ch], b1 = reinterpret_cast<const float4*>(bias)[2 * ch + 1];
                v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w;
                v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
            }
            if (raw != nullptr) {
                v[0] *= dphi1(bf_lo(x[c4].x)); v[1] *= dphi1(bf_hi(x[c4].x));
                v[2] *= dphi1(bf_lo(x[c4].y)); v[3] *= dphi1(bf_hi(x[c4].y));
                v[4] *= dphi1(bf_lo(x[c4].z)); v[5] *= dphi1(bf_hi(x[c4].z));
                v[6] *= dphi1(bf_lo(x[c4].w)); v[7] *= dphi1(bf_hi(x[c4].w));
            }
            d4[ch] = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
        }
    }
}

// ---------------------------------------------------------------------------------------------
// pass 1: dQ
// ---------------------------------------------------------------------------------------------
constexpr uint32_t C1_W = 0, C1_DQ = 128, C1_SX = 192;  // W/P | dQ' | state (80 columns)
// per stage K | V | dO, then ones tile, dden side tile per stage, state operand (2 blocks x 8 KB)
constexpr size_t SMEM1_BYTES = NSTAGE * 3 * TILE_BYTES + (1 + NSTAGE) * TILE_BYTES + 2 * 8192 + 1024;

__global__ void __launch_bounds__(NTHREADS, 1)
linattn_tc_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                         const __grid_constant__ CUtensorMap tmG, LinBwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full[NSTAGE], stage_free[NSTAGE], mapped[NSTAGE], w_full, p_ready, o_full, o_free, s_done, sprev_ready;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    auto sK = [&](int st) { return smem + (st * 3 + 0) * TILE_BYTES; };
    auto sV = [&](int st) { return smem + (st * 3 + 1) * TILE_BYTES; };
    auto sG = [&](int st) { return smem + (st * 3 + 2) * TILE_BYTES; };  // dO, rescaled to dnum in place
    uint8_t* sOnes = smem + NSTAGE * 3 * TILE_BYTES;  // [128][64] bf16, column 0 = 1
    auto sDden = [&](int st) { return sOnes + (1 + st) * TILE_BYTES; };  // [128 tokens][64] bf16, column 0 = dden_t
    uint8_t* sPrev = sOnes + (1 + NSTAGE) * TILE_BYTES;  // block 0: S_prev [64 d][64 e]; block 1: column 0 = z_prev

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int b = blockIdx.x / p.sgp.G, g = blockIdx.x % p.sgp.G;  // batch unit, sequence group
    const int c0 = g * p.sgp.gc;                                    // first chunk of the group
    const int nc = min((p.S + CH - 1) / CH, c0 + p.sgp.gc) - c0;    // chunks of the group
    const Guard guard{&abort_flag, p.status};

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < NSTAGE; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&stage_free[s], 1);
        }
        mbar_init(&w_full, 1);
        mbar_init(&o_full, 1);
        mbar_init(&s_done, 1);
        // one barrier per stage: the two halves of the preparation warps may be a chunk apart
        for (int s = 0; s < NSTAGE; s++) mbar_init(&mapped[s], 8);  // one arrival per preparation warp
        mbar_init(&p_ready, 4);
        mbar_init(&o_free, 4);
        mbar_init(&sprev_ready, 4);
        fence_barrier_init();
    }
    if (warp == 5) tmem_alloc(&tmem_slot, TMEM_COLS);
    for (int i = threadIdx.x; i < ((1 + NSTAGE) * TILE_BYTES + 2 * 8192) / 16; i += NTHREADS)
        reinterpret_cast<uint4*>(sOnes)[i] = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
    if (threadIdx.x < CH)
        *reinterpret_cast<uint16_t*>(sOnes + threadIdx.x * 128 + (threadIdx.x & 7) * 16) = 0x3f80;  // bf16 1.0
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;

    // Register budget (512 threads x 128 at launch): the compute warps hold whole rows, every other
    // warp group gives registers back; 4 x 32 x (208 - 128) <= 12 x 32 x (128 - 96).
    if (warp >= 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");

    if (warp == 4) {
        if (lane == 0) {
            prefetch_tmap(&tmK);
            prefetch_tmap(&tmV);
            prefetch_tmap(&tmG);
            for (int c = 0; c < nc; c++) {
                const int st = c % NSTAGE;
                if (c >= NSTAGE) mbar_wait(&stage_free[st], ((c / NSTAGE) - 1) & 1, guard, 801);
                mbar_expect_tx(&full[st], 3 * TILE_BYTES);
                tma_load_4d(sK(st), &tmK, &full[st], 0, 0, (c0 + c) * CH, b);
                tma_load_4d(sV(st), &tmV, &full[st], 0, 0, (c0 + c) * CH, b);
                tma_load_4d(sG(st), &tmG, &full[st], 0, 0, (c0 + c) * CH, b);
            }
        }
    } else if (warp == 5) {
        // MMA issuer: the whole warp runs the loop (uniform control flow and operands); one elected lane issues
        {
            const uint32_t el = elect_one();
            constexpr uint32_t IDESC_W = idesc_bf16(CH, CH, 0, 0);  // dnum V^T (+ dden 1^T): both K-major
            constexpr uint32_t IDESC_I = idesc_bf16(CH, DE, 0, 0);  // [dnum|dden][S_prev|z]^T: both K-major
            constexpr uint32_t IDESC_P = idesc_bf16(CH, DE, 0, 1);  // P phiK: A in TMEM, B MN-major
            constexpr uint32_t IDESC_S = idesc_bf16(CH, 80, 1, 1);  // phiK^T [V | 1]: both MN-major
            const uint64_t dOnes = smem_desc_sw128(smem_u32(sOnes), 16);
            const uint64_t dPrev0 = smem_desc_sw128(smem_u32(sPrev), 16), dPrev1 = smem_desc_sw128(smem_u32(sPrev) + 8192, 16);
            for (int c = 0; c < nc; c++) {
                const int st = c % NSTAGE;
                const uint64_t dDd = smem_desc_sw128(smem_u32(sDden(st)), 16);
                const uint64_t dG = smem_desc_sw128(smem_u32(sG(st)), 16), dVk = smem_desc_sw128(smem_u32(sV(st)), 16);
                const uint64_t dKm = smem_desc_sw128(smem_u32(sK(st)), 0);
                const uint64_t dV1 = smem_desc_sw128(smem_u32(sV(st)), smem_u32(sOnes) - smem_u32(sV(st)));
                mbar_wait_poll(&mapped[st], (c / NSTAGE) & 1, guard, 811);
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < DE / 16; k++) umma_ss_e(el, tmem + C1_W, dG + 2 * k, dVk + 2 * k, IDESC_W, k > 0);
                umma_ss_e(el, tmem + C1_W, dDd, dOnes, IDESC_W, true);  // + dden_t for every column
                umma_commit_e(el, &w_full);
                mbar_wait_poll(&sprev_ready, c & 1, guard, 812);
                if (c > 0) mbar_wait_poll(&o_free, (c - 1) & 1, guard, 813);
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < DE / 16; k++) umma_ss_e(el, tmem + C1_DQ, dG + 2 * k, dPrev0 + 2 * k, IDESC_I, k > 0);
                umma_ss_e(el, tmem + C1_DQ, dDd, dPrev1, IDESC_I, true);  // + dden_t z_prev
#pragma unroll
                for (int k = 0; k < CH / 16; k++)
                    umma_ss_e(el, tmem + C1_SX, dKm + 128 * k, dV1 + 128 * k, IDESC_S, g > 0 || c > 0 || k > 0);
                umma_commit_e(el, &s_done);
                mbar_wait_poll(&p_ready, c & 1, guard, 814);
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < CH / 16; k++)
                    umma_ts_e(el, tmem + C1_DQ, tmem + C1_W + 8 * k, dKm + 128 * k, IDESC_P, true);
                umma_commit_e(el, &o_full);
                umma_commit_e(el, &stage_free[st]);
            }
        }
    } else if (warp >= 14) {
        // idle warps: they only take part in the register hand-over
    } else if (warp >= 6) {
        // ---------------- preparation warps: step 1 and the feature map, as soon as a chunk has landed ----------------
        // warps 6-9: step 1 on the dO tile; warps 10-13: the feature map of the K tile (a lone warp per
        // scheduler doing both would set the pace of the kernel)
        // The second group also writes the dQ rows, one chunk behind (its warps 10-13 sit on the TMEM
        // lane quarters 2, 3, 0, 1): dQ = dQ' o phi'(Q).
        const int r = ((warp - 6) % 4) * 32 + lane;
        const bool second = warp >= 10;
        const int rq = (warp % 4) * 32 + lane;  // row of this thread's TMEM lane
        const uint32_t lane_q = tmem + (static_cast<uint32_t>((warp % 4) * 32) << 16);
        auto write_dq = [&](int c) {
            mbar_wait(&o_full, c & 1, guard, 824);
            tc_fence_after();
            uint32_t o0[32], o1[32];
            tmem_ld32(lane_q + C1_DQ, o0);
            tmem_ld32(lane_q + C1_DQ + 32, o1);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&o_free);
            const int tok = (c0 + c) * CH + rq;
            const int64_t row = (int64_t)b * p.S + tok;
            if (tok < p.S) store_grad_row(p.dQ + row * DE, p.map_elu ? p.Q + row * DE : nullptr, o0, o1, nullptr);
        };
        for (int k = 0; k < 2 && k < nc; k++)  // the first two chunks' rows: nobody asked for them yet
            if ((c0 + k) * CH + r < p.S) prefetch_row((second ? p.Q : p.O) + ((int64_t)b * p.S + (c0 + k) * CH + r) * DE);
        for (int c = 0; c < nc; c++) {
            const int st = c % NSTAGE;
            const int tok = (c0 + c) * CH + r;
            const bool ok = tok < p.S;
            const int64_t row = (int64_t)b * p.S + tok;
            const float den = (!second && ok) ? p.den[row] : 1.f;
            if (tok + 2 * CH < p.S)  // the rows step 1 / write_dq will read two chunks from now
                prefetch_row((second ? p.Q : p.O) + (row + 2 * CH) * DE);
            mbar_wait(&full[st], (c / NSTAGE) & 1, guard, 821);
            if (!second)
                step1_row(sG(st) + r * 128, p.O + row * DE, den, ok, r & 7, sDden(st) + r * 128 + (r & 7) * 16);
            else if (p.map_elu)
                map_row(sK(st) + r * 128, ok, true, r & 7);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&mapped[st]);
            if (second && c > 0) write_dq(c - 1);
        }
        if (second) write_dq(nc - 1);
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
        const int r = warp * 32 + lane;
        const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
        // a later sequence group starts from the sum of the states of the groups before it
        if (g > 0) init_state_row(p.sgp, b, 0, g, r, lane_base + C1_SX, sPrev);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sprev_ready);
        for (int c = 0; c < nc; c++) {
            // W -> mask s <= t -> bf16 P, written over the first 64 columns of W (each thread only
            // touches its own TMEM lane and has its whole row in registers before it stores)
            mbar_wait(&w_full, c & 1, guard, 822);
            tc_fence_after();
            uint32_t pk[64];
#pragma unroll
            for (int h = 0; h < 2; h++) {
                uint32_t v0[32], v1[32];
                const bool need0 = 64 * h <= warp * 32 + 31, need1 = 64 * h + 32 <= warp * 32 + 31;
                if (need0) tmem_ld32(lane_base + C1_W + 64 * h, v0);
                if (need1) tmem_ld32(lane_base + C1_W + 64 * h + 32, v1);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const float a0 = (need0 && 64 * h + i <= r) ? __uint_as_float(v0[i]) : 0.f;
                    const float a1 = (need0 && 64 * h + i + 1 <= r) ? __uint_as_float(v0[i + 1]) : 0.f;
                    const float b0 = (need1 && 64 * h + 32 + i <= r) ? __uint_as_float(v1[i]) : 0.f;
                    const float b1 = (need1 && 64 * h + 32 + i + 1 <= r) ? __uint_as_float(v1[i + 1]) : 0.f;
                    pk[32 * h + i / 2] = pack_bf16(a0, a1);
                    pk[32 * h + 16 + i / 2] = pack_bf16(b0, b1);
                }
            }
            tmem_st32(lane_base + C1_W, reinterpret_cast<const uint32_t(&)[32]>(pk[0]));
            tmem_st32(lane_base + C1_W + 32, reinterpret_cast<const uint32_t(&)[32]>(pk[32]));
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready);

            mbar_wait(&s_done, c & 1, guard, 823);
            tc_fence_after();
            if (c + 1 < nc) {
                state_to_smem(lane_base + C1_SX, sPrev, r);
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

// ---------------------------------------------------------------------------------------------
// pass 2: dK, dV (chunks in descending order)
// ---------------------------------------------------------------------------------------------
constexpr uint32_t C2_AT = 0, C2_W = 128, C2_DV = 256, C2_DK = 320, C2_SX = 384;
// per stage Q | K | V | dO, then ones tile, dden side tile, state operand (2 blocks x 8 KB)
constexpr size_t SMEM2_BYTES = NSTAGE * 4 * TILE_BYTES + (1 + NSTAGE) * TILE_BYTES + 2 * 8192 + 1024;

__global__ void __launch_bounds__(NTHREADS, 1)
linattn_tc_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                           const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmG,
                           LinBwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full[NSTAGE], stage_free[NSTAGE], mapped[NSTAGE], aw_full, p_ready, o_full, o_free, s_done, snext_ready;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ __align__(16) float zstar[3][DE];  // z*_next in fp32, added to dK; three buffers: written in iteration n for n + 1,
                                    // read by the output warps until iteration n + 2 is under way

    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    auto sQ = [&](int st) { return smem + (st * 4 + 0) * TILE_BYTES; };
    auto sK = [&](int st) { return smem + (st * 4 + 1) * TILE_BYTES; };
    auto sV = [&](int st) { return smem + (st * 4 + 2) * TILE_BYTES; };
    auto sG = [&](int st) { return smem + (st * 4 + 3) * TILE_BYTES; };
    uint8_t* sOnes = smem + NSTAGE * 4 * TILE_BYTES;
    auto sDden = [&](int st) { return sOnes + (1 + st) * TILE_BYTES; };
    uint8_t* sNext = sOnes + (1 + NSTAGE) * TILE_BYTES;  // block 0: S*_next [64 d][64 e]; block 1: column 0 = z*_next

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int b = blockIdx.x / p.sgs.G, g = blockIdx.x % p.sgs.G;  // batch unit, sequence group
    const int c0 = g * p.sgs.gc;                                    // first chunk of the group
    const int nc = min((p.S + CH - 1) / CH, c0 + p.sgs.gc) - c0;    // chunks of the group
    const bool seeded = g + 1 < p.sgs.G;                            // later groups exist: start from their states
    const Guard guard{&abort_flag, p.status};

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < NSTAGE; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&stage_free[s], 1);
        }
        mbar_init(&aw_full, 1);
        mbar_init(&o_full, 1);
        mbar_init(&s_done, 1);
        // one barrier per stage: the two halves of the preparation warps may be a chunk apart
        for (int s = 0; s < NSTAGE; s++) mbar_init(&mapped[s], 8);  // one arrival per preparation warp
        mbar_init(&p_ready, 4);
        mbar_init(&o_free, 4);
        mbar_init(&snext_ready, 4);
        fence_barrier_init();
    }
    if (warp == 5) tmem_alloc(&tmem_slot, TMEM_COLS);
    for (int i = threadIdx.x; i < ((1 + NSTAGE) * TILE_BYTES + 2 * 8192) / 16; i += NTHREADS)
        reinterpret_cast<uint4*>(sOnes)[i] = make_uint4(0u, 0u, 0u, 0u);
    if (threadIdx.x < DE) zstar[0][threadIdx.x] = 0.f;
    __syncthreads();
    if (threadIdx.x < CH)
        *reinterpret_cast<uint16_t*>(sOnes + threadIdx.x * 128 + (threadIdx.x & 7) * 16) = 0x3f80;  // bf16 1.0
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;

    // Register budget as in the first pass.
    if (warp >= 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");

    // iteration n = 0 .. nc-1 handles chunk c = c0 + nc-1-n
    if (warp == 4) {
        if (lane == 0) {
            prefetch_tmap(&tmQ);
            prefetch_tmap(&tmK);
            prefetch_tmap(&tmV);
            prefetch_tmap(&tmG);
            for (int n = 0; n < nc; n++) {
                const int st = n % NSTAGE, c = c0 + nc - 1 - n;
                if (n >= NSTAGE) mbar_wait(&stage_free[st], ((n / NSTAGE) - 1) & 1, guard, 901);
                mbar_expect_tx(&full[st], 4 * TILE_BYTES);
                tma_load_4d(sQ(st), &tmQ, &full[st], 0, 0, c * CH, b);
                tma_load_4d(sK(st), &tmK, &full[st], 0, 0, c * CH, b);
                tma_load_4d(sV(st), &tmV, &full[st], 0, 0, c * CH, b);
                tma_load_4d(sG(st), &tmG, &full[st], 0, 0, c * CH, b);
            }
        }
    } else if (warp == 5) {
        // MMA issuer: the whole warp runs the loop (uniform control flow and operands); one elected lane issues
        {
            const uint32_t el = elect_one();
            constexpr uint32_t IDESC_KK = idesc_bf16(CH, CH, 0, 0);  // A^T and W2: both operands K-major
            constexpr uint32_t IDESC_KN = idesc_bf16(CH, DE, 0, 1);  // A K-major (or TMEM), B MN-major
            constexpr uint32_t IDESC_K2 = idesc_bf16(CH, DE, 0, 0);  // V S*^T: both K-major
            constexpr uint32_t IDESC_S = idesc_bf16(CH, 80, 1, 1);   // phiQ^T [dnum | dden]: both MN-major
            const uint64_t dOnes = smem_desc_sw128(smem_u32(sOnes), 16);
            const uint64_t dNextK = smem_desc_sw128(smem_u32(sNext), 16);  // rows d, K = e   (for V S*^T)
            const uint64_t dNextM = smem_desc_sw128(smem_u32(sNext), 0);   // rows = K = d, N = e (for phiK S*)
            for (int n = 0; n < nc; n++) {
                const int st = n % NSTAGE;
                const uint64_t dQk = smem_desc_sw128(smem_u32(sQ(st)), 16), dKk = smem_desc_sw128(smem_u32(sK(st)), 16);
                const uint64_t dVk = smem_desc_sw128(smem_u32(sV(st)), 16), dGk = smem_desc_sw128(smem_u32(sG(st)), 16);
                const uint64_t dQm = smem_desc_sw128(smem_u32(sQ(st)), 0);  // phiQ MN-major (A of the state, B of dK)
                const uint64_t dGm = smem_desc_sw128(smem_u32(sG(st)), 0);  // dnum MN-major (B of dV)
                const uint64_t dDd = smem_desc_sw128(smem_u32(sDden(st)), 16);
                const uint64_t dG1 = smem_desc_sw128(smem_u32(sG(st)), smem_u32(sDden(st)) - smem_u32(sG(st)));  // [dnum | dden]
                mbar_wait_poll(&mapped[st], (n / NSTAGE) & 1, guard, 911);
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < DE / 16; k++) umma_ss_e(el, tmem + C2_AT, dKk + 2 * k, dQk + 2 * k, IDESC_KK, k > 0);
#pragma unroll
                for (int k = 0; k < DE / 16; k++) umma_ss_e(el, tmem + C2_W, dVk + 2 * k, dGk + 2 * k, IDESC_KK, k > 0);
                umma_ss_e(el, tmem + C2_W, dOnes, dDd, IDESC_KK, true);  // + dden_s for every row
                umma_commit_e(el, &aw_full);
                mbar_wait_poll(&snext_ready, n & 1, guard, 912);
                if (n > 0) mbar_wait_poll(&o_free, (n - 1) & 1, guard, 913);
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < DE / 16; k++)  // dV' = phiK S*_next
                    umma_ss_e(el, tmem + C2_DV, dKk + 2 * k, dNextM + 128 * k, IDESC_KN, k > 0);
#pragma unroll
                for (int k = 0; k < DE / 16; k++)  // dK' = V S*_next^T
                    umma_ss_e(el, tmem + C2_DK, dVk + 2 * k, dNextK + 2 * k, IDESC_K2, k > 0);
#pragma unroll
                for (int k = 0; k < CH / 16; k++)  // S* += phiQ^T [dnum | dden]
                    umma_ss_e(el, tmem + C2_SX, dQm + 128 * k, dG1 + 128 * k, IDESC_S, seeded || n > 0 || k > 0);
                umma_commit_e(el, &s_done);
                mbar_wait_poll(&p_ready, n & 1, guard, 914);
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < CH / 16; k++)  // dV' += P1 dnum
                    umma_ts_e(el, tmem + C2_DV, tmem + C2_AT + 8 * k, dGm + 128 * k, IDESC_KN, true);
#pragma unroll
                for (int k = 0; k < CH / 16; k++)  // dK' += P2 phiQ
                    umma_ts_e(el, tmem + C2_DK, tmem + C2_W + 8 * k, dQm + 128 * k, IDESC_KN, true);
                umma_commit_e(el, &o_full);
                umma_commit_e(el, &stage_free[st]);
            }
        }
    } else if (warp >= 14) {
        // idle warps: they only take part in the register hand-over
    } else if (warp >= 6) {
        // ---------------- preparation warps: step 1 and the feature maps of Q and K ----------------
        // warps 6-9: step 1 on the dO tile and the map of the Q tile; warps 10-13: the map of the K tile
        // The second group also writes the dV and dK rows, one chunk behind (its warps 10-13 sit on the
        // TMEM lane quarters 2, 3, 0, 1): dV = dV', dK = (dK' + z*_next) o phi'(K).
        const int r = ((warp - 6) % 4) * 32 + lane;
        const bool second = warp >= 10;
        const int rq = (warp % 4) * 32 + lane;  // row of this thread's TMEM lane
        const uint32_t lane_q = tmem + (static_cast<uint32_t>((warp % 4) * 32) << 16);
        auto write_dkdv = [&](int n) {
            const int tok = (c0 + nc - 1 - n) * CH + rq;
            const bool valid = tok < p.S;
            const int64_t row = (int64_t)b * p.S + tok;
            mbar_wait(&o_full, n & 1, guard, 924);
            tc_fence_after();
            uint32_t o0[32], o1[32];
            tmem_ld32(lane_q + C2_DV, o0);
            tmem_ld32(lane_q + C2_DV + 32, o1);
            tmem_ld_wait();
            if (valid) store_grad_row(p.dV + row * DE, nullptr, o0, o1, nullptr);
            tmem_ld32(lane_q + C2_DK, o0);
            tmem_ld32(lane_q + C2_DK + 32, o1);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&o_free);
            if (valid) store_grad_row(p.dK + row * DE, p.map_elu ? p.K + row * DE : nullptr, o0, o1, zstar[n % 3]);
        };
        for (int k = 0; k < 2 && k < nc; k++)  // the first two chunks' rows: nobody asked for them yet
            if ((c0 + nc - 1 - k) * CH + r < p.S)
                prefetch_row((second ? p.K : p.O) + ((int64_t)b * p.S + (c0 + nc - 1 - k) * CH + r) * DE);
        for (int n = 0; n < nc; n++) {
            const int st = n % NSTAGE, c = c0 + nc - 1 - n;
            const int tok = c * CH + r;
            const bool ok = tok < p.S;
            const int64_t row = (int64_t)b * p.S + tok;
            const float den = (!second && ok) ? p.den[row] : 1.f;
            if (tok >= 2 * CH)  // the rows step 1 / write_dkdv will read two chunks from now
                prefetch_row((second ? p.K : p.O) + (row - 2 * CH) * DE);
            mbar_wait(&full[st], (n / NSTAGE) & 1, guard, 921);
            if (!second) {
                step1_row(sG(st) + r * 128, p.O + row * DE, den, ok, r & 7, sDden(st) + r * 128 + (r & 7) * 16);
                if (p.map_elu) map_row(sQ(st) + r * 128, ok, true, r & 7);
            } else if (p.map_elu) {
                map_row(sK(st) + r * 128, ok, true, r & 7);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&mapped[st]);
            if (second && n > 0) write_dkdv(n - 1);
        }
        if (second) write_dkdv(nc - 1);
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
        const int r = warp * 32 + lane;
        const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
        // an earlier sequence group starts from the sum of the states of the groups after it
        if (seeded) init_state_row(p.sgs, b, g + 1, p.sgs.G, r, lane_base + C2_SX, sNext, zstar[0]);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&snext_ready);
        for (int n = 0; n < nc; n++) {
            // A^T and W2 -> mask s >= t -> bf16 P1, P2 (each over the first 64 columns of its source)
            mbar_wait(&aw_full, n & 1, guard, 922);
            tc_fence_after();
#pragma unroll
            for (int m = 0; m < 2; m++) {
                const uint32_t src = lane_base + (m == 0 ? C2_AT : C2_W);
                uint32_t pk[64];
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    uint32_t v0[32], v1[32];
                    // a 32-wide column block entirely below this warp's first row is all masked
                    const bool need0 = 64 * h + 31 >= warp * 32, need1 = 64 * h + 63 >= warp * 32;
                    if (need0) tmem_ld32(src + 64 * h, v0);
                    if (need1) tmem_ld32(src + 64 * h + 32, v1);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float a0 = (need0 && 64 * h + i >= r) ? __uint_as_float(v0[i]) : 0.f;
                        const float a1 = (need0 && 64 * h + i + 1 >= r) ? __uint_as_float(v0[i + 1]) : 0.f;
                        const float b0 = (need1 && 64 * h + 32 + i >= r) ? __uint_as_float(v1[i]) : 0.f;
                        const float b1 = (need1 && 64 * h + 32 + i + 1 >= r) ? __uint_as_float(v1[i + 1]) : 0.f;
                        pk[32 * h + i / 2] = pack_bf16(a0, a1);
                        pk[32 * h + 16 + i / 2] = pack_bf16(b0, b1);
                    }
                }
                tmem_st32(src, reinterpret_cast<const uint32_t(&)[32]>(pk[0]));
                tmem_st32(src + 32, reinterpret_cast<const uint32_t(&)[32]>(pk[32]));
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready);

            // state after this chunk -> operand of the next (earlier) chunk, then step 1 / maps of that
            // chunk, so that its products start while this chunk's outputs are written.  z* goes to the
            // other half of `zstar`: the epilogue below still reads this iteration's half.
            mbar_wait(&s_done, n & 1, guard, 923);
            tc_fence_after();
            if (n + 1 < nc) {
                state_to_smem(lane_base + C2_SX, sNext, r, zstar[(n + 1) % 3]);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&snext_ready);
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

namespace {
// A side stream per device for the suffix-state pre-pass.  Only the dK/dV pass needs that state, so
// the pre-pass runs beside the prefix pre-pass and the dQ pass, in the SMs their last waves leave
// idle.  Fork and join are events on the caller's stream, so its order is kept.  Stream and events
// are shared by all calls on a device: enqueueing is serialised by g_side_mutex, and a call whose
// stream is being captured does not use them at all (work of another thread's uncaptured call must
// not land in that capture), it runs the pre-pass in line.  Callers of side_stream() hold the mutex.
struct SideStream {
    cudaStream_t stream = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
    int state = 0;  // 0 not tried, 1 usable, -1 unavailable
};
std::mutex g_side_mutex;
SideStream* side_stream(int dev, cudaStream_t caller) {
    static SideStream tab[kMaxDevices];
    if (dev < 0 || option(CXXATTN_OPT_LIN_SIDE_STREAM) == 0) return nullptr;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(caller, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) return nullptr;
    SideStream& s = tab[dev];
    if (s.state == 0)
        s.state = cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking) == cudaSuccess &&
                          cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming) == cudaSuccess &&
                          cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming) == cudaSuccess
                      ? 1
                      : -1;
    return s.state == 1 ? &s : nullptr;
}
}  // namespace

int linattn_tc_bwd(const cxxattn_lin_desc& d, const void* Q, const void* K, const void* V, const void* O,
                   const void* dO, const float* den, void* dQ, void* dK, void* dV, void* ws, size_t ws_bytes,
                   cudaStream_t st) {
    if (!linattn_tc_supported(d)) return CXXATTN_ERR_UNSUPPORTED;
    for (const void* q : {Q, K, V, O, dO, (const void*)dQ, (const void*)dK, (const void*)dV})
        if (reinterpret_cast<uintptr_t>(q) % 16) return CXXATTN_ERR_ALIGNMENT;
    const int B = (int)d.B, S = (int)d.S;
    CUtensorMap tmQ, tmK, tmV, tmG;
    if (!make_tmap_bhsd(&tmQ, Q, B, S, 1, DE, (int64_t)S * DE, DE, DE, CH) ||
        !make_tmap_bhsd(&tmK, K, B, S, 1, DE, (int64_t)S * DE, DE, DE, CH) ||
        !make_tmap_bhsd(&tmV, V, B, S, 1, DE, (int64_t)S * DE, DE, DE, CH) ||
        !make_tmap_bhsd(&tmG, dO, B, S, 1, DE, (int64_t)S * DE, DE, DE, CH))
        return CXXATTN_ERR_CUDA;
    LinBwdParams p;
    p.Q = static_cast<const __nv_bfloat16*>(Q);
    p.K = static_cast<const __nv_bfloat16*>(K);
    p.O = static_cast<const __nv_bfloat16*>(O);
    p.den = den;
    p.dQ = static_cast<__nv_bfloat16*>(dQ);
    p.dK = static_cast<__nv_bfloat16*>(dK);
    p.dV = static_cast<__nv_bfloat16*>(dV);
    p.status = status_word();
    if (p.status == nullptr) return CXXATTN_ERR_CUDA;
    p.B = B;
    p.S = S;
    p.map_elu = d.feature_map == CXXATTN_MAP_ELU1;
    // sequence groups when the units alone would leave SMs idle and the caller brought the workspace
    LinGroupPlan plan = linattn_tc_plan(B, S);
    if (plan.G > 1 && (ws == nullptr || ws_bytes < 2 * plan.state_bytes || reinterpret_cast<uintptr_t>(ws) % 16))
        plan = LinGroupPlan{1, (S + CH - 1) / CH, 0};
    float* gsp = static_cast<float*>(ws);
    float* gss = plan.G > 1 ? reinterpret_cast<float*>(static_cast<char*>(ws) + plan.state_bytes) : nullptr;
    p.sgp = SeqGroups{gsp, plan.G, plan.gc};
    p.sgs = SeqGroups{gss, plan.G, plan.gc};
    const int dev = current_device();
    static OncePerDevice attr;
    if (attr.pending(dev)) {
        if (cudaFuncSetAttribute(linattn_tc_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)SMEM1_BYTES) != cudaSuccess ||
            cudaFuncSetAttribute(linattn_tc_bwd_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)SMEM2_BYTES) != cudaSuccess)
            return CXXATTN_ERR_CUDA;
        attr.done(dev);
    }
    std::unique_lock<std::mutex> side_lock(g_side_mutex, std::defer_lock);
    SideStream* side = nullptr;
    int rc = CXXATTN_OK;
    if (plan.G > 1) {
        side_lock.lock();
        side = side_stream(dev, st);
        if (side && (cudaEventRecord(side->fork, st) != cudaSuccess ||
                     cudaStreamWaitEvent(side->stream, side->fork, 0) != cudaSuccess))
            side = nullptr;
        rc = linattn_tc_group_states(0, plan, B, S, p.map_elu, K, V, nullptr, nullptr, gsp, st);
        if (rc == CXXATTN_OK)
            rc = linattn_tc_group_states(1, plan, B, S, p.map_elu, Q, dO, O, den, gss, side ? side->stream : st);
        if (side && cudaEventRecord(side->join, side->stream) != cudaSuccess) {
            // nothing can be joined through the event: drain the side stream instead, once
            cudaStreamSynchronize(side->stream);
            side = nullptr;
            if (rc == CXXATTN_OK) rc = CXXATTN_ERR_CUDA;
        }
    }
    if (rc == CXXATTN_OK) {
        linattn_tc_bwd_dq_kernel<<<(unsigned)(B * plan.G), NTHREADS, SMEM1_BYTES, st>>>(tmK, tmV, tmG, p);
        rc = check_launch();
    }
    // once forked, the side stream is joined on every path out of this function, failures included
    if (side && cudaStreamWaitEvent(st, side->join, 0) != cudaSuccess && rc == CXXATTN_OK) rc = CXXATTN_ERR_CUDA;
    if (rc != CXXATTN_OK) return rc;
    linattn_tc_bwd_dkdv_kernel<<<(unsigned)(B * plan.G), NTHREADS, SMEM2_BYTES, st>>>(tmQ, tmK, tmV, tmG, p);
    return check_launch();
}

}  // namespace cxxattn
