// Causal softmax MHA forward on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), bf16
// operands, fp32 accumulation and softmax, head dimension 64.
//
// Replaces two_stage_cuda::fused_mha_fwd (src/TwoStage/two_stage_cuda_kernels.cu:54-326) for
// dtype BF16.  Where the reference gives one warp one query row and walks the keys one at a
// time with shuffle reductions, this kernel is a FlashAttention pipeline:
//
//   CTA  = persistent, one per SM; a work item = 2 query tiles of 128 rows (rows q0 .. q0+255 of one
//          (batch, head)); 18 warps:
//          warps 0-7   softmax group of tile 0: warp w holds the 32 rows of TMEM lane quarter w % 4 and
//                      the half w / 4 of the 128 key columns, so a query row is shared by two threads
//                      of two warps (they exchange the row maximum through shared memory each step)
//          warps 8-15  softmax group of tile 1, likewise
//          warp  16    TMA producer: Q of the item (two buffers, so the next item's Q is already
//                      there), then K/V tiles of 128 keys through a 3-stage ring
//          warp  17    MMA issuer (the warp runs uniformly, one elected lane issues) and TMEM owner
//          Four softmax warps per scheduler: with a whole row per thread (two warps per scheduler) the
//          exponent unit was 64 % busy and every instruction waited 2.2 cycles on average for a
//          fixed-latency result that no other warp could cover.
//   TMEM = S0 | S1 (128 fp32 columns each) | O0 | O1 (64 columns each) | P0 | P1 (128 bf16 = 64
//          columns each): all 512 columns.  P feeds the PV product directly from TMEM.
//
//   per KV tile j:   S_t = Q_t K_j^T   (SS MMA, 128x128x64)      -> softmax group t
//                    P_t = exp2(c*S_t - m_t), l_t += rowsum      -> TMEM (bf16)
//                    O_t += P_t V_j    (TS MMA, 128x64x128)
//
// A softmax thread pulls its half row of scores (64 values) into registers and releases the score
// columns at once; since P has columns of its own, the MMA warp can then issue S_t(j+1) while the
// exponentials of step j are still running, and a softmax group never waits for its next scores.  KV tiles above the causal diagonal
// are never loaded; only the diagonal tile is masked.  A row's running maximum is only raised
// when it grows by more than 8 (in log2 units), so the rescaling of O in TMEM is rare.
#include <algorithm>

#include "internal.cuh"
#include "tc_common.cuh"

namespace cxxattn {
namespace {

using namespace tc;

constexpr int BM = 128;       // rows per query tile
constexpr int BN = 128;       // keys per KV tile
constexpr int DH = 64;        // head dimension
constexpr int STAGES = 3;
constexpr int TILE_BYTES = BM * DH * 2;  // 16 KB: one 128 x 64 bf16 tile
constexpr int NTHREADS = 576;  // 18 warps: 16 softmax, producer, MMA issuer; 112 registers each fill the register file
constexpr int W_PROD = 16, W_MMA = 17;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t COL_S = 0, COL_O = 256, COL_P = 384;
constexpr size_t SMEM_BYTES = (4 + 2 * STAGES) * TILE_BYTES + 1024;  // Q x2 (2 tiles each), K/V ring, alignment slack

struct FwdParams {
    __nv_bfloat16* O;
    float* lse;  // may be null
    int* status;
    int B, S, H;
    int64_t sb, ss, sh;
    float scale_log2;  // 1/sqrt(Dh) * log2(e)
};

// One work item = one pair of query tiles of one (batch, head).  Items are numbered heavy first (the
// last pair of a sequence meets every KV tile); the persistent CTA j of P takes item j of the first
// round, P-1-j of the second, j of the third, ..., so that every CTA gets a similar mix.  All roles of
// a CTA walk the same list, and every ring of barriers keeps its phase across item borders, so the
// next item's Q load and first scores overlap the last steps and the epilogue of the current one.
struct Item {
    int q0, bh, n0, nkv;
    bool has_t1;
};
__device__ __forceinline__ bool get_item(int round, int npairs, int nbh, int S, Item& w) {
    const int P = gridDim.x, j = blockIdx.x;
    const int id = round * P + ((round & 1) ? P - 1 - j : j);
    if (id >= npairs * nbh) return false;
    const int pair = npairs - 1 - id / nbh;
    w.bh = id % nbh;
    w.q0 = pair * 2 * BM;
    w.has_t1 = w.q0 + BM < S;
    w.n0 = w.q0 / BN;  // diagonal KV tile of query tile 0
    w.nkv = w.has_t1 ? w.n0 + 2 : w.n0 + 1;
    return true;
}

// The exponent unit (16 ex2 per clock and SM) is the busiest pipe of this kernel at head dimension 64, so
// part of the exponentials is computed on the FMA pipe instead: of every POLY_PERIOD groups of four
// scores, POLY_PAIRS have their second pair evaluated by ex2_poly2.
constexpr int POLY_PERIOD = 2, POLY_PAIRS = 1;
// 2^x for two arguments x <= 0 without the exponent unit: x = n + f with n = round(x) (the 1.5*2^23 trick
// leaves n in the low mantissa bits), 2^f by a cubic on [-0.5, 0.5] (relative error 7.5e-5, well inside the
// bf16 rounding of P), and n added into the exponent field.  Arguments below -125 (masked scores are -inf)
// give 2^-125 instead of 0: 1e-38 of a row's largest term.
__device__ __forceinline__ void ex2_poly2(float& x0, float& x1) {
    const float MAGIC = 12582912.0f;
    const uint64_t x2 = pack2(fmaxf(x0, -125.0f), fmaxf(x1, -125.0f));
    const uint64_t xf2 = add2(x2, pack2(MAGIC, MAGIC));
    const uint64_t n2 = add2(xf2, pack2(-MAGIC, -MAGIC));
    const uint64_t f2 = fma2(n2, pack2(-1.0f, -1.0f), x2);
    uint64_t p2 = fma2(f2, pack2(0.0551716685f, 0.0551716685f), pack2(0.2426111251f, 0.2426111251f));
    p2 = fma2(p2, f2, pack2(0.6932609677f, 0.6932609677f));
    p2 = fma2(p2, f2, pack2(0.9999280572f, 0.9999280572f));
    float p0, p1, n0, n1;
    unpack2(p2, p0, p1);
    unpack2(xf2, n0, n1);
    x0 = __uint_as_float(__float_as_uint(p0) + (__float_as_uint(n0) << 23));
    x1 = __uint_as_float(__float_as_uint(p1) + (__float_as_uint(n1) << 23));
}

// LATE_WAIT: the softmax warps form the first half of a step's exponentials before they wait for
// the PV product of the step before (the default: 4 to 11 % faster than waiting first at every
// sequence length measured, 1024 to 16384; CXXATTN_OPT_FWD_LATE_WAIT = 0 selects the other form).
template <bool LATE_WAIT>
__global__ void __launch_bounds__(NTHREADS, 1)
mha_tc_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, FwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t q_full[2], q_free[2], k_full[STAGES], v_full[STAGES], kv_empty[STAGES], s_full[2], s_free[2],
        p_full[2], pv_done[2], o_free[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    // what the two threads of a row tell each other: the maximum of their half of the scores (two slots,
    // by step parity) and, at the end of an item, their half of the row sum
    __shared__ float xmax[2][2][2][BM], xsum[2][2][BM];

    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;                                // 2 buffers x 2 tiles
    uint8_t* sK = smem + 4 * TILE_BYTES;               // STAGES tiles
    uint8_t* sV = smem + (4 + STAGES) * TILE_BYTES;    // STAGES tiles

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int npairs = (p.S + 2 * BM - 1) / (2 * BM);
    const int nbh = p.B * p.H;
    const Guard guard{&abort_flag, p.status};

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < 2; s++) {
            mbar_init(&q_full[s], 1);
            mbar_init(&q_free[s], 1);
        }
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&k_full[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&kv_empty[s], 1);
        }
        for (int t = 0; t < 2; t++) {
            mbar_init(&s_full[t], 1);
            mbar_init(&s_free[t], 8);  // one arrival per softmax warp
            mbar_init(&p_full[t], 8);
            mbar_init(&pv_done[t], 1);
            mbar_init(&o_free[t], 8);  // the output accumulator has been read out (once per item)
        }
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
            prefetch_tmap(&tmQ);
            prefetch_tmap(&tmK);
            prefetch_tmap(&tmV);
            int J = 0;  // KV steps so far, over all items: the ring stage is J % STAGES
            Item w;
            for (int k = 0; get_item(k, npairs, nbh, p.S, w); k++) {
                const int b = w.bh / p.H, h = w.bh % p.H, qb = k & 1;
                // the scores of the item two before have read this Q buffer
                if (k >= 2) mbar_wait(&q_free[qb], ((k >> 1) - 1) & 1, guard, 102);
                mbar_expect_tx(&q_full[qb], 2 * TILE_BYTES);
                tma_load_4d(sQ + qb * 2 * TILE_BYTES, &tmQ, &q_full[qb], 0, h, w.q0, b);
                tma_load_4d(sQ + (qb * 2 + 1) * TILE_BYTES, &tmQ, &q_full[qb], 0, h, w.q0 + BM, b);
                for (int j = 0; j < w.nkv; j++, J++) {
                    const int s = J % STAGES;
                    if (J >= STAGES) mbar_wait(&kv_empty[s], ((J / STAGES) - 1) & 1, guard, 101);
                    mbar_expect_tx(&k_full[s], TILE_BYTES);
                    tma_load_4d(sK + s * TILE_BYTES, &tmK, &k_full[s], 0, h, j * BN, b);
                    mbar_expect_tx(&v_full[s], TILE_BYTES);
                    tma_load_4d(sV + s * TILE_BYTES, &tmV, &v_full[s], 0, h, j * BN, b);
                }
            }
        }
    } else if (warp == W_MMA) {
        // ---------------- MMA issuer ----------------
        // the whole warp runs the loop (uniform control flow and operands); one elected lane issues
        const uint32_t el = elect_one();
        constexpr uint32_t IDESC_S = idesc_bf16(BM, BN, 0, 0);  // Q, K both K-major
        constexpr uint32_t IDESC_O = idesc_bf16(BM, DH, 0, 1);  // P from TMEM, V MN-major
        // Descriptors are built once; a K step or a ring stage only adds a constant to the
        // 14-bit start-address field (units of 16 bytes), which cannot carry out of it.
        const uint64_t dQ0 = smem_desc_sw128(smem_u32(sQ), 16);
        const uint64_t dK0 = smem_desc_sw128(smem_u32(sK), 16);
        const uint64_t dV0 = smem_desc_sw128(smem_u32(sV), 0);
        constexpr uint64_t TILE16 = TILE_BYTES >> 4;
        auto issue_s = [&](int t, int s, int qb) {
            const uint64_t qd = dQ0 + (qb * 2 + t) * TILE16, kd = dK0 + s * TILE16;
            const uint32_t d = tmem + COL_S + t * BN;
#pragma unroll
            for (int kk = 0; kk < DH / 16; kk++) umma_ss_e(el, d, qd + 2 * kk, kd + 2 * kk, IDESC_S, kk > 0);
            umma_commit_e(el, &s_full[t]);
        };
        auto issue_pv = [&](int t, int s, bool acc) {
            const uint64_t vd = dV0 + s * TILE16;
            const uint32_t d = tmem + COL_O + t * DH, a = tmem + COL_P + t * 64;
            umma_ts_e(el, d, a, vd, IDESC_O, acc);
#pragma unroll
            for (int kk = 1; kk < BN / 16; kk++) umma_ts_e(el, d, a + 8 * kk, vd + 128 * kk, IDESC_O, true);
        };
        int J = 0;             // KV steps so far (ring position)
        int c0 = 0, c1 = 0;    // steps so far of query tile 0 / 1 (phases of their barriers)
        int i0 = 0, i1 = 0;    // items so far in which tile 0 / 1 took part
        Item w;
        for (int k = 0; get_item(k, npairs, nbh, p.S, w); k++) {
            const int qb = k & 1;
            const int last0 = w.n0;  // last KV tile of query tile 0; tile 1 runs to nkv - 1
            mbar_wait_poll(&q_full[qb], (k >> 1) & 1, guard, 201);
            mbar_wait_poll(&k_full[J % STAGES], (J / STAGES) & 1, guard, 202);
            // first scores of the item, as soon as the last ones of the item before have been read
            if (c0 > 0) mbar_wait_poll(&s_free[0], (c0 - 1) & 1, guard, 209);
            tc_fence_after();
            issue_s(0, J % STAGES, qb);
            if (w.has_t1) {
                if (c1 > 0) mbar_wait_poll(&s_free[1], (c1 - 1) & 1, guard, 210);
                tc_fence_after();
                issue_s(1, J % STAGES, qb);
            }
            if (w.nkv == 1) umma_commit_e(el, &q_free[qb]);
            for (int j = 0; j < w.nkv; j++) {
                const int s = (J + j) % STAGES, sn = (J + j + 1) % STAGES;
                if (j + 1 < w.nkv) {
                    // next scores of both tiles as soon as this step's have been read into registers
                    mbar_wait_poll(&k_full[sn], ((J + j + 1) / STAGES) & 1, guard, 205);
                    if (j + 1 <= last0) {
                        mbar_wait_poll(&s_free[0], (c0 + j) & 1, guard, 207);
                        tc_fence_after();
                        issue_s(0, sn, qb);
                    }
                    if (w.has_t1) {
                        mbar_wait_poll(&s_free[1], (c1 + j) & 1, guard, 208);
                        tc_fence_after();
                        issue_s(1, sn, qb);
                    }
                    if (j + 2 == w.nkv) umma_commit_e(el, &q_free[qb]);  // the item's last scores are issued
                }
                mbar_wait_poll(&v_full[s], ((J + j) / STAGES) & 1, guard, 203);
                if (j <= last0) {
                    mbar_wait_poll(&p_full[0], (c0 + j) & 1, guard, 204);
                    // the output of the item before has left the accumulator
                    if (j == 0 && i0 > 0) mbar_wait_poll(&o_free[0], (i0 - 1) & 1, guard, 211);
                    tc_fence_after();
                    issue_pv(0, s, j > 0);
                    umma_commit_e(el, &pv_done[0]);
                }
                if (w.has_t1) {
                    mbar_wait_poll(&p_full[1], (c1 + j) & 1, guard, 206);
                    if (j == 0 && i1 > 0) mbar_wait_poll(&o_free[1], (i1 - 1) & 1, guard, 212);
                    tc_fence_after();
                    issue_pv(1, s, j > 0);
                    umma_commit_e(el, &pv_done[1]);
                }
                umma_commit_e(el, &kv_empty[s]);
            }
            J += w.nkv;
            c0 += last0 + 1;
            i0++;
            if (w.has_t1) {
                c1 += w.nkv;
                i1++;
            }
        }
    } else {
        // ---------------- softmax groups ----------------
        const int t = warp / 8;        // query tile of the item
        const int hf = (warp / 4) & 1;  // half of the key columns: 64*hf .. 64*hf + 63
        const int q4 = warp % 4;        // TMEM lane quarter
        const int r = q4 * 32 + lane;   // row inside the tile == TMEM lane
        const uint32_t lane_base = tmem + (static_cast<uint32_t>(q4 * 32) << 16);
        const uint32_t tS = lane_base + COL_S + t * BN + 64 * hf;
        const uint32_t tO = lane_base + COL_O + t * DH + 32 * hf;  // this thread's half of the output row
        const uint32_t tP = lane_base + COL_P + t * 64 + 32 * hf;
        const int pair_bar = 1 + t * 4 + q4;  // named barrier of the two warps that share these 32 rows
        auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory"); };
        int ct = 0;  // steps so far of this group's query tile, over all items (phases of its barriers)
        Item w;
        for (int k = 0; get_item(k, npairs, nbh, p.S, w); k++) {
            if (t == 1 && !w.has_t1) continue;  // a ragged last pair has no second tile
            const int jlast = w.n0 + t;
            float m = -INFINITY, l = 0.f;  // l: this thread's half of the row sum
            for (int j = 0; j <= jlast; j++) {
                const int cj = ct + j;
                mbar_wait(&s_full[t], cj & 1, guard, 301 + t);
                tc_fence_after();
                const bool diag = j == jlast;
                // The half row of scores goes to registers at once, and the score columns are handed
                // back right away: S_t(j+1) is computed while this step's exponentials run.
                uint32_t sv[2][32];
                tmem_ld32(tS, sv[0]);
                tmem_ld32(tS + 32, sv[1]);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&s_free[t]);
                // pass 1: maximum of the half row (two chains); on the diagonal tile key column c is visible iff c <= r
                float mx0 = -INFINITY, mx1 = -INFINITY;
                if (diag) {
#pragma unroll
                    for (int c = 0; c < 2; c++)
#pragma unroll
                        for (int i = 0; i < 32; i++)
                            if (64 * hf + 32 * c + i > r) sv[c][i] = 0xff800000u;  // -inf
                }
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    mx0 = max3(mx0, __uint_as_float(sv[0][i]), __uint_as_float(sv[0][i + 1]));
                    mx1 = max3(mx1, __uint_as_float(sv[1][i]), __uint_as_float(sv[1][i + 1]));
                }
                // the other half's maximum: both threads of a row must scale by the same reference
                xmax[t][cj & 1][hf][r] = fmaxf(mx0, mx1);
                pair_sync();
                const float mx = fmaxf(fmaxf(mx0, mx1), xmax[t][cj & 1][hf ^ 1][r]);
                const float m_new = fmaxf(m, mx * p.scale_log2);
                const bool raise = m_new - m > 8.0f;  // also true on the first tile (m = -inf)
                const float m_use = raise ? m_new : m;
                const float alpha = raise ? ex2(m - m_new) : 1.0f;
                // O_t must be stable and P_t free before this step's P is stored (and before a rescaling
                // of O_t): wait for the PV product of the step before, here or after half the exponentials
                auto settle = [&]() {
                    mbar_wait(&pv_done[t], (cj - 1) & 1, guard, 305 + t);
                    tc_fence_after();
                    if (__any_sync(0xffffffffu, raise)) {  // the partner warp sees the same flags row by row
#pragma unroll
                        for (int h2 = 0; h2 < 2; h2++) {  // 16 columns at a time: the score row fills the registers
                            uint32_t o[16];
                            tmem_ld16(tO + 16 * h2, o);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 16; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                            tmem_st16(tO + 16 * h2, o);
                        }
                    }
                };
                if (!LATE_WAIT && j > 0) settle();
                // (j == 0: P_t is free since the epilogue of the item before waited for its last PV)
                m = m_use;
                // pass 2: P = exp2(c*S - m) as bf16 pairs (masked scores are -inf and give 0); the
                // arguments and the row sum are formed two at a time in packed fp32
                const uint64_t c2 = pack2(p.scale_log2, p.scale_log2), m2 = pack2(-m_use, -m_use);
                uint64_t rs2 = pack2(0.f, 0.f);
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    // the bf16 pairs are packed into the front of the score registers they come from
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        float a0, a1, b0, b1;
                        unpack2(fma2(pack2(__uint_as_float(sv[c][i]), __uint_as_float(sv[c][i + 1])), c2, m2), a0, a1);
                        unpack2(fma2(pack2(__uint_as_float(sv[c][i + 2]), __uint_as_float(sv[c][i + 3])), c2, m2), b0, b1);
                        a0 = ex2(a0);
                        a1 = ex2(a1);
                        if ((i / 4) % POLY_PERIOD < POLY_PAIRS) {
                            ex2_poly2(b0, b1);
                        } else {
                            b0 = ex2(b0);
                            b1 = ex2(b1);
                        }
                        rs2 = add2(rs2, add2(pack2(a0, a1), pack2(b0, b1)));
                        sv[c][i / 2] = pack_bf16(a0, a1);
                        sv[c][i / 2 + 1] = pack_bf16(b0, b1);
                    }
                    if (c == 0 && LATE_WAIT && j > 0) settle();
                    tmem_st16(tP + 16 * c, sv[c]);
                }
                float rs, rs_hi;
                unpack2(rs2, rs, rs_hi);
                rs += rs_hi;
                l = l * alpha + rs;
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&p_full[t]);
            }
            // epilogue: O_t / l -> bf16 -> global; lse.  The accumulator goes back to the MMA warp as
            // soon as it is in registers.
            mbar_wait(&pv_done[t], (ct + jlast) & 1, guard, 311 + t);
            tc_fence_after();
            ct += jlast + 1;
            uint32_t o[32];
            tmem_ld32(tO, o);
            xsum[t][hf][r] = l;
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&o_free[t]);
            pair_sync();
            l += xsum[t][hf ^ 1][r];
            const int qr = w.q0 + t * BM + r;
            const float inv = 1.0f / l;
            const int b = w.bh / p.H, h = w.bh % p.H;
            if (qr < p.S && p.O != nullptr) {
                uint4* dst = reinterpret_cast<uint4*>(p.O + (int64_t)b * p.sb + (int64_t)qr * p.ss + (int64_t)h * p.sh + 32 * hf);
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    uint4 v;
                    v.x = pack_bf16(__uint_as_float(o[i + 0]) * inv, __uint_as_float(o[i + 1]) * inv);
                    v.y = pack_bf16(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
                    v.z = pack_bf16(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
                    v.w = pack_bf16(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
                    dst[i / 8] = v;
                }
            }
            if (hf == 0 && qr < p.S && p.lse != nullptr) p.lse[(int64_t)w.bh * p.S + qr] = (m + log2f(l)) * 0.6931471805599453f;
            // the partner must have read this item's row sum before the next item's is written
            pair_sync();
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

bool mha_tc_supported(const MhaShape& p) {
    return p.Dh == DH && p.sh % 8 == 0 && p.ss % 8 == 0 && p.sb % 8 == 0;
}

int mha_tc_fwd(const MhaShape& p, const void* Q, const void* K, const void* V, void* O, float* lse,
               cudaStream_t st) {
    if (!mha_tc_supported(p)) return CXXATTN_ERR_UNSUPPORTED;
    for (const void* q : {Q, K, V, (const void*)O})  // O may be null: statistics-only pass
        if (reinterpret_cast<uintptr_t>(q) % 16) return CXXATTN_ERR_ALIGNMENT;
    CUtensorMap tmQ, tmK, tmV;
    if (!make_tmap_bhsd(&tmQ, Q, p.B, p.S, p.H, p.Dh, p.sb, p.ss, p.sh, BM) ||
        !make_tmap_bhsd(&tmK, K, p.B, p.S, p.H, p.Dh, p.sb, p.ss, p.sh, BN) ||
        !make_tmap_bhsd(&tmV, V, p.B, p.S, p.H, p.Dh, p.sb, p.ss, p.sh, BN))
        return CXXATTN_ERR_CUDA;
    FwdParams fp;
    fp.O = static_cast<__nv_bfloat16*>(O);
    fp.lse = lse;
    fp.status = status_word();
    if (fp.status == nullptr) return CXXATTN_ERR_CUDA;
    fp.B = p.B; fp.S = p.S; fp.H = p.H;
    fp.sb = p.sb; fp.ss = p.ss; fp.sh = p.sh;
    fp.scale_log2 = p.scale * 1.4426950408889634f;
    static OncePerDevice attr;
    const int dev = current_device();
    if (attr.pending(dev)) {
        if (cudaFuncSetAttribute(mha_tc_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)SMEM_BYTES) != cudaSuccess ||
            cudaFuncSetAttribute(mha_tc_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)SMEM_BYTES) != cudaSuccess)
            return CXXATTN_ERR_CUDA;
        attr.done(dev);
    }
    // persistent CTAs, one per SM, each walking its share of the (query-tile pair, batch*head) items
    const int npairs = (p.S + 2 * BM - 1) / (2 * BM);
    const int64_t items = (int64_t)npairs * p.B * p.H;
    const int64_t grid = std::min<int64_t>(items, sm_count());
    const bool late = option(CXXATTN_OPT_FWD_LATE_WAIT) != 0;  // -1 (default) and 1: wait late
    if (late) mha_tc_fwd_kernel<true><<<(unsigned)grid, NTHREADS, SMEM_BYTES, st>>>(tmQ, tmK, tmV, fp);
    else mha_tc_fwd_kernel<false><<<(unsigned)grid, NTHREADS, SMEM_BYTES, st>>>(tmQ, tmK, tmV, fp);
    return check_launch();
}

}  // namespace cxxattn
