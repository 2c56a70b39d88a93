// Causal softmax MHA backward on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), bf16
// operands, fp32 accumulation, head dimension 64.
//
// Replaces two_stage_cuda::fused_mha_bwd (src/TwoStage/two_stage_cuda_kernels.cu:334-882) for dtype
// BF16.  The reference keeps the S x S matrices P and dP of one (batch, head) in shared memory or
// in freshly allocated global scratch; here nothing of size S x S exists.  A CTA owns one tile of
// 128 keys, keeps dK and dV for it in tensor memory, walks the query tiles at or below the causal
// diagonal and recomputes the probabilities from the row log-sum-exp:
//
//   S^T  = K Q_i^T                 (SS MMA, keys on the 128 TMEM lanes, queries on 128 columns)
//   dP^T = V dO_i^T                (SS MMA)
//   P^T  = exp2(c S^T - lse2_q)    (lane = key row)  -> bf16 in registers and in TMEM
//   dS^T = P^T o (dP^T - delta_q)  -> bf16 in shared memory, one tile that is both a K-major operand
//                                  [keys][queries] and an MN-major one
//   dV  += P^T dO_i                (TS MMA: P^T from TMEM, dO_i as an MN-major operand)
//   dK  += dS^T Q_i                (SS MMA: dS read K-major, Q_i MN-major)
//   dQ_i = dS K                    (SS MMA: dS read MN-major), drained from TMEM through shared memory
//                                  with one bulk reduce-add per warp into an fp32 accumulator
//
// 16 compute warps in two groups take the query tiles alternately (by the parity of the tile's running
// index); inside a group a warp owns 32 key rows (its TMEM lanes) and one half of the 128 query
// columns, and does both halves of the tile's work on them, so P^T never has to be read back; the MMA
// warp issues S^T(i+1) and dP^T(i+1) as soon as tile i's have been read out of TMEM, so one group is in
// the first half of tile i+1 while the other is in the second half of tile i.  For sequences of up to
// 32 tiles the CTAs are persistent (one per SM) and draw (key tile, batch*head) items from a global
// counter; the rings of barriers keep their phase across items, so the next item's first loads and
// the epilogue of the current one overlap instead of paying the pipeline's fill and drain per CTA.
//
// Three launches per call: a row pre-pass (delta = dO.O, lse in log2 units padded to whole tiles,
// accumulator cleared), the main kernel, and a pass turning the accumulator into bf16 dQ.
// dQ is summed with atomics, so its low bits depend on the order in which CTAs arrive.
#include <algorithm>

#include "internal.cuh"
#include "tc_common.cuh"

namespace cxxattn {
namespace {

using namespace tc;

constexpr int BT = 128;  // rows per tile (queries and keys)
constexpr int DH = 64;
constexpr int TILE_BYTES = BT * DH * 2;  // 16 KB
constexpr int NTHREADS = 640;  // warps 0-15 compute, 16 producer, 17 MMA issuer, 18-19 only hand registers over
constexpr int W_PROD = 16, W_MMA = 17;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t COL_ST = 0, COL_DP = 128, COL_DV = 256, COL_DK = 320, COL_DQ = 384, COL_P = 448;
// K | V | Q x3 | dO x2 | dS x2 (2 blocks each) | (lse2, delta) x3 | dQ staging
constexpr int NQ = 3;                  // Q stages: Q_i is read first (S^T) and last (dK) in a tile's life
constexpr int NTILES = 2 + NQ + 2 + 4;
constexpr int STAGE_BYTES = 8 * 4096;  // dQ staging: 32 rows x 32 fp32 per warp of the draining group
constexpr size_t SMEM_BYTES = NTILES * TILE_BYTES + NQ * 1024 + STAGE_BYTES + 1024;

struct BwdParams {
    const float* lse2;   // [BH][Spad]  lse * log2(e), +inf on padding rows
    const float* delta;  // [BH][Spad]
    float* dq_acc;       // [BH][Spad/128] tiles of [row / 32][column / 32][row % 32][32]; the 16-byte chunk ch
                         // of such a 128-byte row is stored at chunk ch ^ (row & 7)
    __nv_bfloat16* dK;
    __nv_bfloat16* dV;
    int* status;
    int* counter;  // next work item; zero at launch
    int B, S, H, Spad;
    int64_t sb, ss, sh;
    float scale, scale_log2;
};

// Eight threads per (batch*head, row < Spad), 16 bytes of O and dO each: delta, lse2, and a cleared
// accumulator row.
__global__ void mha_tc_bwd_pre_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO,
                                      const float* __restrict__ lse, float* __restrict__ lse2,
                                      float* __restrict__ delta, float* __restrict__ dq_acc, int* __restrict__ counter,
                                      int B, int S, int H, int Spad, int64_t sb, int64_t ss, int64_t sh) {
    const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / 8;
    const int part = threadIdx.x % 8;
    if (row >= (int64_t)B * H * Spad) return;  // whole groups of 8 threads leave together
    const int s = row % Spad;
    const int bh = row / Spad;
    float4* z = reinterpret_cast<float4*>(dq_acc + row * DH + part * 8);
    z[0] = make_float4(0.f, 0.f, 0.f, 0.f);
    z[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    float acc = 0.f;
    if (s < S) {
        const int64_t off = (int64_t)(bh / H) * sb + (int64_t)s * ss + (int64_t)(bh % H) * sh + part * 8;
        const uint4 o = *reinterpret_cast<const uint4*>(O + off);
        const uint4 g = *reinterpret_cast<const uint4*>(dO + off);
        const uint32_t ow[4] = {o.x, o.y, o.z, o.w}, gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ow[i]));
            const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw[i]));
            acc = fmaf(a.x, c.x, fmaf(a.y, c.y, acc));
        }
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (row == 0 && part == 0) *counter = 0;  // the main kernel's work-item counter
    if (part == 0) {
        delta[row] = acc;
        lse2[row] = s < S ? lse[(int64_t)bh * S + s] * 1.4426950408889634f : INFINITY;
    }
}

// dQ[b,s,h,:] = bf16(scale * acc[bh][s][:]); eight threads per row, 8 columns each.
__global__ void mha_tc_bwd_post_kernel(const float* __restrict__ dq_acc, __nv_bfloat16* __restrict__ dQ, int B,
                                       int S, int H, int Spad, int64_t sb, int64_t ss, int64_t sh, float scale) {
    const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / 8;
    const int part = threadIdx.x % 8;
    if (row >= (int64_t)B * H * S) return;
    const int s = row % S;
    const int bh = row / S;
    // accumulator layout of the main kernel: per tile of 128 rows, blocks [row / 32][column / 32] of
    // 32 rows x 32 floats, the 16-byte chunk ch of a row stored at chunk position ch ^ (row & 7)
    const int rt = s % BT;
    const float* src = dq_acc + ((int64_t)bh * (Spad / BT) + s / BT) * (BT * DH) + ((rt / 32) * 2 + part / 4) * 1024 +
                       (rt % 32) * 32;
    const int ch = 2 * (part % 4);
    const float4 a = *reinterpret_cast<const float4*>(src + ((ch ^ (rt & 7)) * 4));
    const float4 c = *reinterpret_cast<const float4*>(src + (((ch + 1) ^ (rt & 7)) * 4));
    const int64_t off = (int64_t)(bh / H) * sb + (int64_t)s * ss + (int64_t)(bh % H) * sh + part * 8;
    *reinterpret_cast<uint4*>(dQ + off) =
        make_uint4(pack_bf16(a.x * scale, a.y * scale), pack_bf16(a.z * scale, a.w * scale),
                   pack_bf16(c.x * scale, c.y * scale), pack_bf16(c.z * scale, c.w * scale));
}

__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// Adds `bytes` of fp32 from shared memory into global memory (one bulk reduction in the L2).
__device__ __forceinline__ void bulk_reduce_add_f32(float* gdst, const void* ssrc, uint32_t bytes) {
    asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(gdst),
                 "r"(smem_u32(ssrc)), "r"(bytes)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// One arrival per warp, after every lane of the warp has done its part.
__device__ __forceinline__ void warp_arrive(uint64_t* bar, int lane) {
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
}
// P^T for 32 query columns of one key row: exp2(c*S - lse2_q) as 16 bf16 pairs; on the diagonal
// tile key row r is visible to query column qc iff r <= qc.
template <bool DIAG>
__device__ __forceinline__ void p_chunk(uint32_t (&v)[32], const float* l2, float c, int r, int qc0, uint32_t* pk) {
    // three passes over the 32 values (arguments, exponentials, packing) keep many independent
    // operations in flight: the warp has few partners to hide latencies behind
    const float4* l4 = reinterpret_cast<const float4*>(l2);
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
        const float4 la = l4[i / 4];
        v[i] = __float_as_uint(fmaf(__uint_as_float(v[i]), c, -la.x));
        v[i + 1] = __float_as_uint(fmaf(__uint_as_float(v[i + 1]), c, -la.y));
        v[i + 2] = __float_as_uint(fmaf(__uint_as_float(v[i + 2]), c, -la.z));
        v[i + 3] = __float_as_uint(fmaf(__uint_as_float(v[i + 3]), c, -la.w));
    }
#pragma unroll
    for (int i = 0; i < 32; i++) {
        float a = ex2(__uint_as_float(v[i]));
        if (DIAG) a = r <= qc0 + i ? a : 0.f;
        v[i] = __float_as_uint(a);
    }
#pragma unroll
    for (int i = 0; i < 32; i += 2) pk[i / 2] = pack_bf16(__uint_as_float(v[i]), __uint_as_float(v[i + 1]));
}
// dS^T = P^T o (dP^T - delta_q) for 32 query columns, in packed bf16 arithmetic (the result is a
// bf16 MMA operand anyway).
__device__ __forceinline__ void ds_chunk(const uint32_t* p16, uint32_t (&v)[32], const float* dl, uint32_t* ds) {
    const float4* d4 = reinterpret_cast<const float4*>(dl);
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
        const float4 d = d4[i / 4];
        v[i] = __float_as_uint(__uint_as_float(v[i]) - d.x);
        v[i + 1] = __float_as_uint(__uint_as_float(v[i + 1]) - d.y);
        v[i + 2] = __float_as_uint(__uint_as_float(v[i + 2]) - d.z);
        v[i + 3] = __float_as_uint(__uint_as_float(v[i + 3]) - d.w);
    }
#pragma unroll
    for (int i = 0; i < 32; i += 2) v[i / 2] = pack_bf16(__uint_as_float(v[i]), __uint_as_float(v[i + 1]));
#pragma unroll
    for (int i = 0; i < 16; i++) {
        const __nv_bfloat162 r0 = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&p16[i]),
                                          *reinterpret_cast<const __nv_bfloat162*>(&v[i]));
        ds[i] = *reinterpret_cast<const uint32_t*>(&r0);
    }
}
// Half a key row (32 fp32 TMEM columns of this lane, columns c0..c0+31) -> scaled bf16 -> global.
__device__ __forceinline__ void store_rows(uint32_t taddr, __nv_bfloat16* base, float f, int key, int c0, int b, int h,
                                           const BwdParams& p) {
    uint32_t o0[32];
    tmem_ld32(taddr + c0, o0);
    tmem_ld_wait();
    if (key >= p.S) return;
    uint4* dst = reinterpret_cast<uint4*>(base + (int64_t)b * p.sb + (int64_t)key * p.ss + (int64_t)h * p.sh + c0);
#pragma unroll
    for (int i = 0; i < 32; i += 8)
        dst[i / 8] = make_uint4(pack_bf16(__uint_as_float(o0[i]) * f, __uint_as_float(o0[i + 1]) * f),
                                pack_bf16(__uint_as_float(o0[i + 2]) * f, __uint_as_float(o0[i + 3]) * f),
                                pack_bf16(__uint_as_float(o0[i + 4]) * f, __uint_as_float(o0[i + 5]) * f),
                                pack_bf16(__uint_as_float(o0[i + 6]) * f, __uint_as_float(o0[i + 7]) * f));
}

// One work item = one (key tile, batch*head).  Items are numbered heavy first (key tile 0 meets every
// query tile) and handed out through a global counter, so a CTA that finishes early takes the next
// one.  The producer thread draws the numbers and passes them to the other roles of its CTA through a
// two-entry ring in shared memory; all roles therefore walk the same list.
struct Item {
    int n, bh, niter;  // key tile, batch*head, query tiles to visit (n .. ntile-1)
};
struct ItemRing {
    int slot[2];
    uint64_t full[2], empty[2];
};
__device__ __forceinline__ bool decode_item(int id, int ntile, int nbh, Item& w) {
    if (id < 0 || id >= ntile * nbh) return false;
    w.n = id / nbh;
    w.bh = id % nbh;
    w.niter = ntile - w.n;
    return true;
}
// The k-th item of this CTA, for every role but the producer: all lanes of the warp read the entry,
// then the warp gives it back.
__device__ __forceinline__ bool next_item(ItemRing& ring, int k, int lane, int ntile, int nbh, Item& w,
                                          const Guard& guard) {
    mbar_wait(&ring.full[k & 1], (k >> 1) & 1, guard, 701);
    const int id = *reinterpret_cast<volatile int*>(&ring.slot[k & 1]);
    __syncwarp();
    if (lane == 0) mbar_arrive(&ring.empty[k & 1]);
    // after a timed-out wait the ring no longer means anything: every role leaves its item loop
    if (*reinterpret_cast<volatile int*>(guard.abort_flag)) return false;
    return decode_item(id, ntile, nbh, w);
}

// PERSIST: CTAs draw work items from the global counter until none is left (worth it when items are
// short: the fill and drain of the pipeline overlap between items).  Otherwise CTA i does item i and
// the item bookkeeping folds away.
template <bool PERSIST>
__global__ void __launch_bounds__(NTHREADS, 1)
mha_tc_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, BwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t kv_full, q_full[NQ], q_free[NQ], do_full[2], s_full[2], dp_full[2], dv_done[2], dq_full[2], s_free,
        dp_free, p_ready, ds_ready[2], dq_free, stage_free[8], item_done, acc_free;
    __shared__ ItemRing ring;
    __shared__ int item_stash[16][8];  // per compute warp: what it needs of its current item only between tiles
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sK = smem;
    uint8_t* sV = smem + TILE_BYTES;
    uint8_t* sQ = smem + 2 * TILE_BYTES;          // NQ stages
    uint8_t* sdO = smem + (2 + NQ) * TILE_BYTES;  // 2 stages
    uint8_t* sDS = smem + (4 + NQ) * TILE_BYTES;  // 2 buffers x 2 blocks of 64 queries: [128 keys][64 queries] bf16 each
    float* sStat = reinterpret_cast<float*>(smem + NTILES * TILE_BYTES);  // [Q stage][lse2 | delta][128]
    uint8_t* sStage = smem + NTILES * TILE_BYTES + NQ * 1024;             // [warp % 8][32 rows][128 B]

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int ntile = p.Spad / BT;
    const int nbh = p.B * p.H;
    const Guard guard{&abort_flag, p.status};
    // Query tiles are counted through all items of the CTA: tile T (global index) uses Q stage T % NQ,
    // dO stage / dS buffer / compute group T & 1, and every ring keeps its phase across item borders.

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(&kv_full, 1);
        for (int s = 0; s < NQ; s++) {
            mbar_init(&q_full[s], 1);
            mbar_init(&q_free[s], 1);
        }
        for (int s = 0; s < 2; s++) {  // indexed by the parity of the query tile
            mbar_init(&do_full[s], 1);
            mbar_init(&s_full[s], 1);
            mbar_init(&dp_full[s], 1);
            mbar_init(&dv_done[s], 1);
            mbar_init(&dq_full[s], 1);
        }
        mbar_init(&item_done, 1);
        mbar_init(&acc_free, 16);  // every compute warp, once per item
        // waited on by the MMA warp, tile after tile; one arrival per warp of the group that signals
        mbar_init(&s_free, 8);
        mbar_init(&p_ready, 8);
        mbar_init(&dp_free, 8);
        // dS^T(i+1) may be complete before dS^T(i) is (it waits for neither dK(i) nor dQ(i)): one barrier per group
        mbar_init(&ds_ready[0], 8);
        mbar_init(&ds_ready[1], 8);
        mbar_init(&dq_free, 8);
        for (int w = 0; w < 8; w++) mbar_init(&stage_free[w], 1);
        for (int e = 0; e < 2; e++) {
            mbar_init(&ring.full[e], 1);
            mbar_init(&ring.empty[e], 17);  // 16 compute warps and the MMA warp
        }
        fence_barrier_init();
    }
    if (warp == W_MMA) tmem_alloc(&tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;

    if (warp >= W_PROD) {
        // Warps 16-19 form one warp group; all four execute this one instruction together and hand
        // part of their registers to the compute warps.
        asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    }
    if (warp == W_PROD) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            prefetch_tmap(&tmQ);
            prefetch_tmap(&tmK);
            prefetch_tmap(&tmV);
            prefetch_tmap(&tmdO);
            int T = 0;
            Item w;
            int next = PERSIST ? atomicAdd(p.counter, 1) : (int)blockIdx.x;
            for (int k = 0; PERSIST || k == 0; k++) {
                const int id = next;
                const bool more = decode_item(id, ntile, nbh, w);
                const int b = w.bh / p.H, h = w.bh % p.H;
                if (PERSIST) {
                    if (more) next = atomicAdd(p.counter, 1);  // drawn one item ahead: its latency is hidden
                    if (k >= 2) mbar_wait(&ring.empty[k & 1], ((k >> 1) - 1) & 1, guard, 404);
                    ring.slot[k & 1] = more ? id : -1;
                    mbar_arrive(&ring.full[k & 1]);
                }
                if (!more || *reinterpret_cast<volatile int*>(&abort_flag)) break;
                for (int it = 0; it < w.niter; it++, T++) {
                    const int qs = T % NQ, s = T & 1, q0 = (w.n + it) * BT;
                    // Q (with the row statistics) is held until dK of its tile has read it; dO until dV has
                    if (T >= NQ) mbar_wait(&q_free[qs], ((T / NQ) - 1) & 1, guard, 401);
                    mbar_expect_tx(&q_full[qs], TILE_BYTES + 1024);
                    tma_load_4d(sQ + qs * TILE_BYTES, &tmQ, &q_full[qs], 0, h, q0, b);
                    bulk_load_1d(sStat + qs * 256, p.lse2 + (int64_t)w.bh * p.Spad + q0, 512, &q_full[qs]);
                    bulk_load_1d(sStat + qs * 256 + 128, p.delta + (int64_t)w.bh * p.Spad + q0, 512, &q_full[qs]);
                    if (T >= 2) mbar_wait(&dv_done[s], ((T / 2) - 1) & 1, guard, 402);
                    mbar_expect_tx(&do_full[s], TILE_BYTES);
                    tma_load_4d(sdO + s * TILE_BYTES, &tmdO, &do_full[s], 0, h, q0, b);
                    if (it == 0) {
                        // K and V of this item, once every product of the item before has read the old ones
                        // (the first Q and dO tiles above are already on their way)
                        if (k > 0) mbar_wait(&item_done, (k - 1) & 1, guard, 403);
                        mbar_expect_tx(&kv_full, 2 * TILE_BYTES);
                        tma_load_4d(sK, &tmK, &kv_full, 0, h, w.n * BT, b);
                        tma_load_4d(sV, &tmV, &kv_full, 0, h, w.n * BT, b);
                    }
                }
            }
        }
    } else if (warp == W_MMA) {
        // ---------------- MMA issuer ----------------
        // the whole warp runs the loop (uniform control flow and operands); one elected lane issues
        const uint32_t el = elect_one();
        constexpr uint32_t IDESC_SS = idesc_bf16(BT, BT, 0, 0);  // S^T, dP^T: both operands K-major
        constexpr uint32_t IDESC_KN = idesc_bf16(BT, DH, 0, 1);  // dV, dK: A K-major, B MN-major
        constexpr uint32_t IDESC_DQ = idesc_bf16(BT, DH, 1, 1);  // dQ: dS and K both MN-major
        // Descriptors are built once; K steps and ring stages add constants to the start-address
        // field (units of 16 bytes).
        constexpr uint64_t TILE16 = TILE_BYTES >> 4;
        const uint64_t dK = smem_desc_sw128(smem_u32(sK), 16), dV = smem_desc_sw128(smem_u32(sV), 16);
        const uint64_t dQ0 = smem_desc_sw128(smem_u32(sQ), 16), dG0 = smem_desc_sw128(smem_u32(sdO), 16);
        const uint64_t dDSk = smem_desc_sw128(smem_u32(sDS), 16);          // dS as [keys][queries]: K-major A
        const uint64_t dDSm = smem_desc_sw128(smem_u32(sDS), TILE_BYTES);  // dS as MN-major A (M = queries)
        auto issue_st = [&](int s, int qs) {
            const uint64_t q = dQ0 + qs * TILE16;
#pragma unroll
            for (int k = 0; k < DH / 16; k++) umma_ss_e(el, tmem + COL_ST, dK + 2 * k, q + 2 * k, IDESC_SS, k > 0);
            umma_commit_e(el, &s_full[s]);
        };
        auto issue_dp = [&](int s) {
            const uint64_t g = dG0 + s * TILE16;
#pragma unroll
            for (int k = 0; k < DH / 16; k++) umma_ss_e(el, tmem + COL_DP, dV + 2 * k, g + 2 * k, IDESC_SS, k > 0);
            umma_commit_e(el, &dp_full[s]);
        };
        int T = 0;
        Item w;
        for (int k = 0; PERSIST ? next_item(ring, k, lane, ntile, nbh, w, guard)
                                : (k == 0 && decode_item(blockIdx.x, ntile, nbh, w));
             k++) {
            mbar_wait_poll(&kv_full, k & 1, guard, 501);
            {
                // first tile of the item: its scores and dP^T need the new K and V, so they cannot be
                // issued during the tile before, as all later ones are
                const int s = T & 1, qs = T % NQ;
                mbar_wait_poll(&q_full[qs], (T / NQ) & 1, guard, 502);
                if (T > 0) mbar_wait_poll(&s_free, (T - 1) & 1, guard, 511);
                tc_fence_after();
                issue_st(s, qs);
                mbar_wait_poll(&do_full[s], (T >> 1) & 1, guard, 503);
                if (T > 0) mbar_wait_poll(&dp_free, (T - 1) & 1, guard, 512);
                tc_fence_after();
                issue_dp(s);
            }
            for (int it = 0; it < w.niter; it++, T++) {
                const int s = T & 1, sn = s ^ 1;
                const int qs = T % NQ, qn = (T + 1) % NQ;
                const uint64_t q = dQ0 + qs * TILE16, g = dG0 + s * TILE16;
                const uint64_t dsk = dDSk + s * 2 * TILE16, dsm = dDSm + s * 2 * TILE16;
                if (it + 1 < w.niter) {  // next scores as soon as this tile's are in registers
                    mbar_wait_poll(&q_full[qn], ((T + 1) / NQ) & 1, guard, 506);
                    mbar_wait_poll(&s_free, T & 1, guard, 504);
                    tc_fence_after();
                    issue_st(sn, qn);
                }
                mbar_wait_poll(&p_ready, T & 1, guard, 505);
                // dV and dK of the item before have left TMEM
                if (it == 0 && k > 0) mbar_wait_poll(&acc_free, (k - 1) & 1, guard, 513);
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < BT / 16; kk++)  // dV += P^T dO_i   (A: P^T bf16 in TMEM)
                    umma_ts_e(el, tmem + COL_DV, tmem + COL_P + 8 * kk, g + 128 * kk, IDESC_KN, it > 0 || kk > 0);
                umma_commit_e(el, &dv_done[s]);  // P^T may be overwritten, and this dO stage refilled
                if (it + 1 < w.niter) {  // next dP^T as soon as this tile's is in registers
                    mbar_wait_poll(&do_full[sn], ((T + 1) >> 1) & 1, guard, 509);
                    mbar_wait_poll(&dp_free, T & 1, guard, 510);
                    tc_fence_after();
                    issue_dp(sn);
                }
                mbar_wait_poll(&ds_ready[s], (T >> 1) & 1, guard, 507);
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < BT / 16; kk++)  // dK += dS^T Q_i   (A: dS in smem, rows = keys, K = queries)
                    umma_ss_e(el, tmem + COL_DK, dsk + (kk / 4) * TILE16 + 2 * (kk % 4), q + 128 * kk, IDESC_KN,
                              it > 0 || kk > 0);
                umma_commit_e(el, &q_free[qs]);
                if (T > 0) {
                    mbar_wait_poll(&dq_free, (T - 1) & 1, guard, 508);
                    tc_fence_after();
                }
#pragma unroll
                for (int kk = 0; kk < BT / 16; kk++)  // dQ_i = dS K       (A: the same tile read MN-major)
                    umma_ss_e(el, tmem + COL_DQ, dsm + 128 * kk, dK + 128 * kk, IDESC_DQ, kk > 0);
                umma_commit_e(el, &dq_full[s]);  // dQ_i is ready, and this dS buffer may be overwritten
            }
            // every product of the item: K and V may be replaced, dK and dV read out
            umma_commit_e(el, &item_done);
        }
    } else if (warp > W_MMA) {
        // idle warps: they only take part in the register hand-over above
    } else {
        // The increase is served from the registers the CTA got at launch (640 threads x 96) and blocks
        // until they are there: 16 warps x 32 x (104 - 96) must not exceed what warps 16-19 gave back,
        // 4 x 32 x (96 - 56).
        asm volatile("setmaxnreg.inc.sync.aligned.u32 104;");
        // ---------------- compute warps ----------------
        // Group g = warp / 8 owns the query tiles it = g, g+2, ...; inside a group, warp % 4 selects the
        // 32 key rows (TMEM lanes) and c = (warp / 4) % 2 the half of the 128 query columns.  lane = key
        // row: a thread turns its half row of S^T into P^T (bf16, kept in registers and copied to TMEM
        // for the dV product), then P^T and dP^T into dS^T, and last drains its part of dQ of the tile
        // before (the other group's).  While one group is in the second half of tile i the other is
        // already in the first half of tile i+1.
        const int g = warp / 8;
        const int c = (warp / 4) & 1;
        const int q4 = warp % 4;
        const int r = q4 * 32 + lane;
        const uint32_t lane_base = tmem + (static_cast<uint32_t>(q4 * 32) << 16);
        const uint32_t tS = lane_base + COL_ST + 64 * c, tP = lane_base + COL_P + 32 * c;
        const uint32_t tDP = lane_base + COL_DP + 64 * c, tDQ = lane_base + COL_DQ + 32 * c;
        const int sb = warp % 8;  // staging block, shared with the same warp of the other group, drain after drain
        uint8_t* blk = sStage + sb * 4096;
        bool pending = false;  // this warp's last bulk reduction may still be reading blk
        // the staging block goes back to the other group once this warp's reduction has read it
        auto release_stage = [&]() {
            if (pending && lane == 0) {
                bulk_wait_read();
                mbar_arrive(&stage_free[sb]);
            }
            __syncwarp();  // without it lane 0 may run on its own for a long stretch
            pending = false;
        };
        // dQ of the query tile with global index d (tile `qt` of batch*head `bh`): rows 32*q4.., columns
        // 32*c.., one 4 KB reduction
        auto drain_dq = [&](int d, int bh, int qt) {
            uint32_t d0[32];
            tmem_ld32(tDQ, d0);
            tmem_ld_wait();
            tc_fence_before();
            warp_arrive(&dq_free, lane);
            if (d > 0) mbar_wait(&stage_free[sb], (d - 1) & 1, guard, 617);
#pragma unroll
            for (int ch = 0; ch < 8; ch++)
                *reinterpret_cast<uint4*>(blk + lane * 128 + ((ch ^ (lane & 7)) * 16)) =
                    make_uint4(d0[4 * ch], d0[4 * ch + 1], d0[4 * ch + 2], d0[4 * ch + 3]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0)
                bulk_reduce_add_f32(p.dq_acc + ((int64_t)bh * p.Spad + (int64_t)qt * BT) * DH + (q4 * 2 + c) * 1024, blk, 4096);
            pending = true;
        };
        // Between tiles a warp needs little of its item; the rest (key tile, batch*head, the item
        // before, the item count) waits in shared memory so that the tile loop keeps its registers
        // for the score rows.
        volatile int* stash = item_stash[warp];
        int Tb = 0;  // global index of the first query tile of the current item
        if (lane == 0) stash[2] = 0;
        for (int k = 0; PERSIST || k == 0;) {
            Item w;
            if (PERSIST ? !next_item(ring, k, lane, ntile, nbh, w, guard) : !decode_item(blockIdx.x, ntile, nbh, w)) break;
            const int niter = w.niter;
            if (PERSIST) {
                if (lane == 0) {
                    stash[0] = w.n;
                    stash[1] = w.bh;  // stash[2] holds the batch*head of the item before
                    stash[3] = k;
                    stash[4] = Tb + niter;
                }
                __syncwarp();
            }
            for (int it = (g ^ Tb) & 1; it < niter; it += 2) {  // this group's tiles: global index of parity g
                const int T = Tb + it;
                const int ph = (T >> 1) & 1;  // phase parity of the barriers indexed by tile parity
                const int qs = T % NQ;
                mbar_wait(&q_full[qs], (T / NQ) & 1, guard, 601);  // lse2 / delta of this query tile are in smem
                const float* l2 = sStat + qs * 256 + 64 * c;
                const float* dl = l2 + 128;
                mbar_wait(&s_full[g], ph, guard, 602);
                tc_fence_after();
                uint32_t pk[32];
                {
                    // the half row of S^T goes to registers first, so the next scores can be issued while
                    // this tile's exponentials run
                    uint32_t s0[32], s1[32];
                    tmem_ld32(tS, s0);
                    tmem_ld32(tS + 32, s1);
                    tmem_ld_wait();
                    tc_fence_before();
                    warp_arrive(&s_free, lane);
                    release_stage();  // the other group's next drain waits for this: do it early
                    if (it == 0) {  // the diagonal tile
                        p_chunk<true>(s0, l2, p.scale_log2, r, 64 * c, &pk[0]);
                        p_chunk<true>(s1, l2 + 32, p.scale_log2, r, 64 * c + 32, &pk[16]);
                    } else {
                        p_chunk<false>(s0, l2, p.scale_log2, r, 0, &pk[0]);
                        p_chunk<false>(s1, l2 + 32, p.scale_log2, r, 0, &pk[16]);
                    }
                }
                if (T > 0) {  // the dV product of the tile before has read its P^T
                    mbar_wait(&dv_done[(T - 1) & 1], ((T - 1) >> 1) & 1, guard, 603);
                    tc_fence_after();
                }
                tmem_st32(tP, reinterpret_cast<const uint32_t(&)[32]>(pk[0]));
                tmem_st_wait();
                tc_fence_before();
                warp_arrive(&p_ready, lane);

                // second half: dS^T = P^T o (dP^T - delta), written over pk in place
                {
                    uint32_t va[32];
                    mbar_wait(&dp_full[g], ph, guard, 613);
                    tc_fence_after();
                    tmem_ld32(tDP, va);
                    tmem_ld_wait();
                    ds_chunk(&pk[0], va, dl, &pk[0]);
                    tmem_ld32(tDP + 32, va);
                    tmem_ld_wait();
                    tc_fence_before();
                    warp_arrive(&dp_free, lane);  // dP^T of this tile is in registers
                    ds_chunk(&pk[16], va, dl + 32, &pk[16]);
                }
                if (T >= 2)  // dK and dQ of this group's tile before have read this dS buffer
                    mbar_wait(&dq_full[g], ((T - 2) >> 1) & 1, guard, 614);
                // this thread's part of row r of dS: one 128-byte row (queries 64c..64c+63) with the 128-byte swizzle
                uint8_t* ds_row = sDS + (g * 2 + c) * TILE_BYTES + r * 128;
#pragma unroll
                for (int ch = 0; ch < 8; ch++)
                    *reinterpret_cast<uint4*>(ds_row + ((ch ^ (r & 7)) * 16)) =
                        make_uint4(pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                warp_arrive(&ds_ready[g], lane);
                if (T > 0) {  // dQ of the tile before (the other group's) leaves TMEM through this group
                    mbar_wait(&dq_full[(T - 1) & 1], ((T - 1) >> 1) & 1, guard, 615);
                    tc_fence_after();
                    // that tile is this item's query tile n + it - 1, or the last one of the item before
                    if (it > 0) drain_dq(T - 1, PERSIST ? stash[1] : w.bh, (PERSIST ? stash[0] : w.n) + it - 1);
                    else drain_dq(T - 1, stash[2], ntile - 1);
                }
            }
            // end of the item for this group: group 0 stores dV, group 1 stores scale * dK, and the
            // accumulators go back to the MMA warp
            release_stage();
            if (PERSIST) k = stash[3];
            const int n = PERSIST ? stash[0] : w.n, bh = PERSIST ? stash[1] : w.bh;
            Tb = PERSIST ? stash[4] : niter;
            mbar_wait(&item_done, k & 1, guard, 618);
            tc_fence_after();
            if (g == 0) store_rows(lane_base + COL_DV, p.dV, 1.0f, n * BT + r, 32 * c, bh / p.H, bh % p.H, p);
            else store_rows(lane_base + COL_DK, p.dK, p.scale, n * BT + r, 32 * c, bh / p.H, bh % p.H, p);
            tc_fence_before();
            warp_arrive(&acc_free, lane);
            if (lane == 0) stash[2] = bh;
            __syncwarp();
            k++;
        }
        const int prev_bh = stash[2];
        release_stage();
        // the very last tile's dQ is drained by the group that would own the next tile
        if (Tb > 0 && g == (Tb & 1)) {
            mbar_wait(&dq_full[(Tb - 1) & 1], ((Tb - 1) >> 1) & 1, guard, 616);
            tc_fence_after();
            drain_dq(Tb - 1, prev_bh, ntile - 1);
        }
        if (lane == 0) bulk_wait_all();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == W_MMA) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

}  // namespace

// Optional CUDA events recorded right before and after the main backward kernel (see
// cxxattn_set_timing_events); null = off.
static thread_local cudaEvent_t g_ev_start = nullptr, g_ev_stop = nullptr;
void mha_tc_bwd_set_timing_events(void* start, void* stop) {
    g_ev_start = static_cast<cudaEvent_t>(start);
    g_ev_stop = static_cast<cudaEvent_t>(stop);
}

static size_t rows_bytes(const MhaShape& p) {
    const size_t spad = ((size_t)p.S + BT - 1) / BT * BT;
    return align_up((size_t)p.B * p.H * spad * sizeof(float), 256);
}

size_t mha_tc_bwd_workspace(const MhaShape& p, bool have_lse) {
    const size_t rows = rows_bytes(p);
    // lse2 | delta | dQ accumulator | work-item counter | (row statistics when the caller has none)
    return 2 * rows + rows * DH + 256 + (have_lse ? 0 : align_up((size_t)p.B * p.H * p.S * sizeof(float), 256));
}

int mha_tc_bwd(const MhaShape& p, const void* Q, const void* K, const void* V, const void* O, const void* dO,
               const float* lse, void* dQ, void* dK, void* dV, void* ws, size_t ws_bytes, cudaStream_t st) {
    if (!mha_tc_supported(p)) return CXXATTN_ERR_UNSUPPORTED;
    for (const void* q : {Q, K, V, O, dO, (const void*)dQ, (const void*)dK, (const void*)dV})
        if (reinterpret_cast<uintptr_t>(q) % 16) return CXXATTN_ERR_ALIGNMENT;
    if (ws == nullptr || ws_bytes < mha_tc_bwd_workspace(p, lse != nullptr)) return CXXATTN_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(ws) % 256) return CXXATTN_ERR_ALIGNMENT;
    const int Spad = (p.S + BT - 1) / BT * BT;
    const size_t rows = rows_bytes(p);
    char* base = static_cast<char*>(ws);
    float* lse2 = reinterpret_cast<float*>(base);
    float* delta = reinterpret_cast<float*>(base + rows);
    float* dq_acc = reinterpret_cast<float*>(base + 2 * rows);
    int* counter = reinterpret_cast<int*>(base + 2 * rows + rows * DH);
    if (lse == nullptr) {
        // The reference backward recomputes the row statistics from Q and K; so does this pre-pass
        // (the forward kernel with its output store switched off).
        float* tmp = reinterpret_cast<float*>(base + 2 * rows + rows * DH + 256);
        const int rc = mha_tc_fwd(p, Q, K, V, nullptr, tmp, st);
        if (rc != CXXATTN_OK) return rc;
        lse = tmp;
    }
    const int64_t nrows = (int64_t)p.B * p.H * Spad;
    mha_tc_bwd_pre_kernel<<<(unsigned)((nrows + 31) / 32), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(O), static_cast<const __nv_bfloat16*>(dO), lse, lse2, delta, dq_acc, counter, p.B,
        p.S, p.H, Spad, p.sb, p.ss, p.sh);
    if (check_launch() != CXXATTN_OK) return CXXATTN_ERR_CUDA;

    CUtensorMap tmQ, tmK, tmV, tmG;
    if (!make_tmap_bhsd(&tmQ, Q, p.B, p.S, p.H, p.Dh, p.sb, p.ss, p.sh, BT) ||
        !make_tmap_bhsd(&tmK, K, p.B, p.S, p.H, p.Dh, p.sb, p.ss, p.sh, BT) ||
        !make_tmap_bhsd(&tmV, V, p.B, p.S, p.H, p.Dh, p.sb, p.ss, p.sh, BT) ||
        !make_tmap_bhsd(&tmG, dO, p.B, p.S, p.H, p.Dh, p.sb, p.ss, p.sh, BT))
        return CXXATTN_ERR_CUDA;
    BwdParams bp;
    bp.lse2 = lse2; bp.delta = delta; bp.dq_acc = dq_acc;
    bp.dK = static_cast<__nv_bfloat16*>(dK);
    bp.dV = static_cast<__nv_bfloat16*>(dV);
    bp.counter = counter;
    bp.status = status_word();
    if (bp.status == nullptr) return CXXATTN_ERR_CUDA;
    bp.B = p.B; bp.S = p.S; bp.H = p.H; bp.Spad = Spad;
    bp.sb = p.sb; bp.ss = p.ss; bp.sh = p.sh;
    bp.scale = p.scale;
    bp.scale_log2 = p.scale * 1.4426950408889634f;
    static OncePerDevice attr;
    const int dev = current_device();
    if (attr.pending(dev)) {
        if (cudaFuncSetAttribute(mha_tc_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)SMEM_BYTES) != cudaSuccess ||
            cudaFuncSetAttribute(mha_tc_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)SMEM_BYTES) != cudaSuccess)
            return CXXATTN_ERR_CUDA;
        attr.done(dev);
    }
    const int64_t items = (int64_t)(Spad / BT) * p.B * p.H;
    // Short sequences (few query tiles per item): persistent CTAs, one per SM, each walking its share of
    // the (key tile, batch*head) items; long ones: one CTA per item, whose tile loop compiles a little
    // tighter.  CXXATTN_OPT_BWD_PERSISTENT = 0 / 1 forces the choice.
    const int forced = option(CXXATTN_OPT_BWD_PERSISTENT);
    const bool persist = forced >= 0 ? forced != 0 : Spad / BT <= 32;
    const int64_t grid = persist ? std::min<int64_t>(items, sm_count()) : items;
    if (g_ev_start) cudaEventRecord(g_ev_start, st);
    if (persist) mha_tc_bwd_kernel<true><<<(unsigned)grid, NTHREADS, SMEM_BYTES, st>>>(tmQ, tmK, tmV, tmG, bp);
    else mha_tc_bwd_kernel<false><<<(unsigned)grid, NTHREADS, SMEM_BYTES, st>>>(tmQ, tmK, tmV, tmG, bp);
    if (g_ev_stop) cudaEventRecord(g_ev_stop, st);
    if (check_launch() != CXXATTN_OK) return CXXATTN_ERR_CUDA;

    const int64_t orows = (int64_t)p.B * p.H * p.S;
    mha_tc_bwd_post_kernel<<<(unsigned)((orows + 31) / 32), 256, 0, st>>>(dq_acc, static_cast<__nv_bfloat16*>(dQ), p.B,
                                                                      p.S, p.H, Spad, p.sb, p.ss, p.sh, p.scale);
    return check_launch();
}

}  // namespace cxxattn
