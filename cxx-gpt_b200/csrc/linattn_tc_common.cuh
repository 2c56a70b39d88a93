// Pieces shared by the bf16 tensor-core linear-attention kernels (forward, the two backward passes
// and the group-state pre-pass): tile constants, the packed feature map, step 1 on a tile row, the
// state row <-> operand tile conversion, and the sequence-group bookkeeping.
#pragma once
#include "internal.cuh"
#include "tc_common.cuh"

namespace cxxattn {
namespace lintc {

using namespace tc;

constexpr int CH = 128;  // tokens per chunk
constexpr int DE = 64;   // feature width (D = E)
constexpr int TILE_BYTES = CH * DE * 2;  // 16 KB

__device__ __forceinline__ float bf_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ float phi1(float a) { return a > 0.f ? a + 1.f : ex2(a * 1.4426950408889634f); }
__device__ __forceinline__ float dphi1(float a) { return a > 0.f ? 1.f : ex2(a * 1.4426950408889634f); }
// phi on a bf16 pair in packed arithmetic: x > 0 ? x + 1 : 2^(x log2 e), written without a select as
// max(x, 0) + 2^(min(x, 0) log2 e) (for x > 0 the second term is exactly 1, for x <= 0 the first is
// exactly 0).  The product with log2(e) is rounded to bf16 before the exponential (relative effect
// ln2*|t|*2^-9 on values that are then rounded to bf16 anyway).
__device__ __forceinline__ uint32_t phi2(uint32_t v) {
    const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(&v);
    const __nv_bfloat162 zero = __floats2bfloat162_rn(0.f, 0.f);
    const __nv_bfloat162 t = __hmul2(__hmin2(x, zero), __floats2bfloat162_rn(1.4426950408889634f, 1.4426950408889634f));
    uint32_t e;
    asm("ex2.approx.ftz.bf16x2 %0, %1;" : "=r"(e) : "r"(*reinterpret_cast<const uint32_t*>(&t)));
    const __nv_bfloat162 r = __hadd2(__hmax2(x, zero), *reinterpret_cast<const __nv_bfloat162*>(&e));
    return *reinterpret_cast<const uint32_t*>(&r);
}

// In-place feature map of one 128-byte tile row (element order does not matter).
// Rows are 128 bytes apart, so the lanes of a warp must not all touch the same 16-byte chunk
// index at once (that would be a 32-way bank conflict): lane l starts at chunk l & 7.
__device__ __forceinline__ void map_row(uint8_t* row, bool valid, bool elu, int rot) {
    uint4* p = reinterpret_cast<uint4*>(row);
    uint4 v[8];
    // all loads first, all stores last: with run-time chunk positions the compiler cannot reorder
    // a load past an earlier store, and a lone warp would crawl through eight dependent round trips
#pragma unroll
    for (int ch = 0; ch < 8; ch++) v[ch] = p[ch ^ rot];
#pragma unroll
    for (int ch = 0; ch < 8; ch++) {
        if (!valid) v[ch] = make_uint4(0u, 0u, 0u, 0u);
        else if (elu) v[ch] = make_uint4(phi2(v[ch].x), phi2(v[ch].y), phi2(v[ch].z), phi2(v[ch].w));
    }
#pragma unroll
    for (int ch = 0; ch < 8; ch++) p[ch ^ rot] = v[ch];
}

// The same for half a row: chunks 4*half .. 4*half+3 (in the rotated order), so that two threads can
// share a row.
__device__ __forceinline__ void map_half_row(uint8_t* row, bool valid, int rot, int half) {
    uint4* p = reinterpret_cast<uint4*>(row);
    uint4 v[4];
#pragma unroll
    for (int ch = 0; ch < 4; ch++) v[ch] = p[(ch + 4 * half) ^ rot];
#pragma unroll
    for (int ch = 0; ch < 4; ch++) {
        if (!valid) v[ch] = make_uint4(0u, 0u, 0u, 0u);
        else v[ch] = make_uint4(phi2(v[ch].x), phi2(v[ch].y), phi2(v[ch].z), phi2(v[ch].w));
    }
#pragma unroll
    for (int ch = 0; ch < 4; ch++) p[(ch + 4 * half) ^ rot] = v[ch];
}

// Asks for the 128-byte row at `row` to be brought into L2: issued two chunks ahead by the lone warps
// that will read token rows from global memory (a miss costs them ~3000 cycles, and they have
// nothing to hide it behind).
__device__ __forceinline__ void prefetch_row(const void* row) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(row));
}

// Step 1 for one token row: the dO tile row becomes dnum = dO / den in place, dden = -(dO . O) / den
// is returned and also written (bf16) to element 0 of the row's side-tile entry.
__device__ __forceinline__ float step1_row(uint8_t* do_row, const __nv_bfloat16* o_row, float den, bool valid,
                                           int swz, uint8_t* dden_slot) {
    uint4* p = reinterpret_cast<uint4*>(do_row);
    const uint4* o = reinterpret_cast<const uint4*>(o_row);
    const float inv = valid ? 1.0f / den : 0.f;
    // The tile row is stored with its 16-byte chunks permuted: logical chunk ch sits at position
    // ch ^ swz (swz = row & 7, which also spreads the lanes of a warp over the banks); the O row comes
    // from global memory in logical order.  All loads first, all stores last.
    uint4 g[8], ov[8];
#pragma unroll
    for (int ch = 0; ch < 8; ch++) {
        g[ch] = p[ch ^ swz];
        ov[ch] = valid ? o[ch] : make_uint4(0u, 0u, 0u, 0u);
    }
    float dot = 0.f;
#pragma unroll
    for (int ch = 0; ch < 8; ch++) {
        const uint4 a = g[ch], c = ov[ch];
        dot += bf_lo(a.x) * bf_lo(c.x) + bf_hi(a.x) * bf_hi(c.x) + bf_lo(a.y) * bf_lo(c.y) + bf_hi(a.y) * bf_hi(c.y) +
               bf_lo(a.z) * bf_lo(c.z) + bf_hi(a.z) * bf_hi(c.z) + bf_lo(a.w) * bf_lo(c.w) + bf_hi(a.w) * bf_hi(c.w);
        g[ch] = make_uint4(pack_bf16(bf_lo(a.x) * inv, bf_hi(a.x) * inv), pack_bf16(bf_lo(a.y) * inv, bf_hi(a.y) * inv),
                           pack_bf16(bf_lo(a.z) * inv, bf_hi(a.z) * inv), pack_bf16(bf_lo(a.w) * inv, bf_hi(a.w) * inv));
    }
#pragma unroll
    for (int ch = 0; ch < 8; ch++) p[ch ^ swz] = g[ch];
    const float dden = -dot * inv;
    *reinterpret_cast<uint16_t*>(dden_slot) = __bfloat16_as_ushort(__float2bfloat16_rn(dden));
    return dden;
}

// The fp32 state lives in TMEM lanes 0..63 (row d, 64 columns + z in column 64); lanes 64..127 hold an
// identical copy (the state product is issued as M = 128 with its 64-row operand block repeated).
// The four compute warps share the conversion to the bf16 operand tile in shared memory (block 0 =
// [64 d][64 e], block 1 = column 0 holds z): thread r takes row d = r % 64, columns 0..31 if r < 64,
// columns 32..63 and z otherwise.  `half` is one 32-column half of the row in registers.
__device__ __forceinline__ void state_half_to_smem(const uint32_t (&h)[32], float z, uint8_t* sState, int r,
                                                   float* zf32 = nullptr) {
    const int d = r & 63, upper = r >> 6;
    uint8_t* row = sState + d * 128;
#pragma unroll
    for (int ch = 0; ch < 4; ch++)
        *reinterpret_cast<uint4*>(row + (((4 * upper + ch) ^ (d & 7)) * 16)) =
            make_uint4(pack_bf16(__uint_as_float(h[8 * ch]), __uint_as_float(h[8 * ch + 1])),
                       pack_bf16(__uint_as_float(h[8 * ch + 2]), __uint_as_float(h[8 * ch + 3])),
                       pack_bf16(__uint_as_float(h[8 * ch + 4]), __uint_as_float(h[8 * ch + 5])),
                       pack_bf16(__uint_as_float(h[8 * ch + 6]), __uint_as_float(h[8 * ch + 7])));
    if (upper) {
        *reinterpret_cast<uint4*>(sState + 8192 + d * 128 + ((d & 7) * 16)) = make_uint4(pack_bf16(z, 0.f), 0u, 0u, 0u);
        if (zf32 != nullptr) zf32[d] = z;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// Called by all four compute warps with `taddr` = the state region at the warp's own TMEM lanes.
__device__ __forceinline__ void state_to_smem(uint32_t taddr, uint8_t* sState, int r, float* zf32 = nullptr) {
    const int upper = r >> 6;
    uint32_t h[32], s2[32];
    tmem_ld32(taddr + 32 * upper, h);
    if (upper) tmem_ld32(taddr + 64, s2);  // column 64 = z; the rest is not used
    tmem_ld_wait();
    state_half_to_smem(h, upper ? __uint_as_float(s2[0]) : 0.f, sState, r, zf32);
}

// ---- sequence groups ---------------------------------------------------------------------------
// When there are fewer batch units than SMs, the sequence of a unit is cut into G groups of `gc`
// chunks and one CTA takes one (unit, group).  A pre-pass (linattn_tc_state.cu) leaves the state sum
// of every group in `gstate` [unit][group][64 rows][GS_ROW floats] (64 columns + z); a CTA starts
// from the sum over the groups before it (prefix states) or after it (suffix states).
constexpr int GS_ROW = 68;  // floats per state row in global memory (16-byte aligned rows)
struct SeqGroups {
    const float* gstate;  // null: one group
    int G, gc;
};
// The initial state of a group: the sum over groups [g0, g1).  Called by all four compute warps: thread
// r seeds its own TMEM lane with row d = r % 64 (both copies must start equal) and writes its half of
// the bf16 operand tile.
__device__ __forceinline__ void init_state_row(const SeqGroups& sg, int unit, int g0, int g1, int r, uint32_t taddr,
                                               uint8_t* sState, float* zf32 = nullptr) {
    const int d = r & 63, upper = r >> 6;
    float acc[GS_ROW];
#pragma unroll
    for (int i = 0; i < GS_ROW; i++) acc[i] = 0.f;
    for (int g = g0; g < g1; g++) {
        const float4* src = reinterpret_cast<const float4*>(sg.gstate + (((int64_t)unit * sg.G + g) * DE + d) * GS_ROW);
#pragma unroll
        for (int i = 0; i < GS_ROW / 4; i++) {
            const float4 v = src[i];
            acc[4 * i] += v.x; acc[4 * i + 1] += v.y; acc[4 * i + 2] += v.z; acc[4 * i + 3] += v.w;
        }
    }
    uint32_t s0[32], s1[32], s2[32];
#pragma unroll
    for (int i = 0; i < 32; i++) {
        s0[i] = __float_as_uint(acc[i]);
        s1[i] = __float_as_uint(acc[32 + i]);
        s2[i] = i == 0 ? __float_as_uint(acc[64]) : 0u;
    }
    tmem_st32(taddr, s0);
    tmem_st32(taddr + 32, s1);
    tmem_st32(taddr + 64, s2);
    tmem_st_wait();
    if (upper) state_half_to_smem(s1, acc[64], sState, r, zf32);
    else state_half_to_smem(s0, 0.f, sState, r, zf32);
}

}  // namespace lintc

// Host side: how a launch is cut into sequence groups (G = 1: not at all), the workspace that takes,
// and the pre-pass that fills the group states.
struct LinGroupPlan {
    int G, gc;           // groups per unit, chunks per group
    size_t state_bytes;  // one set of group states
};
LinGroupPlan linattn_tc_plan(int B, int S);
// mode 0: prefix states sum phiK (x) [V | 1] of groups 0..G-2; mode 1: suffix states
// sum phiQ (x) [dnum | dden] of groups 1..G-1 (step 1 fused: needs O, dO, den).
int linattn_tc_group_states(int mode, const LinGroupPlan& plan, int B, int S, int map_elu, const void* A, const void* Bm,
                            const void* O, const float* den, float* gstate, cudaStream_t st);

}  // namespace cxxattn
