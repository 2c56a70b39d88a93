// Single-tile checks of the tcgen05 operand conventions the attention kernels rely on.  One CTA,
// one 128-row tile, three modes; the host compares the result with a plain matrix product.
//
//   mode 0  D[128x128] = A[128x64] * B[128x64]^T      both operands K-major from TMA tiles (QK^T)
//   mode 1  D[128x64]  = P[128x128] * V[128x64]        P bf16 in TMEM (stored by the threads), V
//                                                      MN-major from a TMA tile (PV)
//   mode 2  D[128x64]  = A[128(k) x 128(m)]^T * B[128(k) x 64]   A written to shared memory by the
//                                                      threads in the MN-major 128-byte-swizzled
//                                                      layout, B MN-major from TMA (dQ = dS K)
#include "internal.cuh"
#include "tc_common.cuh"

namespace cxxattn {
namespace {

using namespace tc;
constexpr int TILE = 128 * 64 * 2;  // bytes of a 128 x 64 bf16 tile

__global__ void __launch_bounds__(128, 1)
umma_selftest_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const __nv_bfloat16* __restrict__ Araw, float* __restrict__ D, int mode, int* status) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full, done;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;             // 2 tiles (mode 2 uses both)
    uint8_t* sB = smem + 2 * TILE;  // 1 tile
    const int warp = threadIdx.x / 32, r = threadIdx.x;
    const Guard guard{&abort_flag, status};

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(&full, 1);
        mbar_init(&done, 1);
        fence_barrier_init();
    }
    if (warp == 0) tmem_alloc(&tmem_slot, 256);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
    const uint32_t COL_P = 128;

    if (threadIdx.x == 0) {
        mbar_expect_tx(&full, mode == 0 ? 2 * TILE : TILE);
        if (mode == 0) tma_load_4d(sA, &tmA, &full, 0, 0, 0, 0);
        tma_load_4d(sB, &tmB, &full, 0, 0, 0, 0);
    }
    if (mode == 1) {
        // row r of P: 128 bf16 -> 64 packed columns of this thread's TMEM lane
        const uint32_t* src = reinterpret_cast<const uint32_t*>(Araw + (size_t)r * 128);
        uint32_t v[32];
        for (int c = 0; c < 2; c++) {
#pragma unroll
            for (int i = 0; i < 32; i++) v[i] = src[c * 32 + i];
            tmem_st32(lane_base + COL_P + 32 * c, v);
            tmem_st_wait();
        }
    } else if (mode == 2) {
        // row r (a K index) of A holds 128 M values: two blocks of 64, each a 128-byte row whose
        // 16-byte chunks are XOR-swizzled with (r % 8).
        const uint4* src = reinterpret_cast<const uint4*>(Araw + (size_t)r * 128);
#pragma unroll
        for (int mb = 0; mb < 2; mb++)
#pragma unroll
            for (int ch = 0; ch < 8; ch++) {
                uint4 v = src[mb * 8 + ch];
                *reinterpret_cast<uint4*>(sA + mb * TILE + r * 128 + ((ch ^ (r & 7)) * 16)) = v;
            }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();

    if (threadIdx.x == 0) {
        tc_fence_after();
        mbar_wait(&full, 0, guard, 901);
        if (mode == 0) {
            for (int k = 0; k < 4; k++)
                umma_ss(tmem, smem_desc_sw128(smem_u32(sA) + 32 * k, 16), smem_desc_sw128(smem_u32(sB) + 32 * k, 16),
                        idesc_bf16(128, 128, 0, 0), k > 0);
        } else if (mode == 1) {
            for (int k = 0; k < 8; k++)
                umma_ts(tmem, tmem + COL_P + 8 * k, smem_desc_sw128(smem_u32(sB) + 2048 * k, 0),
                        idesc_bf16(128, 64, 0, 1), k > 0);
        } else {
            for (int k = 0; k < 8; k++)
                umma_ss(tmem, smem_desc_sw128(smem_u32(sA) + 2048 * k, TILE), smem_desc_sw128(smem_u32(sB) + 2048 * k, 0),
                        idesc_bf16(128, 64, 1, 1), k > 0);
        }
        umma_commit(&done);
    }
    mbar_wait(&done, 0, guard, 902);
    tc_fence_after();
    const int ncols = mode == 0 ? 128 : 64;
    for (int c = 0; c < ncols / 32; c++) {
        uint32_t v[32];
        tmem_ld32(lane_base + 32 * c, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i++) D[(size_t)r * ncols + c * 32 + i] = __uint_as_float(v[i]);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem, 256);
    }
}

// One CTA of 128 threads with tensor memory allocated, as the attention kernels have: every thread
// waits for a barrier phase that no one completes.  The wait (the routine the attention kernels
// use, with `limit_ns` in place of their two seconds) gives up, records site 990, raises the CTA's
// abort flag, and all warps fall through to the common teardown.
__global__ void __launch_bounds__(128, 1) wait_selftest_kernel(uint64_t limit_ns, int* status) {
    __shared__ uint64_t never;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    const int warp = threadIdx.x / 32;
    const Guard guard{&abort_flag, status};
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(&never, 1);
        fence_barrier_init();
    }
    if (warp == 0) tmem_alloc(&tmem_slot, 32);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    mbar_wait_limit(&never, 0, guard, 990, limit_ns);  // no thread ever arrives on `never`
    // a second wait after the abort returns at once (what keeps a kernel with many waits short)
    mbar_wait_limit(&never, 0, guard, 991, limit_ns);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem, 32);
    }
}

}  // namespace

int wait_selftest(uint64_t limit_ns, cudaStream_t st) {
    int* status = status_word();
    if (status == nullptr) return CXXATTN_ERR_CUDA;
    wait_selftest_kernel<<<1, 128, 0, st>>>(limit_ns, status);
    return check_launch();
}

int umma_selftest(int mode, const void* A, const void* B, float* D, cudaStream_t st) {
    if (mode < 0 || mode > 2) return CXXATTN_ERR_INVALID;
    CUtensorMap tmA, tmB;
    // A as a [128 x 64] tile is only loaded by TMA in mode 0; the map is still built (A has at
    // least 128 x 64 elements in every mode).
    if (!make_tmap_bhsd(&tmA, A, 1, 128, 1, 64, 128 * 64, 64, 64, 128) ||
        !make_tmap_bhsd(&tmB, B, 1, 128, 1, 64, 128 * 64, 64, 64, 128))
        return CXXATTN_ERR_CUDA;
    int* status = status_word();
    if (status == nullptr) return CXXATTN_ERR_CUDA;
    const size_t smem = 3 * TILE + 1024;
    if (cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return CXXATTN_ERR_CUDA;
    umma_selftest_kernel<<<1, 128, smem, st>>>(tmA, tmB, static_cast<const __nv_bfloat16*>(A), D, mode, status);
    return check_launch();
}

static std::atomic<int> g_last_site{0};
int last_timeout_site() { return g_last_site.load(std::memory_order_relaxed); }

int sync_status(cudaStream_t st) {
    int* status = status_word();
    if (status == nullptr) return CXXATTN_ERR_CUDA;
    int host = 0;
    if (cudaMemcpyAsync(&host, status, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess) return CXXATTN_ERR_CUDA;
    if (cudaStreamSynchronize(st) != cudaSuccess) return CXXATTN_ERR_CUDA;
    if (host != 0) {
        g_last_site.store(host, std::memory_order_relaxed);
        cudaMemsetAsync(status, 0, sizeof(int), st);
        cudaStreamSynchronize(st);
        return CXXATTN_ERR_TIMEOUT;
    }
    return CXXATTN_OK;
}

}  // namespace cxxattn
