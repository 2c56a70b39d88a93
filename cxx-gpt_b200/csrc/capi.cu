// extern "C" surface of libcxxattn.so: argument validation and dispatch to the kernel families.
// No device memory is allocated here and nothing is synchronised; a request that no kernel of
// this build covers is an error, never a silent detour.
#include "internal.cuh"
#include <cmath>

using namespace cxxattn;

namespace cxxattn {

namespace {
// defaults: choose by size, choose by size, cost model, side stream on
std::atomic<int> g_options[CXXATTN_OPT_COUNT_] = {{-1}, {-1}, {0}, {1}};
}  // namespace

int option(int which) {
    return which >= 0 && which < CXXATTN_OPT_COUNT_ ? g_options[which].load(std::memory_order_relaxed) : 0;
}

int sm_count() {
    static std::atomic<int> cache[kMaxDevices];
    const int dev = current_device();
    int n = dev >= 0 ? cache[dev].load(std::memory_order_relaxed) : 0;
    if (n <= 0) {
        if (dev < 0 || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        if (dev >= 0) cache[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

}  // namespace cxxattn

namespace {

bool resolve(const cxxattn_mha_desc* d, MhaShape* p) {
    if (d == nullptr || d->B <= 0 || d->S <= 0 || d->H <= 0 || d->Dh <= 0 || d->reserved != 0) return false;
    if (d->B > INT32_MAX || d->S > INT32_MAX || d->H > INT32_MAX || d->Dh > INT32_MAX) return false;
    p->B = (int)d->B; p->S = (int)d->S; p->H = (int)d->H; p->Dh = (int)d->Dh;
    if (d->stride_b == 0 && d->stride_s == 0 && d->stride_h == 0) {
        p->sh = d->Dh; p->ss = d->H * d->Dh; p->sb = d->S * p->ss;
    } else {
        if (d->stride_b <= 0 || d->stride_s <= 0 || d->stride_h <= 0) return false;
        p->sb = d->stride_b; p->ss = d->stride_s; p->sh = d->stride_h;
    }
    p->scale = 1.0f / sqrtf((float)d->Dh);
    return true;
}

bool lin_ok(const cxxattn_lin_desc* d) {
    return d != nullptr && d->B > 0 && d->S > 0 && d->D > 0 && d->E > 0 && (d->ld_qk == 0 || d->ld_qk >= d->D) &&
           d->B <= INT32_MAX && d->S <= INT32_MAX && d->D <= INT32_MAX && d->E <= INT32_MAX &&
           (d->feature_map == CXXATTN_MAP_NONE || d->feature_map == CXXATTN_MAP_ELU1) &&
           (d->eps_in_den == 0 || d->eps_in_den == 1);
}

}  // namespace

extern "C" {

const char* cxxattn_strerror(int code) {
    switch (code) {
        case CXXATTN_OK: return "ok";
        case CXXATTN_ERR_INVALID: return "invalid argument";
        case CXXATTN_ERR_UNSUPPORTED: return "unsupported shape or type for this build";
        case CXXATTN_ERR_WORKSPACE: return "workspace missing or too small";
        case CXXATTN_ERR_CUDA: return "CUDA runtime error";
        case CXXATTN_ERR_TIMEOUT: return "device-side wait timed out";
        case CXXATTN_ERR_ALIGNMENT: return "pointer or stride misaligned";
        case CXXATTN_ERR_TOO_LARGE: return "size beyond a fixed maximum";
        default: return "unknown error";
    }
}

const char* cxxattn_version(void) { return "0.1 sm_100a"; }

int cxxattn_mha_fwd(const cxxattn_mha_desc* desc, const void* Q, const void* K, const void* V,
                    void* O, float* lse, cxxattn_stream_t stream) {
    MhaShape p;
    if (!resolve(desc, &p) || !Q || !K || !V || !O) return CXXATTN_ERR_INVALID;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (desc->dtype == CXXATTN_F32)
        return mha_f32_fwd(p, (const float*)Q, (const float*)K, (const float*)V, (float*)O, lse, st);
    if (desc->dtype == CXXATTN_BF16) return mha_tc_fwd(p, Q, K, V, O, lse, st);
    return CXXATTN_ERR_INVALID;
}

size_t cxxattn_mha_bwd_workspace_bytes(const cxxattn_mha_desc* desc, int have_lse) {
    MhaShape p;
    if (!resolve(desc, &p)) return 0;
    if (desc->dtype == CXXATTN_F32) return mha_f32_bwd_workspace(p, have_lse != 0);
    if (desc->dtype == CXXATTN_BF16 && mha_tc_supported(p)) return mha_tc_bwd_workspace(p, have_lse != 0);
    return 0;
}

int cxxattn_mha_bwd(const cxxattn_mha_desc* desc, const void* Q, const void* K, const void* V,
                    const void* O, const void* dO, const float* lse, void* dQ, void* dK, void* dV,
                    void* workspace, size_t workspace_bytes, cxxattn_stream_t stream) {
    MhaShape p;
    if (!resolve(desc, &p) || !Q || !K || !V || !O || !dO || !dQ || !dK || !dV) return CXXATTN_ERR_INVALID;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (desc->dtype == CXXATTN_F32)
        return mha_f32_bwd(p, (const float*)Q, (const float*)K, (const float*)V, (const float*)O,
                           (const float*)dO, lse, (float*)dQ, (float*)dK, (float*)dV,
                           workspace, workspace_bytes, st);
    if (desc->dtype == CXXATTN_BF16)
        return mha_tc_bwd(p, Q, K, V, O, dO, lse, dQ, dK, dV, workspace, workspace_bytes, st);
    return CXXATTN_ERR_INVALID;
}

size_t cxxattn_linattn_workspace_bytes(const cxxattn_lin_desc* desc) {
    if (!lin_ok(desc)) return 0;
    if (desc->dtype == CXXATTN_F32) return linattn_f32_workspace(*desc);
    if (desc->dtype == CXXATTN_BF16)
        return linattn_tc_supported(*desc) ? linattn_tc_workspace(*desc) : linattn_wide_workspace(*desc);
    return 0;
}

int cxxattn_linattn_fwd(const cxxattn_lin_desc* desc, const void* Q, const void* K, const void* V,
                        void* O, float* den, float* z_cache, void* workspace, size_t workspace_bytes,
                        cxxattn_stream_t stream) {
    if (!lin_ok(desc) || !Q || !K || !V || !O || !den) return CXXATTN_ERR_INVALID;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (desc->dtype == CXXATTN_F32)
        return linattn_f32_fwd(*desc, (const float*)Q, (const float*)K, (const float*)V, (float*)O, den,
                               z_cache, workspace, workspace_bytes, st);
    if (desc->dtype == CXXATTN_BF16) {
        if (linattn_tc_supported(*desc)) {
            if (z_cache != nullptr) return CXXATTN_ERR_UNSUPPORTED;  // D = E = 64 keeps z on chip
            return linattn_tc_fwd(*desc, Q, K, V, O, den, workspace, workspace_bytes, st);
        }
        return linattn_wide_fwd(*desc, Q, K, V, O, den, z_cache, workspace, workspace_bytes, st);
    }
    return CXXATTN_ERR_INVALID;
}

int cxxattn_linattn_fwd_noalloc(const cxxattn_lin_desc* desc, const float* Q, const float* K, const float* V,
                                float* O, float* den, float* z_cache, cxxattn_stream_t stream) {
    if (!lin_ok(desc) || !Q || !K || !V || !O || !den) return CXXATTN_ERR_INVALID;
    if (desc->dtype != CXXATTN_F32) return CXXATTN_ERR_UNSUPPORTED;
    return linattn_f32_fwd_static(*desc, Q, K, V, O, den, z_cache, static_cast<cudaStream_t>(stream));
}

size_t cxxattn_linattn_noalloc_capacity(void) { return linattn_f32_static_capacity(); }

int cxxattn_linattn_bwd_step1(const float* O, const float* dO, const float* den, float* dnum,
                              float* dden, size_t N, size_t E, cxxattn_stream_t stream) {
    if (!O || !dO || !den || !dnum || !dden || N == 0 || E == 0) return CXXATTN_ERR_INVALID;
    return step1_f32(O, dO, den, dnum, dden, N, E, static_cast<cudaStream_t>(stream));
}

int cxxattn_linattn_bwd_dq(const cxxattn_lin_desc* desc, const void* K, const void* V,
                           const void* dnum, const float* dden, const float* z_cache, const void* Q,
                           void* dQ, void* workspace, size_t workspace_bytes, cxxattn_stream_t stream) {
    if (!lin_ok(desc) || !K || !V || !dnum || !dden || !dQ) return CXXATTN_ERR_INVALID;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (desc->dtype == CXXATTN_BF16)  // one wide head; z_cache is not needed
        return linattn_wide_bwd_dq(*desc, K, V, dnum, dden, Q, dQ, workspace, workspace_bytes, st);
    if (desc->dtype != CXXATTN_F32) return CXXATTN_ERR_INVALID;
    return linattn_f32_bwd_dq(*desc, (const float*)K, (const float*)V, (const float*)dnum, dden, z_cache,
                              (const float*)Q, (float*)dQ, workspace, workspace_bytes, st);
}

int cxxattn_linattn_bwd_dkdv(const cxxattn_lin_desc* desc, const void* Q, const void* K,
                             const void* V, const void* dnum, const float* dden, void* dK, void* dV,
                             void* workspace, size_t workspace_bytes, cxxattn_stream_t stream) {
    if (!lin_ok(desc) || !Q || !K || !V || !dnum || !dden || !dK || !dV) return CXXATTN_ERR_INVALID;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (desc->dtype == CXXATTN_BF16)
        return linattn_wide_bwd_dkdv(*desc, Q, K, V, dnum, dden, dK, dV, workspace, workspace_bytes, st);
    if (desc->dtype != CXXATTN_F32) return CXXATTN_ERR_INVALID;
    return linattn_f32_bwd_dkdv(*desc, (const float*)Q, (const float*)K, (const float*)V, (const float*)dnum, dden,
                                (float*)dK, (float*)dV, workspace, workspace_bytes, st);
}

int cxxattn_linattn_bwd(const cxxattn_lin_desc* desc, const void* Q, const void* K, const void* V,
                        const void* O, const void* dO, const float* den, void* dQ, void* dK, void* dV,
                        void* workspace, size_t workspace_bytes, cxxattn_stream_t stream) {
    if (!lin_ok(desc) || !Q || !K || !V || !O || !dO || !den || !dQ || !dK || !dV) return CXXATTN_ERR_INVALID;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (desc->dtype == CXXATTN_F32)
        return linattn_f32_bwd(*desc, (const float*)Q, (const float*)K, (const float*)V, (const float*)O,
                               (const float*)dO, den, (float*)dQ, (float*)dK, (float*)dV,
                               workspace, workspace_bytes, st);
    if (desc->dtype == CXXATTN_BF16) {
        if (linattn_tc_supported(*desc))
            return linattn_tc_bwd(*desc, Q, K, V, O, dO, den, dQ, dK, dV, workspace, workspace_bytes, st);
        return linattn_wide_bwd(*desc, Q, K, V, O, dO, den, dQ, dK, dV, workspace, workspace_bytes, st);
    }
    return CXXATTN_ERR_INVALID;
}

int cxxattn_phi_elu_fwd(const float* x, float* phi, size_t N, size_t D, size_t E, cxxattn_stream_t stream) {
    if (!x || !phi || N == 0 || D == 0 || E == 0 || E > D) return CXXATTN_ERR_INVALID;
    return phi_elu_fwd(x, phi, N, D, E, static_cast<cudaStream_t>(stream));
}

int cxxattn_phi_elu_bwd(const float* dphi, const float* x, float* dx, size_t N, size_t D, size_t E,
                        cxxattn_stream_t stream) {
    if (!dphi || !x || !dx || N == 0 || D == 0 || E == 0 || E > D) return CXXATTN_ERR_INVALID;
    return phi_elu_bwd(dphi, x, dx, N, D, E, static_cast<cudaStream_t>(stream));
}

int cxxattn_rope(float* Q, float* K, size_t B, size_t S, size_t D, size_t head_dim, float sign,
                 cxxattn_stream_t stream) {
    if ((!Q && !K) || B == 0 || S == 0 || D == 0 || head_dim == 0 || head_dim % 2 || D % head_dim)
        return CXXATTN_ERR_INVALID;
    return rope(Q, K, B, S, D, head_dim, sign, static_cast<cudaStream_t>(stream));
}

int cxxattn_set_option(int option, int value) {
    switch (option) {
        case CXXATTN_OPT_FWD_LATE_WAIT:
        case CXXATTN_OPT_BWD_PERSISTENT:
            if (value < -1 || value > 1) return CXXATTN_ERR_INVALID;
            break;
        case CXXATTN_OPT_LIN_GROUPS:
            if (value < 0 || value > 1024) return CXXATTN_ERR_INVALID;
            break;
        case CXXATTN_OPT_LIN_SIDE_STREAM:
            if (value < 0 || value > 1) return CXXATTN_ERR_INVALID;
            break;
        default:
            return CXXATTN_ERR_INVALID;
    }
    g_options[option].store(value, std::memory_order_relaxed);
    return CXXATTN_OK;
}

int cxxattn_get_option(int option, int* value) {
    if (option < 0 || option >= CXXATTN_OPT_COUNT_ || value == nullptr) return CXXATTN_ERR_INVALID;
    *value = cxxattn::option(option);
    return CXXATTN_OK;
}

int cxxattn_selftest_wait_limit(uint64_t limit_ns, cxxattn_stream_t stream) {
    if (limit_ns < 1000 || limit_ns > 2000000000ull) return CXXATTN_ERR_INVALID;
    return wait_selftest(limit_ns, static_cast<cudaStream_t>(stream));
}

void cxxattn_set_timing_events(void* start_event, void* stop_event) {
    mha_tc_bwd_set_timing_events(start_event, stop_event);
}

int cxxattn_sync_status(cxxattn_stream_t stream) { return sync_status(static_cast<cudaStream_t>(stream)); }
int cxxattn_last_timeout_site(void) { return last_timeout_site(); }

int cxxattn_selftest_umma(int mode, const void* A, const void* B, float* D, cxxattn_stream_t stream) {
    if (!A || !B || !D) return CXXATTN_ERR_INVALID;
    return umma_selftest(mode, A, B, D, static_cast<cudaStream_t>(stream));
}

int cxxattn_cast(const void* src, int src_dtype, void* dst, int dst_dtype, size_t n, cxxattn_stream_t stream) {
    if (!src || !dst || n == 0) return CXXATTN_ERR_INVALID;
    return cast(src, src_dtype, dst, dst_dtype, n, static_cast<cudaStream_t>(stream));
}

int cxxattn_linattn_decode_step(const cxxattn_lin_desc* desc, const float* q, const float* k, const float* v,
                                float* state_S, float* state_z, float* o, float* den, cxxattn_stream_t stream) {
    // desc->S is not used by a decoding step; every other field is held to the bounds of lin_ok()
    if (!desc || !q || !k || !v || !state_S || !state_z || !o) return CXXATTN_ERR_INVALID;
    cxxattn_lin_desc one = *desc;
    one.S = 1;
    if (!lin_ok(&one)) return CXXATTN_ERR_INVALID;
    if (desc->dtype != CXXATTN_F32) return CXXATTN_ERR_UNSUPPORTED;
    return linattn_decode_step(*desc, q, k, v, state_S, state_z, o, den, static_cast<cudaStream_t>(stream));
}

static bool decode_ok(const cxxattn_mha_desc* d) {
    // the kernels index with 32-bit grid dimensions: B*H is one of them
    return d && d->B > 0 && d->S > 0 && d->H > 0 && d->Dh > 0 && d->reserved == 0 && d->stride_b == 0 &&
           d->stride_s == 0 && d->stride_h == 0 && d->B <= INT32_MAX && d->S <= INT32_MAX && d->H <= INT32_MAX &&
           d->Dh <= INT32_MAX && d->B * d->H <= INT32_MAX;
}

size_t cxxattn_mha_decode_workspace_bytes(const cxxattn_mha_desc* desc) {
    return decode_ok(desc) ? mha_decode_workspace(*desc) : 0;
}

int cxxattn_mha_decode_step(const cxxattn_mha_desc* desc, const float* q, const float* k, const float* v,
                            float* K_cache, float* V_cache, int64_t pos, float* o, void* workspace,
                            size_t workspace_bytes, cxxattn_stream_t stream) {
    if (!decode_ok(desc) || !q || !k || !v || !K_cache || !V_cache || !o || pos < 0 || pos >= desc->S)
        return CXXATTN_ERR_INVALID;
    if (desc->dtype != CXXATTN_F32 || desc->Dh > 256) return CXXATTN_ERR_UNSUPPORTED;
    return mha_decode_step(*desc, q, k, v, K_cache, V_cache, pos, o, workspace, workspace_bytes,
                           static_cast<cudaStream_t>(stream));
}

int cxxattn_rope_cast(const void* src, int src_dtype, void* dst, int dst_dtype, size_t B, size_t S, size_t D,
                      size_t head_dim, float sign, cxxattn_stream_t stream) {
    if (!src || !dst || B == 0 || S == 0 || D == 0 || head_dim == 0 || head_dim % 4 || D % head_dim)
        return CXXATTN_ERR_INVALID;
    return rope_cast(src, src_dtype, dst, dst_dtype, B, S, D, head_dim, sign, static_cast<cudaStream_t>(stream));
}

int cxxattn_rope_cast_pair(const void* src0, const void* src1, int src_dtype, void* dst0, void* dst1, int dst_dtype,
                           size_t B, size_t S, size_t D, size_t head_dim, float sign, cxxattn_stream_t stream) {
    if (!src0 || !dst0 || !src1 || !dst1 || B == 0 || S == 0 || D == 0 || head_dim == 0 || head_dim % 4 || D % head_dim)
        return CXXATTN_ERR_INVALID;
    return rope_cast_pair(src0, src1, src_dtype, dst0, dst1, dst_dtype, B, S, D, head_dim, sign,
                          static_cast<cudaStream_t>(stream));
}

int cxxattn_adamw_step(float* param, const float* grad, float* m, float* v, size_t n, float grad_scale, float lr,
                       float beta1, float beta2, float weight_decay, float eps, int step, float* grad_norm_sq,
                       cxxattn_stream_t stream) {
    if (!param || !grad || !m || !v || n == 0 || step < 1 || !(beta1 >= 0.f && beta1 < 1.f) ||
        !(beta2 >= 0.f && beta2 < 1.f) || !(eps > 0.f))
        return CXXATTN_ERR_INVALID;
    return adamw_fused(param, grad, CXXATTN_F32, m, v, nullptr, n, grad_scale, lr, beta1, beta2, weight_decay, eps, step,
                       grad_norm_sq, static_cast<cudaStream_t>(stream));
}

int cxxattn_adamw_step_mixed(float* param, const void* grad_bf16, float* m, float* v, void* param_bf16, size_t n,
                             float grad_scale, float lr, float beta1, float beta2, float weight_decay, float eps,
                             int step, float* grad_norm_sq, cxxattn_stream_t stream) {
    if (!param || !grad_bf16 || !m || !v || !param_bf16 || n == 0 || step < 1 || !(beta1 >= 0.f && beta1 < 1.f) ||
        !(beta2 >= 0.f && beta2 < 1.f) || !(eps > 0.f))
        return CXXATTN_ERR_INVALID;
    return adamw_fused(param, grad_bf16, CXXATTN_BF16, m, v, param_bf16, n, grad_scale, lr, beta1, beta2, weight_decay, eps,
                       step, grad_norm_sq, static_cast<cudaStream_t>(stream));
}

int cxxattn_adamw_step_exchange(float* param_shard, float* m_shard, float* v_shard, const void* const* grads,
                                void* const* params, int dtype, int world, int rank, size_t lo, size_t count,
                                float grad_scale, float lr, float beta1, float beta2, float weight_decay, float eps,
                                int step, float* grad_norm_sq, cxxattn_stream_t stream) {
    if (!grads || !params || (count != 0 && (!param_shard || !m_shard || !v_shard)) || step < 1 ||
        !(beta1 >= 0.f && beta1 < 1.f) || !(beta2 >= 0.f && beta2 < 1.f) || !(eps > 0.f) ||
        (dtype != CXXATTN_F32 && dtype != CXXATTN_BF16))
        return CXXATTN_ERR_INVALID;
    return adamw_exchange(param_shard, m_shard, v_shard, grads, params, dtype, world, rank, lo, count, grad_scale, lr,
                          beta1, beta2, weight_decay, eps, step, grad_norm_sq, static_cast<cudaStream_t>(stream));
}

size_t cxxattn_colsum_workspace_bytes(size_t cols) { return cols ? colsum_workspace(cols) : 0; }

int cxxattn_colsum(const void* X, int dtype, void* out, size_t rows, size_t cols, void* workspace, size_t workspace_bytes,
                   cxxattn_stream_t stream) {
    if (!X || !out || rows == 0 || cols == 0 || (dtype != CXXATTN_F32 && dtype != CXXATTN_BF16)) return CXXATTN_ERR_INVALID;
    return colsum(X, dtype, out, rows, cols, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

size_t cxxattn_layernorm_bwd_workspace_bytes(size_t cols) { return cols ? layernorm_bwd_workspace(cols) : 0; }

int cxxattn_layernorm_bwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, void* dx,
                          void* dgamma, void* dbeta, size_t rows, size_t cols, int dtype, void* workspace,
                          size_t workspace_bytes, cxxattn_stream_t stream) {
    if (!dy || !x || !gamma || !mean || !rstd || !dx || !dgamma || !dbeta || rows == 0 || cols == 0 ||
        (dtype != CXXATTN_F32 && dtype != CXXATTN_BF16))
        return CXXATTN_ERR_INVALID;
    return layernorm_bwd(dy, x, gamma, mean, rstd, dx, dgamma, dbeta, rows, cols, dtype, workspace, workspace_bytes,
                         static_cast<cudaStream_t>(stream));
}

int cxxattn_peer_alloc(size_t bytes, void** ptr) { return peer_alloc(bytes, ptr); }
int cxxattn_peer_free(void* ptr) { return ptr ? peer_free(ptr) : CXXATTN_OK; }
int cxxattn_peer_export(const void* ptr, unsigned char handle[CXXATTN_PEER_HANDLE_BYTES]) { return peer_export(ptr, handle); }
int cxxattn_peer_open(const unsigned char handle[CXXATTN_PEER_HANDLE_BYTES], void** ptr) { return peer_open(handle, ptr); }
int cxxattn_peer_close(void* ptr) { return ptr ? peer_close(ptr) : CXXATTN_OK; }

int cxxattn_gelu_exact(const float* A, float* C, size_t n, int deriv, cxxattn_stream_t stream) {
    if (!A || !C || n == 0) return CXXATTN_ERR_INVALID;
    return gelu_exact(A, C, n, deriv != 0, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
