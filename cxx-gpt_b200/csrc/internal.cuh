// Internal declarations shared by the translation units of libcxxattn.so.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <atomic>
#include <cstddef>
#include <cstdint>
#include "cxxattn.h"
#include "cxxattn_diag.h"

namespace cxxattn {

// Softmax MHA problem as the kernels see it (strides resolved, in elements).
struct MhaShape {
    int B, S, H, Dh;
    int64_t sb, ss, sh;
    float scale;  // 1/sqrt(Dh)
};

inline int check_launch() {
    return cudaGetLastError() == cudaSuccess ? CXXATTN_OK : CXXATTN_ERR_CUDA;
}

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// ---- per-device state shared by the launch paths ----
// Host calls may come from several threads at once.  Everything a launch path caches per device
// (function attributes set, SM count, symbol addresses) is a value that every thread would compute
// identically, kept in relaxed atomics: a race only repeats the look-up.
constexpr int kMaxDevices = 64;
// The current device, or -1 when it cannot be read or lies beyond kMaxDevices.
inline int current_device() {
    int d = -1;
    return cudaGetDevice(&d) == cudaSuccess && d >= 0 && d < kMaxDevices ? d : -1;
}
// Streaming multiprocessors of the current device (148 when the attribute cannot be read).
int sm_count();
// One flag per device: `claim()` is true when `done()` has not yet been called for the current device.
struct OncePerDevice {
    std::atomic<bool> set[kMaxDevices];
    bool pending(int dev) const { return dev < 0 || !set[dev].load(std::memory_order_relaxed); }
    void done(int dev) { if (dev >= 0) set[dev].store(true, std::memory_order_relaxed); }
};

// ---- run-time options (cxxattn_set_option) ----
int option(int which);

// ---- exact fp32 SIMT softmax MHA (mha_f32.cu) ----
int mha_f32_fwd(const MhaShape& p, const float* Q, const float* K, const float* V, float* O,
                float* lse, cudaStream_t st);
size_t mha_f32_bwd_workspace(const MhaShape& p, bool have_lse);
int mha_f32_bwd(const MhaShape& p, const float* Q, const float* K, const float* V, const float* O,
                const float* dO, const float* lse, float* dQ, float* dK, float* dV,
                void* ws, size_t ws_bytes, cudaStream_t st);

// ---- tcgen05 bf16 softmax MHA, head dimension 64 (mha_tc_fwd.cu, mha_tc_bwd.cu) ----
bool mha_tc_supported(const MhaShape& p);
int mha_tc_fwd(const MhaShape& p, const void* Q, const void* K, const void* V, void* O, float* lse,
               cudaStream_t st);
size_t mha_tc_bwd_workspace(const MhaShape& p, bool have_lse);
int mha_tc_bwd(const MhaShape& p, const void* Q, const void* K, const void* V, const void* O, const void* dO,
               const float* lse, void* dQ, void* dK, void* dV, void* ws, size_t ws_bytes, cudaStream_t st);

void mha_tc_bwd_set_timing_events(void* start, void* stop);

// ---- tcgen05 bf16 linear attention, D = E = 64 (linattn_tc_fwd.cu) ----
bool linattn_tc_supported(const cxxattn_lin_desc& d);
// Workspace (optional): group states for cutting a unit's sequence over several CTAs; without it
// one CTA walks a whole unit.
size_t linattn_tc_workspace(const cxxattn_lin_desc& d);
int linattn_tc_fwd(const cxxattn_lin_desc& d, const void* Q, const void* K, const void* V, void* O, float* den,
                   void* ws, size_t ws_bytes, cudaStream_t st);
int linattn_tc_bwd(const cxxattn_lin_desc& d, const void* Q, const void* K, const void* V, const void* O,
                   const void* dO, const float* den, void* dQ, void* dK, void* dV, void* ws, size_t ws_bytes,
                   cudaStream_t st);

// ---- tcgen05 bf16 linear attention with one wide head, D and E multiples of 64 (linattn_wide.cu) ----
bool linattn_wide_supported(const cxxattn_lin_desc& d);
size_t linattn_wide_workspace(const cxxattn_lin_desc& d);
int linattn_wide_fwd(const cxxattn_lin_desc& d, const void* Q, const void* K, const void* V, void* O, float* den,
                     float* z_cache, void* ws, size_t ws_bytes, cudaStream_t st);
int linattn_wide_bwd_dq(const cxxattn_lin_desc& d, const void* K, const void* V, const void* dnum, const float* dden,
                        const void* Q, void* dQ, void* ws, size_t ws_bytes, cudaStream_t st);
int linattn_wide_bwd_dkdv(const cxxattn_lin_desc& d, const void* Q, const void* K, const void* V, const void* dnum,
                          const float* dden, void* dK, void* dV, void* ws, size_t ws_bytes, cudaStream_t st);
int linattn_wide_bwd(const cxxattn_lin_desc& d, const void* Q, const void* K, const void* V, const void* O,
                     const void* dO, const float* den, void* dQ, void* dK, void* dV, void* ws, size_t ws_bytes,
                     cudaStream_t st);

// ---- diagnostics (umma_selftest.cu) ----
int umma_selftest(int mode, const void* A, const void* B, float* D, cudaStream_t st);
int wait_selftest(uint64_t limit_ns, cudaStream_t st);
int sync_status(cudaStream_t st);
int last_timeout_site();

// ---- exact fp32 chunk-parallel linear attention (linattn_f32.cu) ----
size_t linattn_f32_workspace(const cxxattn_lin_desc& d);
int linattn_f32_fwd(const cxxattn_lin_desc& d, const float* Q, const float* K, const float* V,
                    float* O, float* den, float* z_cache, void* ws, size_t ws_bytes, cudaStream_t st);
size_t linattn_f32_static_capacity();
int linattn_f32_fwd_static(const cxxattn_lin_desc& d, const float* Q, const float* K, const float* V,
                           float* O, float* den, float* z_cache, cudaStream_t st);
int linattn_f32_bwd_dq(const cxxattn_lin_desc& d, const float* K, const float* V, const float* dnum,
                       const float* dden, const float* z_cache, const float* Q, float* dQ,
                       void* ws, size_t ws_bytes, cudaStream_t st);
int linattn_f32_bwd_dkdv(const cxxattn_lin_desc& d, const float* Q, const float* K, const float* V,
                         const float* dnum, const float* dden, float* dK, float* dV,
                         void* ws, size_t ws_bytes, cudaStream_t st);
int linattn_f32_bwd(const cxxattn_lin_desc& d, const float* Q, const float* K, const float* V,
                    const float* O, const float* dO, const float* den, float* dQ, float* dK, float* dV,
                    void* ws, size_t ws_bytes, cudaStream_t st);

// ---- elementwise (elementwise.cu) ----
int step1_f32(const float* O, const float* dO, const float* den, float* dnum, float* dden,
              size_t N, size_t E, cudaStream_t st);
int phi_elu_fwd(const float* x, float* phi, size_t N, size_t D, size_t E, cudaStream_t st);
int phi_elu_bwd(const float* dphi, const float* x, float* dx, size_t N, size_t D, size_t E, cudaStream_t st);
int rope(float* Q, float* K, size_t B, size_t S, size_t D, size_t hd, float sign, cudaStream_t st);
int gelu_exact(const float* A, float* C, size_t n, int deriv, cudaStream_t st);
int cast(const void* src, int src_dtype, void* dst, int dst_dtype, size_t n, cudaStream_t st);
int linattn_decode_step(const cxxattn_lin_desc& d, const float* q, const float* k, const float* v, float* S, float* z,
                        float* o, float* den, cudaStream_t st);
size_t mha_decode_workspace(const cxxattn_mha_desc& d);
int mha_decode_step(const cxxattn_mha_desc& d, const float* q, const float* k, const float* v, float* Kc, float* Vc,
                    int64_t pos, float* o, void* ws, size_t ws_bytes, cudaStream_t st);
int adamw_fused(float* param, const void* grad, int grad_dtype, float* m, float* v, void* param_copy, size_t n,
                float grad_scale, float lr, float beta1, float beta2, float wd, float eps, int step, float* norm_sq,
                cudaStream_t st);
// ---- gradient exchange + optimiser step over peer memory (adamw_exchange.cu) ----
int adamw_exchange(float* param_shard, float* m_shard, float* v_shard, const void* const* grads, void* const* copies,
                   int dtype, int world, int rank, size_t lo, size_t count, float grad_scale, float lr, float beta1,
                   float beta2, float wd, float eps, int step, float* norm_sq, cudaStream_t st);
int peer_alloc(size_t bytes, void** ptr);
int peer_free(void* ptr);
int peer_export(const void* ptr, unsigned char* handle);
int peer_open(const unsigned char* handle, void** ptr);
int peer_close(void* ptr);
// ---- column sums (colsum.cu) ----
size_t colsum_workspace(size_t cols);
int colsum(const void* X, int dtype, void* out, size_t rows, size_t cols, void* ws, size_t ws_bytes, cudaStream_t st);
// ---- LayerNorm backward (layernorm.cu) ----
size_t layernorm_bwd_workspace(size_t cols);
int layernorm_bwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, void* dx,
                  void* dgamma, void* dbeta, size_t rows, size_t cols, int dtype, void* ws, size_t ws_bytes, cudaStream_t st);
int rope_cast(const void* src, int src_dtype, void* dst, int dst_dtype, size_t B, size_t S, size_t D, size_t hd,
              float sign, cudaStream_t st);
int rope_cast_pair(const void* src0, const void* src1, int src_dtype, void* dst0, void* dst1, int dst_dtype, size_t B,
                   size_t S, size_t D, size_t hd, float sign, cudaStream_t st);

}  // namespace cxxattn
