/* cxxattn — B200 (sm_100a) attention kernels behind CXX-GPT's kernel entry points.
 *
 * C-ABI of libcxxattn.so.  Every function takes plain device (or, for the *_host functions,
 * host) pointers and sizes, launches on the given CUDA stream without synchronising (the
 * *_host functions synchronise before returning), never allocates device memory unless stated,
 * never aborts, and returns CXXATTN_OK or a negative error code (cxxattn_strerror()).
 *
 * Citations name the reference interface each entry point replaces, as
 * file:line inside the CXX-GPT source tree ("ts.cuh" = src/TwoStage/two_stage_cuda_kernels.cuh,
 * "ts.cu" the matching .cu, "lin.cuh"/"lin.cu" = src/LinearAttention/linear_cuda_kernels.cuh/.cu).
 *
 * Layouts (all row-major):
 *   softmax MHA   Q,K,V,O,dO,dQ,dK,dV : (B*S, H*Dh); element (b,s,h,c) at ((b*S+s)*H+h)*Dh+c
 *                 (ts.cuh:13-15), or any layout given by the element strides in the descriptor.
 *                 lse : (B, H, S) float, natural-log-sum-exp of the scaled causal scores.
 *   linear attn   Q,K,dQ,dK,z_cache : (B*S, D);  V,O,dO,dV,dnum : (B*S, E);  den,dden : (B*S).
 *                 Multi-head tensors are passed with heads folded into B (layout [B,H,S,Dh]).
 */
#ifndef CXXATTN_H_
#define CXXATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Opaque CUDA stream handle (cudaStream_t); NULL is the legacy default stream, which is the
 * stream the reference launches on (ts.cu:44, lin.cu:93). */
typedef void* cxxattn_stream_t;

enum {
    CXXATTN_OK = 0,
    CXXATTN_ERR_INVALID = -1,     /* null pointer, zero/negative size, bad enum               */
    CXXATTN_ERR_UNSUPPORTED = -2, /* valid request that no kernel of this build covers        */
    CXXATTN_ERR_WORKSPACE = -3,   /* workspace pointer null or smaller than *_workspace_bytes */
    CXXATTN_ERR_CUDA = -4,        /* a CUDA runtime call failed (launch, copy, attribute)     */
    CXXATTN_ERR_TIMEOUT = -5,     /* a bounded device-side wait gave up (status word set)     */
    CXXATTN_ERR_ALIGNMENT = -6,   /* pointer or stride not aligned as the chosen kernel needs */
    CXXATTN_ERR_TOO_LARGE = -7    /* size beyond a stated fixed maximum                       */
};

enum { CXXATTN_F32 = 0, CXXATTN_BF16 = 1 };

/* feature map applied to Q and K inside the linear-attention kernels */
enum {
    CXXATTN_MAP_NONE = 0, /* inputs are already mapped (linear_cuda::*, lin.cuh:11-37)        */
    CXXATTN_MAP_ELU1 = 1  /* phi(x) = x > 0 ? x + 1 : exp(x) fused (two_stage_cuda, ts.cu:928) */
};

/* Softmax MHA problem.  dtype F32 selects the exact fp32 SIMT kernels; dtype BF16 selects the
 * tcgen05 tensor-core kernels (bf16 operands, fp32 accumulation and softmax). */
typedef struct cxxattn_mha_desc {
    int64_t B, S, H, Dh;
    int64_t stride_b, stride_s, stride_h; /* element strides shared by all 8 tensors; all three 0
                                             = reference layout (S*H*Dh, H*Dh, Dh)              */
    int32_t dtype;                        /* CXXATTN_F32 | CXXATTN_BF16                          */
    int32_t reserved;                     /* must be 0                                           */
} cxxattn_mha_desc;

/* Causal linear attention problem. */
typedef struct cxxattn_lin_desc {
    int64_t B, S, D, E;
    int32_t dtype;       /* type of Q,K,V,O,dO,dQ,dK,dV; den, dden, dnum, z_cache are always float */
    int32_t feature_map; /* CXXATTN_MAP_*                                                        */
    int32_t eps_in_den;  /* 0: den = phi(q).z stored, O = num/(den+1e-8)   (ts.cu:971-972)
                            1: den = q.z + 1e-8 stored, O = num/den        (lin.cu:66-75)        */
    int32_t ld_qk;       /* row stride, in elements, of the D-wide tensors (Q, K, dQ, dK, z_cache): 0 = D
                            (dense).  A larger stride addresses the first D columns of wider rows in
                            place: LinearGPT pads its mapped features with zero columns from n_embd to
                            the next power of two (lin.cu:316-323), and a caller that knows it passes
                            D = n_embd, ld_qk = the padded width instead of scanning the zeros.  The
                            columns beyond D are neither read nor written.  fp32, and bf16 with one wide
                            head and feature_map NONE; other kernels want 0 or D.                       */
} cxxattn_lin_desc;

const char* cxxattn_strerror(int code);
/* "major.minor sm_100a" build string. */
const char* cxxattn_version(void);

/* ---- softmax MHA ------------------------------------------------------------------------- */

/* O = softmax_causal(QK^T / sqrt(Dh)) V.  Replaces two_stage_cuda::fused_mha_fwd (ts.cuh:18-20,
 * ts.cu:285-326).  lse may be NULL; when given it receives the row log-sum-exp that
 * cxxattn_mha_bwd can reuse (the reference forward emits none and its backward recomputes). */
int cxxattn_mha_fwd(const cxxattn_mha_desc* desc, const void* Q, const void* K, const void* V,
                    void* O, float* lse, cxxattn_stream_t stream);

/* Bytes of device workspace cxxattn_mha_bwd needs (0 on a bad descriptor). */
size_t cxxattn_mha_bwd_workspace_bytes(const cxxattn_mha_desc* desc, int have_lse);

/* dQ, dK, dV of the above given dO and the stored O; outputs are overwritten.  Replaces
 * two_stage_cuda::fused_mha_bwd (ts.cuh:22-27, ts.cu:830-882).  lse may be NULL: the row
 * statistics are then recomputed from Q,K in a pre-pass, as the reference's backward does. */
int cxxattn_mha_bwd(const cxxattn_mha_desc* desc, const void* Q, const void* K, const void* V,
                    const void* O, const void* dO, const float* lse,
                    void* dQ, void* dK, void* dV,
                    void* workspace, size_t workspace_bytes, cxxattn_stream_t stream);

/* ---- causal linear attention ------------------------------------------------------------- */

/* Workspace shared by all linear-attention entry points of one descriptor. */
size_t cxxattn_linattn_workspace_bytes(const cxxattn_lin_desc* desc);

/* Forward.  Replaces two_stage_cuda::kernel_attn_fwd (ts.cuh:39-44, ts.cu:1133-1185) with
 * feature_map=ELU1, eps_in_den=0 and linear_cuda::causal_linear_attention_fwd (lin.cuh:11-17,
 * lin.cu:81-99) with feature_map=NONE, eps_in_den=1.  z_cache may be NULL (then not written); the
 * bf16 kernels for D = E = 64 do not take one.
 * The reference's S_buf / z_buf scratch arguments have no counterpart: the sequence is cut into
 * chunks whose states live in `workspace`. */
int cxxattn_linattn_fwd(const cxxattn_lin_desc* desc, const void* Q, const void* K, const void* V,
                        void* O, float* den, float* z_cache,
                        void* workspace, size_t workspace_bytes, cxxattn_stream_t stream);

/* Forward for callers that cannot hand over a workspace.  Some hosts of this library run where
 * device allocation is off the table: a plugin called from inside another engine's execution
 * callback, which owns the memory pool and forbids cudaMalloc/cudaFree (both synchronise the
 * device); a real-time loop that may not take the allocator's locks; a process whose whole device
 * memory budget was handed out at start-up.  For them this variant of cxxattn_linattn_fwd (float
 * tensors, same results) keeps its chunk states in a fixed scratch array that is part of the
 * library's device image: cxxattn_linattn_noalloc_capacity() bytes (8 MiB), held on every GPU
 * that loads the library until the process exits.  It calls no cudaMalloc, cudaFree or allocating
 * library routine.
 *   - Limit: with nc = ceil(S/64), B*nc*D*(E+1)*4 bytes (each part rounded up to 256) must fit
 *     the capacity; otherwise CXXATTN_ERR_TOO_LARGE is returned and nothing is launched.
 *   - The first call on each device looks up the array's device address (that device must be
 *     current); make that first call before any stream capture.
 *   - All calls share the one array, which keeps the previous call's contents.  Nothing in it has
 *     to start at zero (every state is rewritten before it is read), but two calls that overlap
 *     on the GPU (different streams, or different host threads) race on it: serialise them.
 * It has no counterpart in the reference, whose wrappers allocate their scratch per call. */
int cxxattn_linattn_fwd_noalloc(const cxxattn_lin_desc* desc, const float* Q, const float* K, const float* V,
                                float* O, float* den, float* z_cache, cxxattn_stream_t stream);
size_t cxxattn_linattn_noalloc_capacity(void);

/* dnum = dO/den, dden = -(dO.O)/den per row.  Replaces two_stage_cuda::kernel_attn_bwd_step1
 * (ts.cuh:46-49, ts.cu:1235-1248) and linear_cuda::causal_linear_attention_bwd_step1
 * (lin.cuh:19-23, lin.cu:136-150).  O and dO are float. */
int cxxattn_linattn_bwd_step1(const float* O, const float* dO, const float* den,
                              float* dnum, float* dden, size_t N, size_t E,
                              cxxattn_stream_t stream);

/* dQ from (dnum, dden).  Replaces two_stage_cuda::kernel_attn_bwd_dQ (ts.cuh:51-55,
 * ts.cu:1408-1453; Q needed for phi') and linear_cuda::causal_linear_attention_bwd_dQ
 * (lin.cuh:25-30, lin.cu:199-215; Q may be NULL).  z_cache may be NULL: the z term is then
 * rebuilt from K.  K, V, dnum, Q, dQ are of desc->dtype: float, or bf16 for one wide head (D and E
 * multiples of 64 other than 64/64; z_cache is then not read); dden and z_cache are float. */
int cxxattn_linattn_bwd_dq(const cxxattn_lin_desc* desc, const void* K, const void* V,
                           const void* dnum, const float* dden, const float* z_cache,
                           const void* Q, void* dQ,
                           void* workspace, size_t workspace_bytes, cxxattn_stream_t stream);

/* dK, dV from (dnum, dden).  Replaces two_stage_cuda::kernel_attn_bwd_dKdV (ts.cuh:57-61,
 * ts.cu:1743-1809) and linear_cuda::causal_linear_attention_bwd_dKdV (lin.cuh:32-37,
 * lin.cu:275-298).  Tensor types as for cxxattn_linattn_bwd_dq. */
int cxxattn_linattn_bwd_dkdv(const cxxattn_lin_desc* desc, const void* Q, const void* K,
                             const void* V, const void* dnum, const float* dden,
                             void* dK, void* dV,
                             void* workspace, size_t workspace_bytes, cxxattn_stream_t stream);

/* Whole backward in one call (step1 + dQ + dK/dV without the dnum/dden/z_cache round trips).
 * Same results as the three calls above; the grouping has no reference counterpart. */
int cxxattn_linattn_bwd(const cxxattn_lin_desc* desc, const void* Q, const void* K, const void* V,
                        const void* O, const void* dO, const float* den,
                        void* dQ, void* dK, void* dV,
                        void* workspace, size_t workspace_bytes, cxxattn_stream_t stream);

/* ---- decoding with carried state ----------------------------------------------------------- */
/* Not in the reference, whose generate() re-runs the whole context through both attention stages
 * for every new token (two_stage_gpt.hpp:458-474).  One call = one new token per batch unit; the
 * results equal the last row of the corresponding forward call on the whole prefix. */

/* Linear stage.  q, k [B, D], v [B, E] are the new token's rows; state_S [B, D, E] and state_z
 * [B, D] (fp32, zero before the first token) are updated in place: z += phi(k), S += phi(k) (x) v;
 * o [B, E] = phi(q)^T S / (phi(q).z + 1e-8); den [B] (may be NULL) as cxxattn_linattn_fwd stores
 * it (desc->eps_in_den).  desc->S is not used; dtype must be CXXATTN_F32.  Row t of
 * kernel_attn_fwd (ts.cu:889-976) / causal_linear_attention_fwd (lin.cu:10-79). */
int cxxattn_linattn_decode_step(const cxxattn_lin_desc* desc, const float* q, const float* k, const float* v,
                                float* state_S, float* state_z, float* o, float* den, cxxattn_stream_t stream);

/* Softmax stage with a key/value cache.  desc->S is the cache capacity; K_cache, V_cache
 * [B, S, H*Dh] fp32 in the reference layout (strides must be 0), rows 0..pos-1 filled by earlier
 * steps.  q, k, v [B, H*Dh] are the new token's rows: k, v are appended at row pos, then
 * o [B, H*Dh] = softmax(q.K[0..pos] / sqrt(Dh)) V[0..pos].  Row pos of fused_mha_fwd
 * (ts.cu:54-125).  Few (batch, head) units are cut along the keys through `workspace`
 * (cxxattn_mha_decode_workspace_bytes, sized for the capacity; 0 when never needed). */
size_t cxxattn_mha_decode_workspace_bytes(const cxxattn_mha_desc* desc);
int cxxattn_mha_decode_step(const cxxattn_mha_desc* desc, const float* q, const float* k, const float* v,
                            float* K_cache, float* V_cache, int64_t pos, float* o, void* workspace,
                            size_t workspace_bytes, cxxattn_stream_t stream);

/* ---- elementwise neighbours that share the reference headers ------------------------------ */

/* phi[n,d] = ELU(x[n,d])+1 for d<E, 0 for E<=d<D.  linear_cuda::phi_elu_forward (lin.cuh:39-42,
 * lin.cu:327-340). */
int cxxattn_phi_elu_fwd(const float* x, float* phi, size_t N, size_t D, size_t E,
                        cxxattn_stream_t stream);
/* dx[n,e] = dphi[n,e] * (x>0 ? 1 : exp(x)).  linear_cuda::phi_elu_backward (lin.cuh:44-46,
 * lin.cu:366-378). */
int cxxattn_phi_elu_bwd(const float* dphi, const float* x, float* dx, size_t N, size_t D, size_t E,
                        cxxattn_stream_t stream);
/* In-place rotary embedding of Q and/or K (either may be NULL, they may alias: the rotation is
 * then applied twice, as the reference kernel does).  sign=+1: two_stage_cuda::rope_fwd,
 * sign=-1: rope_bwd (ts.cuh:72-76, ts.cu:1820-1880). */
int cxxattn_rope(float* Q, float* K, size_t B, size_t S, size_t D, size_t head_dim, float sign,
                 cxxattn_stream_t stream);
/* Rotary embedding fused with the type conversion either side of the tensor-core kernels:
 * dst = rope(src, sign) out of place, src and dst each CXXATTN_F32 or CXXATTN_BF16, one tensor
 * [B*S, D] per call.  Stands for two_stage_cuda::rope_fwd followed by the fp32 -> bf16 conversion
 * of Q or K (sign=+1; two_stage_gpt.hpp:102,113), and for the bf16 -> fp32 conversion of dQ or dK
 * followed by rope_bwd (sign=-1; two_stage_gpt.hpp:160,174).  head_dim must be a multiple of 4
 * and divide D; 16-byte aligned pointers; src and dst must not overlap. */
int cxxattn_rope_cast(const void* src, int src_dtype, void* dst, int dst_dtype, size_t B, size_t S, size_t D,
                      size_t head_dim, float sign, cxxattn_stream_t stream);
/* The same for two tensors of one shape in one launch, as the reference rotates Q and K together
 * (two_stage_cuda::rope_fwd(Q, K, ...), ts.cuh:72-79): dst0 = rope(src0), dst1 = rope(src1). */
int cxxattn_rope_cast_pair(const void* src0, const void* src1, int src_dtype, void* dst0, void* dst1, int dst_dtype,
                           size_t B, size_t S, size_t D, size_t head_dim, float sign, cxxattn_stream_t stream);
/* erf-GELU (deriv=0) and its derivative (deriv=1).  two_stage_cuda::gelu_exact /
 * gelu_exact_deriv (ts.cuh:84-85, ts.cu:1888-1924). */
int cxxattn_gelu_exact(const float* A, float* C, size_t n, int deriv, cxxattn_stream_t stream);
/* Dense element-wise conversion between CXXATTN_F32 and CXXATTN_BF16 (round to nearest even), for
 * callers that hold the reference's fp32 tensors and want the tensor-core kernels; 16-byte aligned
 * pointers. */
int cxxattn_cast(const void* src, int src_dtype, void* dst, int dst_dtype, size_t n, cxxattn_stream_t stream);

/* ---- the optimiser step of the data-parallel training step ----------------------------------- */

/* One fused pass over flat fp32 buffers of n elements (16-byte aligned): g = grad * grad_scale (1/world
 * after an all-reduce that summed the ranks' gradients; grad itself is not modified), then AdamW as
 * the reference's optimiser applies it, gpt_cuda::adamw_step with the factors AdamW::step() passes
 * (gpt_cuda_kernels.cu:488-512, gpt_gpt.hpp:273-286):
 *   m = beta1 m + (1-beta1) g;  v = beta2 v + (1-beta2) g^2;
 *   param -= lr sqrt(1-beta2^step)/(1-beta1^step) * m / (sqrt(v) + eps sqrt(1-beta2^step)) + lr weight_decay param
 * step counts from 1.  If grad_norm_sq is not NULL, the sum of g^2 is ADDED to that device float
 * (clear it first); the reference computes it per parameter in a kernel of its own with an
 * allocation and a blocking copy (gpt_cuda::grad_norm_squared, gpt_cuda_kernels.cu:517-547). */
int cxxattn_adamw_step(float* param, const float* grad, float* m, float* v, size_t n, float grad_scale, float lr,
                       float beta1, float beta2, float weight_decay, float eps, int step, float* grad_norm_sq,
                       cxxattn_stream_t stream);

/* The same step for mixed-precision training: the gradient is bf16 (n elements, 16-byte aligned), the fp32
 * master parameters and moments are updated as above, and the bf16 working copy param_bf16 (8-byte
 * aligned) that the forward and backward passes read is rewritten in the same pass. */
int cxxattn_adamw_step_mixed(float* param, const void* grad_bf16, float* m, float* v, void* param_bf16, size_t n,
                             float grad_scale, float lr, float beta1, float beta2, float weight_decay, float eps,
                             int step, float* grad_norm_sq, cxxattn_stream_t stream);

/* The gradient exchange and the optimiser step of `world` data-parallel ranks (one process per GPU) as
 * one kernel over peer memory, in place of an all-reduce followed by cxxattn_adamw_step[_mixed].  Rank
 * `rank` owns elements [lo, lo + count) of the flat buffers (multiples of 8 elements for CXXATTN_BF16,
 * of 4 for CXXATTN_F32; count may be 0).  grads[r] / params[r], r = 0..world-1 (at most 16), are device
 * addresses, valid on the calling rank's GPU, of rank r's whole gradient buffer and of the whole
 * parameter buffer its forward pass reads, both of `dtype` (16-byte aligned; the calling rank's own
 * buffers by their local address, the others' as mapped by cxxattn_peer_open).  The kernel sums the
 * ranks' gradients of the shard in fp32, applies grad_scale (1/world) and AdamW as above to the fp32
 * master parameters and moments of the shard (param_shard, m_shard, v_shard: `count` floats each), and
 * writes the updated values as `dtype` into params[r] of every rank.  grad_norm_sq receives the shard's
 * share of the squared gradient norm (added).  The caller orders the call between two barriers over the
 * ranks: after every rank's gradients are final, and before any rank reads its parameters again.  The
 * kernel itself waits for nothing and uses plain loads and stores.  The reference trains on one GPU and
 * has no counterpart. */
int cxxattn_adamw_step_exchange(float* param_shard, float* m_shard, float* v_shard, const void* const* grads,
                                void* const* params, int dtype, int world, int rank, size_t lo, size_t count,
                                float grad_scale, float lr, float beta1, float beta2, float weight_decay, float eps,
                                int step, float* grad_norm_sq, cxxattn_stream_t stream);

/* Column sums out[c] = sum_r X[r][c] of a dense row-major matrix (rows x cols, CXXATTN_F32 or CXXATTN_BF16,
 * cols a multiple of 4 / 8, X 16-byte aligned), accumulated in fp32: the bias gradient of a linear layer
 * (TensorN::cuda::sum_axis(dout, 0) in the reference's Linear::backward, gpt_gpt.hpp:111).  `workspace`
 * (cxxattn_colsum_workspace_bytes(cols), 16-byte aligned) must be all zero before the first call; every
 * call leaves it all zero, so one buffer cleared once serves all later calls on the same stream (calls
 * sharing a workspace must not overlap).  The order of the fp32 additions is not fixed. */
size_t cxxattn_colsum_workspace_bytes(size_t cols);
int cxxattn_colsum(const void* X, int dtype, void* out, size_t rows, size_t cols, void* workspace, size_t workspace_bytes,
                   cxxattn_stream_t stream);

/* LayerNorm backward over rows of `cols` elements (gpt_cuda::layernorm_backward, gpt_cuda_kernels.cu:250-320):
 * with xhat = (x - mean[r]) rstd[r] and g = dy gamma,
 *   dx = rstd (g - (sum_c g + xhat sum_c g xhat) / cols),  dgamma[c] = sum_r dy xhat,  dbeta[c] = sum_r dy.
 * dy, x, dx (rows x cols), gamma, dgamma, dbeta (cols) are `dtype` (CXXATTN_F32 / CXXATTN_BF16; cols a multiple
 * of 4 / 8; dy, x, gamma, dx 16-byte aligned), mean and rstd are fp32 as the forward pass saved them; sums are
 * formed in fp32.  dgamma and dbeta are OVERWRITTEN (the reference adds into them).  `workspace`
 * (cxxattn_layernorm_bwd_workspace_bytes(cols), 16-byte aligned): all zero before the first call, left all
 * zero by every call; calls sharing one must not overlap.  The order of the fp32 additions is not fixed. */
size_t cxxattn_layernorm_bwd_workspace_bytes(size_t cols);
int cxxattn_layernorm_bwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, void* dx,
                          void* dgamma, void* dbeta, size_t rows, size_t cols, int dtype, void* workspace,
                          size_t workspace_bytes, cxxattn_stream_t stream);

/* Device buffers that other processes' GPUs of the same machine can map (CUDA IPC): _alloc / _free own
 * the memory, _export fills the handle another process passes to _open, which returns the address the
 * buffer has in the opening process (peer access is enabled as needed); _close unmaps it.  A handle
 * cannot be opened by the process that exported it. */
#define CXXATTN_PEER_HANDLE_BYTES 64
int cxxattn_peer_alloc(size_t bytes, void** ptr);
int cxxattn_peer_free(void* ptr);
int cxxattn_peer_export(const void* ptr, unsigned char handle[CXXATTN_PEER_HANDLE_BYTES]);
int cxxattn_peer_open(const unsigned char handle[CXXATTN_PEER_HANDLE_BYTES], void** ptr);
int cxxattn_peer_close(void* ptr);

/* ---- host-buffer entry points ------------------------------------------------------------- */

/* Softmax MHA forward + backward on HOST tensors in the reference layout (what kernel_test.cpp
 * does around fused_mha_fwd / fused_mha_bwd with fromTensor / toTensor, kernel_test.cpp:225-249):
 * the plan owns device buffers for up to four chunks of `batch_per_chunk` batch items
 * (allocated by _create, freed by _destroy) and pipelines copy-in, kernels and copy-out across
 * chunks.  cxxattn_mha_fwd_bwd_host returns after all results are in the host buffers. */
typedef struct cxxattn_host_plan cxxattn_host_plan;
int cxxattn_host_plan_create(cxxattn_host_plan** out, const cxxattn_mha_desc* desc, int batch_per_chunk);
void cxxattn_host_plan_destroy(cxxattn_host_plan* plan);
int cxxattn_mha_fwd_bwd_host(cxxattn_host_plan* plan, const void* hQ, const void* hK, const void* hV,
                             const void* hdO, void* hO, void* hdQ, void* hdK, void* hdV);

/* The same for causal linear attention: forward + fused backward on HOST tensors (what
 * kernel_test.cpp does around kernel_attn_fwd / _bwd_step1 / _bwd_dQ / _bwd_dKdV,
 * kernel_test.cpp:266-292), chunked over the units of desc->B.  hQ, hK, hdQ, hdK are (B*S, D),
 * hV, hdO, hO, hdV (B*S, E) of desc->dtype, hden (B*S) float.  Both *_host calls return
 * CXXATTN_ERR_TIMEOUT when a device-side wait gave up during the call, and refuse a plan made on
 * another device than the current one. */
typedef struct cxxattn_lin_host_plan cxxattn_lin_host_plan;
int cxxattn_lin_host_plan_create(cxxattn_lin_host_plan** out, const cxxattn_lin_desc* desc, int units_per_chunk);
void cxxattn_lin_host_plan_destroy(cxxattn_lin_host_plan* plan);
int cxxattn_linattn_fwd_bwd_host(cxxattn_lin_host_plan* plan, const void* hQ, const void* hK, const void* hV,
                                 const void* hdO, void* hO, float* hden, void* hdQ, void* hdK, void* hdV);

/* ---- status and diagnostics (no reference counterpart) ------------------------------------- */

/* Synchronises `stream`, then reports whether any tensor-core kernel launched so far on the
 * current device gave up a bounded device-side wait (CXXATTN_ERR_TIMEOUT, and the flag is
 * cleared) or not (CXXATTN_OK).  Results of a launch that timed out are undefined. */
int cxxattn_sync_status(cxxattn_stream_t stream);

/* The wait site (a small kernel-specific number, for bug reports) of the last timeout that
 * cxxattn_sync_status reported in this process; 0 if none. */
int cxxattn_last_timeout_site(void);

/* ---- run-time options (no reference counterpart) --------------------------------------------- */

/* Process-wide switches that override a choice the launch paths otherwise make from the problem
 * size.  They are read at every call (no environment variable is consulted anywhere in the
 * library) and may be set from any thread; results are the same under every setting, only the
 * schedule changes. */
enum {
    CXXATTN_OPT_FWD_LATE_WAIT = 0,  /* bf16 softmax forward: where a softmax warp waits for the PV product
                                       of the step before.  -1 the library's choice (default; today 1),
                                       0 before the exponentials, 1 after half of them                 */
    CXXATTN_OPT_BWD_PERSISTENT = 1, /* bf16 softmax backward: -1 by sequence length (default), 1 one
                                       persistent CTA per SM drawing (key tile, batch*head) items,
                                       0 one CTA per item                                               */
    CXXATTN_OPT_LIN_GROUPS = 2,     /* bf16 linear attention: sequence groups per unit; 0 cost model
                                       (default), G > 0 forces G (rounded so that no group is empty)    */
    CXXATTN_OPT_LIN_SIDE_STREAM = 3,/* bf16 linear backward: 1 (default) the suffix-state pre-pass runs on
                                       a library-owned side stream beside the dQ pass, 0 in line        */
    CXXATTN_OPT_COUNT_ = 4
};
/* CXXATTN_ERR_INVALID for an unknown option or a value outside the option's range. */
int cxxattn_set_option(int option, int value);
int cxxattn_get_option(int option, int* value);

/* ---- threads ---------------------------------------------------------------------------------- */
/* Host calls may be made from several threads, also for the same device: what the library caches
 * per device (kernel attributes, SM count, symbol addresses) is kept in atomics and is the same
 * whichever thread fills it.  Work on the GPU is ordered by the streams the caller passes, with
 * three exceptions that the caller must serialise per device: calls that share one workspace,
 * cxxattn_linattn_fwd_noalloc (one scratch array), and cxxattn_sync_status (one status word). */

#ifdef __cplusplus
}
#endif
#endif /* CXXATTN_H_ */
