// Adapter: CXX-GPT's C++ kernel entry points on top of the C-ABI of libcxxattn.so.
//
// Semantics kept from the reference wrappers (two_stage_cuda_kernels.cu:285-326, 830-882, 1133-1185,
// 1235-1248, 1408-1453, 1743-1809, 1859-1924; linear_cuda_kernels.cu:81-99, 136-150, 199-215,
// 275-298, 327-378): launches go to the legacy default stream without synchronising, outputs are
// overwritten, temporary scratch is owned by the callee, and a failure throws std::runtime_error
// (what CHECK_CUDA_ERROR does there).  Unlike the reference, Dh > 256 throws instead of aborting.
// The S_buf / z_buf arguments are accepted and left untouched: the chunked scan keeps its states
// in the adapter's scratch.
#include "cxxgpt_kernels.hpp"

#include <cstdlib>
#include <mutex>
#include <string>
#include <unordered_map>

#include "cxxattn.h"

namespace {

void ok(int rc, const char* what) {
    if (rc != CXXATTN_OK) throw std::runtime_error(std::string(what) + ": " + cxxattn_strerror(rc));
}

// Per-device scratch that only grows; freed at process exit by the driver.
void* scratch(size_t bytes) {
    static void* buf[64] = {};
    static size_t cap[64] = {};
    int dev = 0;
    CHECK_CUDA_ERROR(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) throw std::runtime_error("device index out of range");
    if (cap[dev] < bytes) {
        if (buf[dev]) {
            CHECK_CUDA_ERROR(cudaDeviceSynchronize());
            CHECK_CUDA_ERROR(cudaFree(buf[dev]));
        }
        CHECK_CUDA_ERROR(cudaMalloc(&buf[dev], bytes));
        cap[dev] = bytes;
    }
    return buf[dev];
}

cxxattn_mha_desc mha(size_t B, size_t S, size_t H, size_t Dh) {
    cxxattn_mha_desc d = {};
    d.B = (int64_t)B; d.S = (int64_t)S; d.H = (int64_t)H; d.Dh = (int64_t)Dh;
    d.dtype = CXXATTN_F32;
    return d;
}

cxxattn_lin_desc lin(size_t B, size_t S, size_t D, size_t E, int map, int eps_in_den) {
    cxxattn_lin_desc d = {};
    d.B = (int64_t)B; d.S = (int64_t)S; d.D = (int64_t)D; d.E = (int64_t)E;
    d.dtype = CXXATTN_F32;
    d.feature_map = map;
    d.eps_in_den = eps_in_den;
    return d;
}

}  // namespace

// Opt-in: the kept fp32 signatures run on the bf16 tensor-core kernels (inputs rounded to bf16 on the
// way in, results widened on the way out; 2e-2 instead of 1e-5): the softmax attention for head
// dimension 64, the linear attention for one wide head (D and E multiples of 64 other than 64/64, the
// widths of TwoStageGPT's stage 2 and of LinearGPT).  Everything else stays on the exact fp32 kernels.
// Environment CXXATTN_COMPAT_PRECISION=tensorcore (read by this adapter, not by the library), or
// cxxattn_compat::set_tensorcore(true).
namespace {
int g_tensorcore = -1;
bool tensorcore_on() {
    if (g_tensorcore < 0) {
        const char* e = std::getenv("CXXATTN_COMPAT_PRECISION");
        g_tensorcore = (e != nullptr && std::string(e) == "tensorcore") ? 1 : 0;
    }
    return g_tensorcore == 1;
}
bool tensorcore(size_t Dh) { return tensorcore_on() && Dh == 64; }
bool tensorcore_lin(int64_t D, int64_t E) { return tensorcore_on() && D % 64 == 0 && E % 64 == 0 && !(D == 64 && E == 64); }
size_t blk256(size_t bytes) { return (bytes + 255) / 256 * 256; }
// bf16 copy of an fp32 tensor inside the scratch block
void* to_bf16(const float* src, char*& cursor, size_t n) {
    void* dst = cursor;
    cursor += blk256(n * 2);
    ok(cxxattn_cast(src, CXXATTN_F32, dst, CXXATTN_BF16, n, nullptr), "cxxattn_cast");
    return dst;
}
void* take(char*& cursor, size_t bytes) {
    void* p = cursor;
    cursor += blk256(bytes);
    return p;
}

// (The tensor-core detour converts dense fp32 tensors; descriptors that address padded rows in place stay
// on the exact kernels.)
void lin_fwd(cxxattn_lin_desc d, const float* Q, const float* K, const float* V, float* O, float* den, float* zc) {
    if (d.ld_qk == 0 && tensorcore_lin(d.D, d.E)) {
        d.dtype = CXXATTN_BF16;
        const size_t nD = (size_t)(d.B * d.S * d.D), nE = (size_t)(d.B * d.S * d.E);
        const size_t ws = blk256(cxxattn_linattn_workspace_bytes(&d));
        char* cur = static_cast<char*>(scratch(2 * blk256(nD * 2) + 2 * blk256(nE * 2) + ws));
        void* q = to_bf16(Q, cur, nD);
        void* k = to_bf16(K, cur, nD);
        void* v = to_bf16(V, cur, nE);
        void* o = take(cur, nE * 2);
        ok(cxxattn_linattn_fwd(&d, q, k, v, o, den, zc, cur, ws, nullptr), "cxxattn_linattn_fwd");
        ok(cxxattn_cast(o, CXXATTN_BF16, O, CXXATTN_F32, nE, nullptr), "cxxattn_cast");
        return;
    }
    const size_t n = cxxattn_linattn_workspace_bytes(&d);
    ok(cxxattn_linattn_fwd(&d, Q, K, V, O, den, zc, scratch(n), n, nullptr), "cxxattn_linattn_fwd");
}
void lin_dq(cxxattn_lin_desc d, const float* K, const float* V, const float* dnum, const float* dden,
            const float* zc, const float* Q, float* dQ) {
    if (d.ld_qk == 0 && tensorcore_lin(d.D, d.E)) {
        d.dtype = CXXATTN_BF16;
        const size_t nD = (size_t)(d.B * d.S * d.D), nE = (size_t)(d.B * d.S * d.E);
        const size_t ws = blk256(cxxattn_linattn_workspace_bytes(&d));
        char* cur = static_cast<char*>(scratch(3 * blk256(nD * 2) + 2 * blk256(nE * 2) + ws));
        void* k = to_bf16(K, cur, nD);
        void* v = to_bf16(V, cur, nE);
        void* g = to_bf16(dnum, cur, nE);
        void* q = Q ? to_bf16(Q, cur, nD) : nullptr;
        void* dq = take(cur, nD * 2);
        ok(cxxattn_linattn_bwd_dq(&d, k, v, g, dden, nullptr, q, dq, cur, ws, nullptr), "cxxattn_linattn_bwd_dq");
        ok(cxxattn_cast(dq, CXXATTN_BF16, dQ, CXXATTN_F32, nD, nullptr), "cxxattn_cast");
        return;
    }
    const size_t n = cxxattn_linattn_workspace_bytes(&d);
    ok(cxxattn_linattn_bwd_dq(&d, K, V, dnum, dden, zc, Q, dQ, scratch(n), n, nullptr), "cxxattn_linattn_bwd_dq");
}
void lin_dkdv(cxxattn_lin_desc d, const float* Q, const float* K, const float* V, const float* dnum,
              const float* dden, float* dK, float* dV) {
    if (d.ld_qk == 0 && tensorcore_lin(d.D, d.E)) {
        d.dtype = CXXATTN_BF16;
        const size_t nD = (size_t)(d.B * d.S * d.D), nE = (size_t)(d.B * d.S * d.E);
        const size_t ws = blk256(cxxattn_linattn_workspace_bytes(&d));
        char* cur = static_cast<char*>(scratch(3 * blk256(nD * 2) + 3 * blk256(nE * 2) + ws));
        void* q = to_bf16(Q, cur, nD);
        void* k = to_bf16(K, cur, nD);
        void* v = to_bf16(V, cur, nE);
        void* g = to_bf16(dnum, cur, nE);
        void* dk = take(cur, nD * 2);
        void* dv = take(cur, nE * 2);
        ok(cxxattn_linattn_bwd_dkdv(&d, q, k, v, g, dden, dk, dv, cur, ws, nullptr), "cxxattn_linattn_bwd_dkdv");
        ok(cxxattn_cast(dk, CXXATTN_BF16, dK, CXXATTN_F32, nD, nullptr), "cxxattn_cast");
        ok(cxxattn_cast(dv, CXXATTN_BF16, dV, CXXATTN_F32, nE, nullptr), "cxxattn_cast");
        return;
    }
    const size_t n = cxxattn_linattn_workspace_bytes(&d);
    ok(cxxattn_linattn_bwd_dkdv(&d, Q, K, V, dnum, dden, dK, dV, scratch(n), n, nullptr), "cxxattn_linattn_bwd_dkdv");
}
}  // namespace

namespace cxxattn_compat {
void set_tensorcore(bool on) { g_tensorcore = on ? 1 : 0; }

typedef const TensorN::CudaTensor<float>& In;
typedef TensorN::CudaTensor<float>& Out;

// rotated copy of an fp32 tensor inside the scratch block, in the type the attention kernel takes
static void* rotated(const float* src, char*& cursor, int dtype, size_t B, size_t S, size_t D, size_t Dh) {
    void* dst = cursor;
    cursor += (B * S * D * (dtype == CXXATTN_BF16 ? 2 : 4) + 255) / 256 * 256;
    ok(cxxattn_rope_cast(src, CXXATTN_F32, dst, dtype, B, S, D, Dh, 1.0f, nullptr), "cxxattn_rope_cast");
    return dst;
}

void rope_fused_mha_fwd(In Q, In K, In V, Out O, size_t B, size_t S, size_t H, size_t Dh) {
    cxxattn_mha_desc d = mha(B, S, H, Dh);
    const size_t n = B * S * H * Dh, D = H * Dh;
    if (tensorcore(Dh)) {
        d.dtype = CXXATTN_BF16;
        const size_t blk = (n * 2 + 255) / 256 * 256;
        char* cur = static_cast<char*>(scratch(4 * blk));
        void* q = rotated(Q.device_ptr(), cur, CXXATTN_BF16, B, S, D, Dh);
        void* k = rotated(K.device_ptr(), cur, CXXATTN_BF16, B, S, D, Dh);
        void* v = to_bf16(V.device_ptr(), cur, n);
        void* o = cur;
        ok(cxxattn_mha_fwd(&d, q, k, v, o, nullptr, nullptr), "cxxattn_mha_fwd");
        ok(cxxattn_cast(o, CXXATTN_BF16, O.device_ptr(), CXXATTN_F32, n, nullptr), "cxxattn_cast");
        return;
    }
    const size_t blk = (n * 4 + 255) / 256 * 256;
    char* cur = static_cast<char*>(scratch(2 * blk));
    void* q = rotated(Q.device_ptr(), cur, CXXATTN_F32, B, S, D, Dh);
    void* k = rotated(K.device_ptr(), cur, CXXATTN_F32, B, S, D, Dh);
    ok(cxxattn_mha_fwd(&d, q, k, V.device_ptr(), O.device_ptr(), nullptr, nullptr), "cxxattn_mha_fwd");
}

void rope_fused_mha_bwd(In Q, In K, In V, In O, In dO, Out dQ, Out dK, Out dV, size_t B, size_t S, size_t H,
                        size_t Dh) {
    cxxattn_mha_desc d = mha(B, S, H, Dh);
    const size_t n = B * S * H * Dh, D = H * Dh;
    if (tensorcore(Dh)) {
        d.dtype = CXXATTN_BF16;
        const size_t blk = (n * 2 + 255) / 256 * 256;
        const size_t ws = (cxxattn_mha_bwd_workspace_bytes(&d, 0) + 255) / 256 * 256;
        char* cur = static_cast<char*>(scratch(8 * blk + ws));
        void* q = rotated(Q.device_ptr(), cur, CXXATTN_BF16, B, S, D, Dh);
        void* k = rotated(K.device_ptr(), cur, CXXATTN_BF16, B, S, D, Dh);
        void* v = to_bf16(V.device_ptr(), cur, n);
        void* o = to_bf16(O.device_ptr(), cur, n);
        void* g = to_bf16(dO.device_ptr(), cur, n);
        char* dq = cur;
        char* dk = dq + blk;
        char* dv = dk + blk;
        char* w = dv + blk;
        ok(cxxattn_mha_bwd(&d, q, k, v, o, g, nullptr, dq, dk, dv, w, ws, nullptr), "cxxattn_mha_bwd");
        ok(cxxattn_rope_cast(dq, CXXATTN_BF16, dQ.device_ptr(), CXXATTN_F32, B, S, D, Dh, -1.0f, nullptr),
           "cxxattn_rope_cast");
        ok(cxxattn_rope_cast(dk, CXXATTN_BF16, dK.device_ptr(), CXXATTN_F32, B, S, D, Dh, -1.0f, nullptr),
           "cxxattn_rope_cast");
        ok(cxxattn_cast(dv, CXXATTN_BF16, dV.device_ptr(), CXXATTN_F32, n, nullptr), "cxxattn_cast");
        return;
    }
    const size_t blk = (n * 4 + 255) / 256 * 256;
    const size_t ws = (cxxattn_mha_bwd_workspace_bytes(&d, 0) + 255) / 256 * 256;
    char* cur = static_cast<char*>(scratch(2 * blk + ws));
    void* q = rotated(Q.device_ptr(), cur, CXXATTN_F32, B, S, D, Dh);
    void* k = rotated(K.device_ptr(), cur, CXXATTN_F32, B, S, D, Dh);
    ok(cxxattn_mha_bwd(&d, q, k, V.device_ptr(), O.device_ptr(), dO.device_ptr(), nullptr, dQ.device_ptr(),
                       dK.device_ptr(), dV.device_ptr(), cur, ws, nullptr),
       "cxxattn_mha_bwd");
    ok(cxxattn_rope(dQ.device_ptr(), dK.device_ptr(), B, S, D, Dh, -1.0f, nullptr), "cxxattn_rope");
}
}  // namespace cxxattn_compat

namespace two_stage_cuda {

void fused_mha_fwd(In Q, In K, In V, Out O, size_t B, size_t S, size_t H, size_t Dh) {
    if (tensorcore(Dh)) {
        cxxattn_mha_desc d = mha(B, S, H, Dh);
        d.dtype = CXXATTN_BF16;
        const size_t n = B * S * H * Dh, blk = (n * 2 + 255) / 256 * 256;
        char* cur = static_cast<char*>(scratch(4 * blk));
        void* q = to_bf16(Q.device_ptr(), cur, n);
        void* k = to_bf16(K.device_ptr(), cur, n);
        void* v = to_bf16(V.device_ptr(), cur, n);
        void* o = cur;
        ok(cxxattn_mha_fwd(&d, q, k, v, o, nullptr, nullptr), "cxxattn_mha_fwd");
        ok(cxxattn_cast(o, CXXATTN_BF16, O.device_ptr(), CXXATTN_F32, n, nullptr), "cxxattn_cast");
        return;
    }
    const cxxattn_mha_desc d = mha(B, S, H, Dh);
    ok(cxxattn_mha_fwd(&d, Q.device_ptr(), K.device_ptr(), V.device_ptr(), O.device_ptr(), nullptr, nullptr),
       "cxxattn_mha_fwd");
}

void fused_mha_bwd(In Q, In K, In V, In O, In dO, Out dQ, Out dK, Out dV, size_t B, size_t S, size_t H, size_t Dh) {
    if (tensorcore(Dh)) {
        cxxattn_mha_desc d = mha(B, S, H, Dh);
        d.dtype = CXXATTN_BF16;
        const size_t n = B * S * H * Dh, blk = (n * 2 + 255) / 256 * 256;
        const size_t ws = (cxxattn_mha_bwd_workspace_bytes(&d, 0) + 255) / 256 * 256;
        char* cur = static_cast<char*>(scratch(8 * blk + ws));
        void* q = to_bf16(Q.device_ptr(), cur, n);
        void* k = to_bf16(K.device_ptr(), cur, n);
        void* v = to_bf16(V.device_ptr(), cur, n);
        void* o = to_bf16(O.device_ptr(), cur, n);
        void* g = to_bf16(dO.device_ptr(), cur, n);
        char* dq = cur;
        char* dk = dq + blk;
        char* dv = dk + blk;
        char* w = dv + blk;
        // no row statistics in this signature: the library recomputes them, as the reference does
        ok(cxxattn_mha_bwd(&d, q, k, v, o, g, nullptr, dq, dk, dv, w, ws, nullptr), "cxxattn_mha_bwd");
        ok(cxxattn_cast(dq, CXXATTN_BF16, dQ.device_ptr(), CXXATTN_F32, n, nullptr), "cxxattn_cast");
        ok(cxxattn_cast(dk, CXXATTN_BF16, dK.device_ptr(), CXXATTN_F32, n, nullptr), "cxxattn_cast");
        ok(cxxattn_cast(dv, CXXATTN_BF16, dV.device_ptr(), CXXATTN_F32, n, nullptr), "cxxattn_cast");
        return;
    }
    const cxxattn_mha_desc d = mha(B, S, H, Dh);
    const size_t n = cxxattn_mha_bwd_workspace_bytes(&d, 0);
    ok(cxxattn_mha_bwd(&d, Q.device_ptr(), K.device_ptr(), V.device_ptr(), O.device_ptr(), dO.device_ptr(), nullptr,
                       dQ.device_ptr(), dK.device_ptr(), dV.device_ptr(), scratch(n), n, nullptr),
       "cxxattn_mha_bwd");
}

void kernel_attn_fwd(In Q, In K, In V, Out O, Out den_cache, Out z_cache, Out, Out, size_t B, size_t S, size_t D,
                     size_t E) {
    lin_fwd(lin(B, S, D, E, CXXATTN_MAP_ELU1, 0), Q.device_ptr(), K.device_ptr(), V.device_ptr(), O.device_ptr(),
            den_cache.device_ptr(), z_cache.device_ptr());
}

void kernel_attn_bwd_step1(In O, In dO, In den_cache, Out dnum, Out dden, size_t N, size_t E) {
    ok(cxxattn_linattn_bwd_step1(O.device_ptr(), dO.device_ptr(), den_cache.device_ptr(), dnum.device_ptr(),
                                 dden.device_ptr(), N, E, nullptr),
       "cxxattn_linattn_bwd_step1");
}

void kernel_attn_bwd_dQ(In K, In V, In dnum, In dden, In z_cache, In Q, Out dQ, Out, size_t B, size_t S, size_t D,
                        size_t E) {
    lin_dq(lin(B, S, D, E, CXXATTN_MAP_ELU1, 0), K.device_ptr(), V.device_ptr(), dnum.device_ptr(), dden.device_ptr(),
           z_cache.device_ptr(), Q.device_ptr(), dQ.device_ptr());
}

void kernel_attn_bwd_dKdV(In Q, In K, In V, In dnum, In dden, Out dK, Out dV, size_t B, size_t S, size_t D, size_t E) {
    lin_dkdv(lin(B, S, D, E, CXXATTN_MAP_ELU1, 0), Q.device_ptr(), K.device_ptr(), V.device_ptr(), dnum.device_ptr(),
             dden.device_ptr(), dK.device_ptr(), dV.device_ptr());
}

void rope_fwd(Out Q, Out K, size_t B, size_t S, size_t D, size_t head_dim) {
    ok(cxxattn_rope(Q.device_ptr(), K.device_ptr(), B, S, D, head_dim, 1.0f, nullptr), "cxxattn_rope");
}
void rope_bwd(Out dQ, Out dK, size_t B, size_t S, size_t D, size_t head_dim) {
    ok(cxxattn_rope(dQ.device_ptr(), dK.device_ptr(), B, S, D, head_dim, -1.0f, nullptr), "cxxattn_rope");
}
void gelu_exact(In A, Out C) { ok(cxxattn_gelu_exact(A.device_ptr(), C.device_ptr(), A.size(), 0, nullptr), "cxxattn_gelu_exact"); }
void gelu_exact_deriv(In A, Out C) { ok(cxxattn_gelu_exact(A.device_ptr(), C.device_ptr(), A.size(), 1, nullptr), "cxxattn_gelu_exact"); }

}  // namespace two_stage_cuda

// Zero padding of LinearGPT's mapped features.  phi_elu_forward writes phi(x) into the first E columns of
// rows of D = next_pow2(E) and zeros into the rest (linear_cuda_kernels.cu:316-323), and the scan then
// multiplies those zeros: a quarter of the state work at n_embd = 768.  The adapter remembers which
// device tensors its own phi_elu_forward produced; when the scan entry points are handed such tensors
// they run on the first E columns only (row stride D) and the padded columns of the outputs are set to
// the zeros the full computation would give.  For the forward and dQ it is K_phi that decides (a zero
// K column makes the state row, the z entry and the dQ column zero whatever Q holds); dK's padded
// columns also need Q_phi's to be zero.  On by default; CXXATTN_COMPAT_SKIP_PADDING=0 in the environment or
// cxxattn_compat::set_skip_padding(false) turns it off.
namespace {
std::mutex g_pad_mutex;
std::unordered_map<const void*, std::pair<size_t, size_t>> g_padded;  // device pointer -> (D, E) of phi_elu_forward
int g_skip_padding = -1;  // -1: not read yet; CXXATTN_COMPAT_SKIP_PADDING=0 in the environment turns it off
bool skip_padding() {
    if (g_skip_padding < 0) {
        const char* e = std::getenv("CXXATTN_COMPAT_SKIP_PADDING");
        g_skip_padding = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return g_skip_padding == 1;
}

void remember_padded(const void* ptr, size_t D, size_t E) {
    std::lock_guard<std::mutex> lock(g_pad_mutex);
    if (g_padded.size() > 4096) g_padded.clear();
    if (E < D) g_padded[ptr] = {D, E};
    else g_padded.erase(ptr);
}
// The number of leading columns that can be non-zero in a D-wide tensor at ptr: E if this adapter's
// phi_elu_forward wrote it with that D, else D.
size_t live_columns(const void* ptr, size_t D, size_t E) {
    // in tensor-core mode the dense tensors are converted as they are; the zero columns cost little there
    if (!skip_padding() || tensorcore_lin((int64_t)D, (int64_t)E)) return D;
    std::lock_guard<std::mutex> lock(g_pad_mutex);
    auto it = g_padded.find(ptr);
    return (it != g_padded.end() && it->second.first == D) ? it->second.second : D;
}
// columns live..D-1 of N rows := 0
void zero_pad(float* base, size_t N, size_t D, size_t live) {
    if (live < D)
        CHECK_CUDA_ERROR(cudaMemset2DAsync(base + live, D * sizeof(float), 0, (D - live) * sizeof(float), N, nullptr));
}
cxxattn_lin_desc lin_padded(size_t B, size_t S, size_t D, size_t live, size_t E) {
    cxxattn_lin_desc d = lin(B, S, live, E, CXXATTN_MAP_NONE, 1);
    d.ld_qk = live < D ? (int32_t)D : 0;
    return d;
}
}  // namespace

namespace cxxattn_compat {
void set_skip_padding(bool on) { g_skip_padding = on ? 1 : 0; }
}  // namespace cxxattn_compat

namespace linear_cuda {

void causal_linear_attention_fwd(In Q_phi, In K_phi, In V, Out O, Out den_cache, Out z_cache, Out, Out, size_t B,
                                 size_t S, size_t D, size_t E) {
    const size_t live = live_columns(K_phi.device_ptr(), D, E);
    lin_fwd(lin_padded(B, S, D, live, E), Q_phi.device_ptr(), K_phi.device_ptr(), V.device_ptr(),
            O.device_ptr(), den_cache.device_ptr(), z_cache.device_ptr());
    zero_pad(z_cache.device_ptr(), B * S, D, live);
}
void causal_linear_attention_bwd_step1(In O, In dO, In den_cache, Out dnum, Out dden, size_t N, size_t E) {
    ok(cxxattn_linattn_bwd_step1(O.device_ptr(), dO.device_ptr(), den_cache.device_ptr(), dnum.device_ptr(),
                                 dden.device_ptr(), N, E, nullptr),
       "cxxattn_linattn_bwd_step1");
}
void causal_linear_attention_bwd_dQ(In K_phi, In V, In dnum, In dden, In z_cache, Out dQ_phi, Out, size_t B, size_t S,
                                    size_t D, size_t E) {
    const size_t live = live_columns(K_phi.device_ptr(), D, E);
    lin_dq(lin_padded(B, S, D, live, E), K_phi.device_ptr(), V.device_ptr(), dnum.device_ptr(),
           dden.device_ptr(), z_cache.device_ptr(), nullptr, dQ_phi.device_ptr());
    zero_pad(dQ_phi.device_ptr(), B * S, D, live);
}
void causal_linear_attention_bwd_dKdV(In Q_phi, In K_phi, In V, In dnum, In dden, Out dK_phi, Out dV, size_t B,
                                      size_t S, size_t D, size_t E) {
    // both must be padded the same way: dK's padded columns are zero only if Q_phi's are
    const size_t lk = live_columns(K_phi.device_ptr(), D, E), lq = live_columns(Q_phi.device_ptr(), D, E);
    const size_t live = lk == lq ? lk : D;
    lin_dkdv(lin_padded(B, S, D, live, E), Q_phi.device_ptr(), K_phi.device_ptr(), V.device_ptr(),
             dnum.device_ptr(), dden.device_ptr(), dK_phi.device_ptr(), dV.device_ptr());
    zero_pad(dK_phi.device_ptr(), B * S, D, live);
}
void phi_elu_forward(In x, Out phi, size_t D, size_t E) {
    ok(cxxattn_phi_elu_fwd(x.device_ptr(), phi.device_ptr(), x.shape()[0], D, E, nullptr), "cxxattn_phi_elu_fwd");
    remember_padded(phi.device_ptr(), D, E);
}
void phi_elu_backward(In dphi, In x, Out dx, size_t D, size_t E) {
    ok(cxxattn_phi_elu_bwd(dphi.device_ptr(), x.device_ptr(), dx.device_ptr(), dphi.shape()[0], D, E, nullptr),
       "cxxattn_phi_elu_bwd");
}

}  // namespace linear_cuda
