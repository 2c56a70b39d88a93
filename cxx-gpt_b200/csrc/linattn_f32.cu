// Exact fp32 causal linear attention as a chunk-parallel scan, forward and backward.
//
// The reference walks the sequence one timestep at a time inside one CTA per batch item
// (src/TwoStage/two_stage_cuda_kernels.cu:917, 1273, 1622; src/LinearAttention/
// linear_cuda_kernels.cu:35, 173, 243).  Here the sequence is cut into chunks of CH rows and
// every entry point becomes three fully parallel launches:
//
//   1. chunk_state : per chunk, the local state  S_c = X_c^T Y_c  (D x E) and  z_c = X_c^T w
//   2. chunk_scan  : exclusive prefix (forward) or suffix (backward) of the chunk states
//   3. chunk_apply : per chunk,  out_t = sum_{s in chunk, s<=t (or >=t)} score(t,s) c_s
//                                       + a_t . State_prev
//
// All four products of the method share that shape (the last line), so one kernel template
// covers them; `Mode` selects operands, causality direction and epilogue:
//
//   FWD : a=phi(Q) b=phi(K) c=V      state S[d][e]      O   = num/(den+1e-8), den, z_cache
//   DQ  : a=dnum   b=V      c=phi(K) state S[d][e]^T    dQ  = (.. + z_t*dden_t) * phi'(Q)
//   DV  : a=phi(K) b=phi(Q) c=dnum   state S*[d][e]     dV             (s >= t)
//   DK  : a=V      b=dnum   c=phi(Q) state S*[d][e]^T   dK  = (.. + z*) * phi'(K)   (s >= t)
//
// with score(t,s) = a_t.b_s (+ dden_s for DK, + dden_t for DQ when z_cache is not supplied).
// The feature map phi(x) = x>0 ? x+1 : exp(x) is applied while loading (CXXATTN_MAP_ELU1) or
// skipped (CXXATTN_MAP_NONE: inputs are pre-mapped, gradients are w.r.t. the mapped features).
// Arbitrary D and E are handled by zero padding inside shared memory.
#include "internal.cuh"

namespace cxxattn {
namespace {

constexpr int NT = 256;  // 16 x 16 threads, 4 x 4 register tile each
constexpr int CH = 64;   // rows per chunk
constexpr int TI = 32;   // slice of the contracted feature dimension staged per step
constexpr int TJ = 64;   // output feature columns per CTA
constexpr int LDI = TI + 4;
constexpr int LDJ = TJ + 4;

enum Mode { FWD = 0, DQ = 1, DV = 2, DK = 3 };

__device__ __forceinline__ float phi(float x) { return x > 0.f ? x + 1.f : expf(x); }
__device__ __forceinline__ float phi_der(float x) { return x > 0.f ? 1.f : expf(x); }

struct ApplyArgs {
    const float* a;      // [N][I]
    const float* b;      // [N][I]
    const float* c;      // [N][J]
    const float* state;  // [B*nc][D*E] exclusive prefix/suffix of the chunk states
    const float* zstate; // [B*nc][D]   same for z
    const float* dden;   // [N] (DQ, DK)
    const float* zcache; // [N][D] (DQ, optional)
    const float* X;      // [N][J] pre-map input whose phi' scales the output (DQ: Q, DK: K), or null
    float* out;          // [N][J]
    float* den;          // [N]    (FWD)
    float* zc_out;       // [N][D] (FWD, optional)
    int S, D, E, nc;
    int ldd;             // row stride (elements) of the D-wide tensors: Q, K, dQ, dK, z_cache; >= D
    int map;             // CXXATTN_MAP_*
    int eps_in_den;
};

// Loads a [CH][W] slice (columns col0..col0+W-1 of rows row0..) of a dense [.][ld] matrix into
// shared memory with pitch LDS, applying phi when asked; rows >= nrows and columns >= ncols
// become exact zeros (phi(0) = 1 must not leak into the padding).
template <int W, int LDS>
__device__ __forceinline__ void load_slice(float* dst, const float* __restrict__ src, int64_t row0,
                                           int nrows, int ld, int col0, int ncols, bool map) {
    for (int i = threadIdx.x; i < CH * W; i += NT) {
        const int r = i / W, cc = i % W, col = col0 + cc;
        float v = 0.f;
        if (r < nrows && col < ncols) {
            v = src[(row0 + r) * ld + col];
            if (map) v = phi(v);
        }
        dst[r * LDS + cc] = v;
    }
}

// Four CTAs per SM (64 registers, a few spilled words): the kernel alternates between loading a slice
// from global memory and computing on it, so what hides the loads is other CTAs; with the 128
// registers the compiler takes when left alone only two fit and the step was 1.4x slower.
template <int MODE>
__global__ void __launch_bounds__(NT, 4) chunk_apply_kernel(ApplyArgs g) {
    constexpr bool REV = (MODE == DV || MODE == DK);
    constexpr bool STATE_T = (MODE == DQ || MODE == DK);  // state read as [j][i] instead of [i][j]
    const int I = (MODE == FWD || MODE == DV) ? g.D : g.E;
    const int J = (MODE == FWD || MODE == DV) ? g.E : g.D;
    const int ldI = (MODE == FWD || MODE == DV) ? g.ldd : g.E;  // a, b are the D-wide tensors in FWD and DV
    const int ldJ = (MODE == FWD || MODE == DV) ? g.E : g.ldd;  // c, X and the output are in DQ and DK

    // As | Bs | St are live during the loop over the contracted dimension; Cs reuses their space
    // afterwards (2*CH*LDI + TI*LDJ >= CH*LDJ), which keeps the CTA under 48 KB of static smem.
    __shared__ __align__(16) float stage[2 * CH * LDI + TI * LDJ];
    __shared__ __align__(16) float Ws[CH * LDJ];
    __shared__ float zs[TI];
    static_assert(2 * CH * LDI + TI * LDJ >= CH * LDJ, "Cs must fit in the staging area");
    float* As = stage;
    float* Bs = stage + CH * LDI;
    float* St = stage + 2 * CH * LDI;
    float* Cs = stage;

    const int njt = (J + TJ - 1) / TJ;
    const int jt = blockIdx.x % njt;
    const int bc = blockIdx.x / njt;  // b * nc + c
    const int c = bc % g.nc, b = bc / g.nc;
    const int t0 = c * CH;
    const int nrows = min(CH, g.S - t0);
    const int64_t row0 = (int64_t)b * g.S + t0;
    const int j0 = jt * TJ;
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
    const bool map_a = g.map == CXXATTN_MAP_ELU1 && (MODE == FWD || MODE == DV);
    const bool map_b = map_a;
    const bool map_c = g.map == CXXATTN_MAP_ELU1 && (MODE == DQ || MODE == DK);
    const float* state = g.state + (int64_t)bc * g.D * g.E;
    const float* zstate = g.zstate + (int64_t)bc * g.D;

    float w[4][4], out[4][4], rowx[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        rowx[i] = 0.f;
#pragma unroll
        for (int j = 0; j < 4; j++) w[i][j] = out[i][j] = 0.f;
    }

    for (int i0 = 0; i0 < I; i0 += TI) {
        __syncthreads();
        load_slice<TI, LDI>(As, g.a, row0, nrows, ldI, i0, I, map_a);
        load_slice<TI, LDI>(Bs, g.b, row0, nrows, ldI, i0, I, map_b);
        for (int k = threadIdx.x; k < TI * TJ; k += NT) {
            const int ii = STATE_T ? k % TI : k / TJ, jj = STATE_T ? k / TI : k % TJ;  // coalesced either way
            float v = 0.f;
            if (i0 + ii < I && j0 + jj < J)
                v = STATE_T ? state[(int64_t)(j0 + jj) * I + (i0 + ii)]   // S[d=j][e=i]
                            : state[(int64_t)(i0 + ii) * J + (j0 + jj)];  // S[d=i][e=j]
            St[ii * LDJ + jj] = v;
        }
        if (MODE == FWD && threadIdx.x < TI) zs[threadIdx.x] = i0 + threadIdx.x < I ? zstate[i0 + threadIdx.x] : 0.f;
        __syncthreads();

        // scores: w[t][s] += a_t . b_s over this slice
#pragma unroll
        for (int d = 0; d < TI; d += 4) {
            float4 av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; i++) av[i] = *reinterpret_cast<const float4*>(As + (ty * 4 + i) * LDI + d);
#pragma unroll
            for (int j = 0; j < 4; j++) bv[j] = *reinterpret_cast<const float4*>(Bs + (tx + 16 * j) * LDI + d);
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    w[i][j] = fmaf(av[i].x, bv[j].x, w[i][j]);
                    w[i][j] = fmaf(av[i].y, bv[j].y, w[i][j]);
                    w[i][j] = fmaf(av[i].z, bv[j].z, w[i][j]);
                    w[i][j] = fmaf(av[i].w, bv[j].w, w[i][j]);
                }
        }
        // inter-chunk part: out[t][j] += a_t . State[:, j]
#pragma unroll 4
        for (int ii = 0; ii < TI; ii++) {
            float av[4], sv[4];
#pragma unroll
            for (int i = 0; i < 4; i++) av[i] = As[(ty * 4 + i) * LDI + ii];
#pragma unroll
            for (int j = 0; j < 4; j++) sv[j] = St[ii * LDJ + tx + 16 * j];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                if (MODE == FWD) rowx[i] = fmaf(av[i], zs[ii], rowx[i]);
#pragma unroll
                for (int j = 0; j < 4; j++) out[i][j] = fmaf(av[i], sv[j], out[i][j]);
            }
        }
        // z_cache: running sum of phi(K) down the chunk on top of the prefix z
        if (MODE == FWD && g.zc_out != nullptr && jt == 0 && threadIdx.x < TI && i0 + threadIdx.x < I) {
            float run = zs[threadIdx.x];
            for (int r = 0; r < nrows; r++) {
                run += Bs[r * LDI + threadIdx.x];
                g.zc_out[(row0 + r) * g.ldd + i0 + threadIdx.x] = run;
            }
        }
    }

    // causal mask inside the chunk, score biases, denominators
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int t = ty * 4 + i;
        float rs = 0.f;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int s = tx + 16 * j;
            const bool valid = (REV ? s >= t : s <= t) && s < nrows && t < nrows;
            float v = w[i][j];
            if (MODE == DQ && g.zcache == nullptr && valid) v += g.dden[row0 + t];
            if (MODE == DK && valid) v += g.dden[row0 + s];
            v = valid ? v : 0.f;
            Ws[t * LDJ + s] = v;
            rs += v;
        }
        if (MODE == FWD) {
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) rs += __shfl_xor_sync(0xffffffffu, rs, o);
            rowx[i] += rs;  // den_t = sum_s score + phi(q_t).z_prev
        }
    }
    __syncthreads();  // every reader of As/Bs/St is done before Cs overwrites them
    load_slice<TJ, LDJ>(Cs, g.c, row0, nrows, ldJ, j0, J, map_c);
    __syncthreads();

    // intra-chunk part: out[t][j] += sum_s w[t][s] c_s[j]
#pragma unroll 2
    for (int s = 0; s < CH; s += 4) {
        float4 wv[4];
#pragma unroll
        for (int i = 0; i < 4; i++) wv[i] = *reinterpret_cast<const float4*>(Ws + (ty * 4 + i) * LDJ + s);
#pragma unroll
        for (int ss = 0; ss < 4; ss++) {
            float cv[4];
#pragma unroll
            for (int j = 0; j < 4; j++) cv[j] = Cs[(s + ss) * LDJ + tx + 16 * j];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float x = ss == 0 ? wv[i].x : ss == 1 ? wv[i].y : ss == 2 ? wv[i].z : wv[i].w;
#pragma unroll
                for (int j = 0; j < 4; j++) out[i][j] = fmaf(x, cv[j], out[i][j]);
            }
        }
    }

#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int t = ty * 4 + i;
        if (t >= nrows) continue;
        const int64_t row = row0 + t;
        if (MODE == FWD && jt == 0 && tx == 0) g.den[row] = g.eps_in_den ? rowx[i] + 1e-8f : rowx[i];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int col = j0 + tx + 16 * j;
            if (col >= J) continue;
            float v = out[i][j];
            if (MODE == FWD) v = v / (rowx[i] + 1e-8f);
            if (MODE == DQ) v += g.zcache ? g.zcache[row * g.ldd + col] * g.dden[row] : g.dden[row] * zstate[col];
            if (MODE == DK) v += zstate[col];
            if ((MODE == DQ || MODE == DK) && g.X != nullptr) v *= phi_der(g.X[row * ldJ + col]);
            g.out[row * ldJ + col] = v;
        }
    }
}

// Local chunk states: S_c[d][e] = sum_{t in chunk} X_t[d] Y_t[e], z_c[d] = sum_t X_t[d] w_t (w = 1 if null).
// One CTA per (batch, chunk, 64 x 64 tile of the state).
__global__ void __launch_bounds__(NT) chunk_state_kernel(const float* __restrict__ X, const float* __restrict__ Y,
                                                         const float* __restrict__ wgt, float* __restrict__ state,
                                                         float* __restrict__ zstate, int S, int D, int E, int nc,
                                                         int ldx, bool map_x) {
    __shared__ __align__(16) float Xs[CH * LDJ];
    __shared__ __align__(16) float Ys[CH * LDJ];
    const int ndt = (D + TJ - 1) / TJ, net = (E + TJ - 1) / TJ;
    const int et = blockIdx.x % net;
    const int dt = (blockIdx.x / net) % ndt;
    const int bc = blockIdx.x / (net * ndt);
    const int c = bc % nc, b = bc / nc;
    const int t0 = c * CH;
    const int nrows = min(CH, S - t0);
    const int64_t row0 = (int64_t)b * S + t0;
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;

    load_slice<TJ, LDJ>(Xs, X, row0, nrows, ldx, dt * TJ, D, map_x);
    load_slice<TJ, LDJ>(Ys, Y, row0, nrows, E, et * TJ, E, false);
    __syncthreads();

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
#pragma unroll 4
    for (int t = 0; t < CH; t++) {
        const float4 xv = *reinterpret_cast<const float4*>(Xs + t * LDJ + ty * 4);
        float yv[4];
#pragma unroll
        for (int j = 0; j < 4; j++) yv[j] = Ys[t * LDJ + tx + 16 * j];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            acc[0][j] = fmaf(xv.x, yv[j], acc[0][j]);
            acc[1][j] = fmaf(xv.y, yv[j], acc[1][j]);
            acc[2][j] = fmaf(xv.z, yv[j], acc[2][j]);
            acc[3][j] = fmaf(xv.w, yv[j], acc[3][j]);
        }
    }
    float* st = state + (int64_t)bc * D * E;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int d = dt * TJ + ty * 4 + i;
        if (d >= D) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int e = et * TJ + tx + 16 * j;
            if (e < E) st[(int64_t)d * E + e] = acc[i][j];
        }
    }
    if (et == 0 && threadIdx.x < TJ && dt * TJ + threadIdx.x < D) {
        float z = 0.f;
        for (int t = 0; t < nrows; t++) z = fmaf(Xs[t * LDJ + threadIdx.x], wgt ? wgt[row0 + t] : 1.f, z);
        zstate[(int64_t)bc * D + dt * TJ + threadIdx.x] = z;
    }
}

// In-place exclusive prefix (rev = false) or suffix (rev = true) over the nc chunks of each batch
// item, for a buffer of `width` floats per chunk.  One thread per (batch, element); the chunk values are
// read sixteen at a time so that the loads are in flight together (one dependent load per chunk made
// this the slowest kernel of a step: 1.2 ms for 200 MB), and added in sequence order as before.
__global__ void chunk_scan_kernel(float* __restrict__ buf, int64_t width, int nc, int64_t total, bool rev) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int64_t b = i / width, k = i % width;
    float* p = buf + b * nc * width + k;
    float run = 0.f;
    constexpr int U = 16;
    for (int n0 = 0; n0 < nc; n0 += U) {
        float v[U];
#pragma unroll
        for (int j = 0; j < U; j++) {
            const int n = n0 + j, c = rev ? nc - 1 - n : n;
            v[j] = n < nc ? p[(int64_t)c * width] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < U; j++) {
            const int n = n0 + j, c = rev ? nc - 1 - n : n;
            if (n < nc) {
                p[(int64_t)c * width] = run;
                run += v[j];
            }
        }
    }
}

struct Ws {
    float* state;
    float* zstate;
    float* dnum;
    float* dden;
    int nc;
};

inline int chunks(const cxxattn_lin_desc& d) { return (int)((d.S + CH - 1) / CH); }

Ws carve(const cxxattn_lin_desc& d, void* ws) {
    Ws w;
    w.nc = chunks(d);
    char* p = static_cast<char*>(ws);
    w.state = reinterpret_cast<float*>(p);
    p += align_up((size_t)d.B * w.nc * d.D * d.E * sizeof(float), 256);
    w.zstate = reinterpret_cast<float*>(p);
    p += align_up((size_t)d.B * w.nc * d.D * sizeof(float), 256);
    w.dnum = reinterpret_cast<float*>(p);
    p += align_up((size_t)d.B * d.S * d.E * sizeof(float), 256);
    w.dden = reinterpret_cast<float*>(p);
    return w;
}

// Chunk states of (X, Y, weight) followed by their exclusive scan.
int build_states(const cxxattn_lin_desc& d, const Ws& w, const float* X, const float* Y,
                 const float* wgt, bool map_x, bool rev, cudaStream_t st) {
    const int ndt = (int)((d.D + TJ - 1) / TJ), net = (int)((d.E + TJ - 1) / TJ);
    const int64_t grid = (int64_t)d.B * w.nc * ndt * net;
    chunk_state_kernel<<<(unsigned)grid, NT, 0, st>>>(X, Y, wgt, w.state, w.zstate, (int)d.S, (int)d.D,
                                                      (int)d.E, w.nc, (int)(d.ld_qk ? d.ld_qk : d.D), map_x);
    if (check_launch() != CXXATTN_OK) return CXXATTN_ERR_CUDA;
    int64_t width = d.D * d.E, total = d.B * width;
    chunk_scan_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(w.state, width, w.nc, total, rev);
    width = d.D;
    total = d.B * width;
    chunk_scan_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(w.zstate, width, w.nc, total, rev);
    return check_launch();
}

template <int MODE>
int launch_apply(const cxxattn_lin_desc& d, ApplyArgs g, cudaStream_t st) {
    const int J = (MODE == FWD || MODE == DV) ? (int)d.E : (int)d.D;
    const int64_t grid = (int64_t)d.B * g.nc * ((J + TJ - 1) / TJ);
    chunk_apply_kernel<MODE><<<(unsigned)grid, NT, 0, st>>>(g);
    return check_launch();
}

ApplyArgs base_args(const cxxattn_lin_desc& d, const Ws& w) {
    ApplyArgs g = {};
    g.state = w.state;
    g.zstate = w.zstate;
    g.S = (int)d.S;
    g.D = (int)d.D;
    g.E = (int)d.E;
    g.nc = w.nc;
    g.ldd = (int)(d.ld_qk ? d.ld_qk : d.D);
    g.map = d.feature_map;
    g.eps_in_den = d.eps_in_den;
    return g;
}

}  // namespace

size_t linattn_f32_workspace(const cxxattn_lin_desc& d) {
    const size_t nc = (size_t)chunks(d);
    return align_up((size_t)d.B * nc * d.D * d.E * sizeof(float), 256) +
           align_up((size_t)d.B * nc * d.D * sizeof(float), 256) +
           align_up((size_t)d.B * d.S * d.E * sizeof(float), 256) +
           align_up((size_t)d.B * d.S * sizeof(float), 256);
}

int linattn_f32_fwd(const cxxattn_lin_desc& d, const float* Q, const float* K, const float* V,
                    float* O, float* den, float* z_cache, void* ws, size_t ws_bytes, cudaStream_t st) {
    if (ws == nullptr || ws_bytes < linattn_f32_workspace(d)) return CXXATTN_ERR_WORKSPACE;
    const Ws w = carve(d, ws);
    const bool map = d.feature_map == CXXATTN_MAP_ELU1;
    int rc = build_states(d, w, K, V, nullptr, map, false, st);
    if (rc != CXXATTN_OK) return rc;
    ApplyArgs g = base_args(d, w);
    g.a = Q; g.b = K; g.c = V; g.out = O; g.den = den; g.zc_out = z_cache;
    return launch_apply<FWD>(d, g, st);
}

// ---- forward with built-in scratch -----------------------------------------------------------
// Scratch for linattn_f32_fwd_static: chunk states and z states of one forward call.  It lives in
// the library's device image, so every GPU that loads the library holds these bytes until the
// process exits.
constexpr size_t kStaticScratchBytes = 8u << 20;  // 8 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Bytes of g_static_scratch a forward call with this descriptor uses (states, then z states).
static size_t static_fwd_bytes(const cxxattn_lin_desc& d) {
    const size_t nc = (size_t)chunks(d);
    return align_up((size_t)d.B * nc * d.D * d.E * sizeof(float), 256) +
           align_up((size_t)d.B * nc * d.D * sizeof(float), 256);
}

size_t linattn_f32_static_capacity() { return kStaticScratchBytes; }

// Same kernels and launch order as linattn_f32_fwd, with the scratch taken from g_static_scratch
// instead of a caller buffer.  In host code `g_static_scratch` is only a handle: its device
// address is looked up with cudaGetSymbolAddress, once per device, with that device current (the
// first call on a device does this look-up, so it should come before any stream capture).
// No allocation, no free, no allocating library call.
int linattn_f32_fwd_static(const cxxattn_lin_desc& d, const float* Q, const float* K, const float* V,
                           float* O, float* den, float* z_cache, cudaStream_t st) {
    if (static_fwd_bytes(d) > kStaticScratchBytes) return CXXATTN_ERR_TOO_LARGE;
    static std::atomic<void*> addr[kMaxDevices];  // filled with the same value by whichever thread comes first
    const int dev = current_device();
    if (dev < 0) return CXXATTN_ERR_CUDA;
    void* scratch = addr[dev].load(std::memory_order_relaxed);
    if (scratch == nullptr) {
        if (cudaGetSymbolAddress(&scratch, g_static_scratch) != cudaSuccess || scratch == nullptr) return CXXATTN_ERR_CUDA;
        addr[dev].store(scratch, std::memory_order_relaxed);
    }
    // carve() lays out states | z states | (dnum | dden); the forward touches the first two only,
    // and static_fwd_bytes() bounds exactly those.  Every chunk state is fully rewritten by
    // chunk_state_kernel before it is read, so stale contents of an earlier call do not matter.
    const Ws w = carve(d, scratch);
    const bool map = d.feature_map == CXXATTN_MAP_ELU1;
    int rc = build_states(d, w, K, V, nullptr, map, false, st);
    if (rc != CXXATTN_OK) return rc;
    ApplyArgs g = base_args(d, w);
    g.a = Q; g.b = K; g.c = V; g.out = O; g.den = den; g.zc_out = z_cache;
    return launch_apply<FWD>(d, g, st);
}

int linattn_f32_bwd_dq(const cxxattn_lin_desc& d, const float* K, const float* V, const float* dnum,
                       const float* dden, const float* z_cache, const float* Q, float* dQ,
                       void* ws, size_t ws_bytes, cudaStream_t st) {
    if (ws == nullptr || ws_bytes < linattn_f32_workspace(d)) return CXXATTN_ERR_WORKSPACE;
    const Ws w = carve(d, ws);
    const bool map = d.feature_map == CXXATTN_MAP_ELU1;
    if (map && Q == nullptr) return CXXATTN_ERR_INVALID;
    int rc = build_states(d, w, K, V, nullptr, map, false, st);
    if (rc != CXXATTN_OK) return rc;
    ApplyArgs g = base_args(d, w);
    g.a = dnum; g.b = V; g.c = K; g.dden = dden; g.zcache = z_cache; g.X = map ? Q : nullptr; g.out = dQ;
    return launch_apply<DQ>(d, g, st);
}

int linattn_f32_bwd_dkdv(const cxxattn_lin_desc& d, const float* Q, const float* K, const float* V,
                         const float* dnum, const float* dden, float* dK, float* dV,
                         void* ws, size_t ws_bytes, cudaStream_t st) {
    if (ws == nullptr || ws_bytes < linattn_f32_workspace(d)) return CXXATTN_ERR_WORKSPACE;
    const Ws w = carve(d, ws);
    const bool map = d.feature_map == CXXATTN_MAP_ELU1;
    int rc = build_states(d, w, Q, dnum, dden, map, true, st);
    if (rc != CXXATTN_OK) return rc;
    ApplyArgs g = base_args(d, w);
    g.a = K; g.b = Q; g.c = dnum; g.out = dV;
    rc = launch_apply<DV>(d, g, st);
    if (rc != CXXATTN_OK) return rc;
    g = base_args(d, w);
    g.a = V; g.b = dnum; g.c = Q; g.dden = dden; g.X = map ? K : nullptr; g.out = dK;
    return launch_apply<DK>(d, g, st);
}

int linattn_f32_bwd(const cxxattn_lin_desc& d, const float* Q, const float* K, const float* V,
                    const float* O, const float* dO, const float* den, float* dQ, float* dK, float* dV,
                    void* ws, size_t ws_bytes, cudaStream_t st) {
    if (ws == nullptr || ws_bytes < linattn_f32_workspace(d)) return CXXATTN_ERR_WORKSPACE;
    const Ws w = carve(d, ws);
    int rc = step1_f32(O, dO, den, w.dnum, w.dden, (size_t)(d.B * d.S), (size_t)d.E, st);
    if (rc != CXXATTN_OK) return rc;
    rc = linattn_f32_bwd_dq(d, K, V, w.dnum, w.dden, nullptr, Q, dQ, ws, ws_bytes, st);
    if (rc != CXXATTN_OK) return rc;
    return linattn_f32_bwd_dkdv(d, Q, K, V, w.dnum, w.dden, dK, dV, ws, ws_bytes, st);
}

}  // namespace cxxattn
