// CPU oracle for the attention hot path.  TEST INFRASTRUCTURE ONLY.
//
// This file restates, on the CPU, the arithmetic of the reference kernels so that the
// CUDA kernels of this library can be checked against it.  Nothing in the product path
// may call it: only the tests, the smoke check and the cpu_baseline / reference arm of the
// benchmark load the shared object built from this file.
//
// Parity status
//   * softmax MHA and ELU+1 kernel attention: restated from the reference's own CPU test
//     code (src/TwoStage/kernel_test.cpp:16-193) and pinned against that code compiled
//     unmodified (oracle/ref_wrap.cpp -> oracle/_ref/) on the kernel_test shapes:
//     bit-identical results.
//   * LinearGPT scan (src/LinearAttention/linear_cuda_kernels.cu) has no CPU code and no
//     kernel-level test in the reference: restated from the CUDA source, "parity unpinned"
//     except through the identity linear(phi(Q),phi(K),V) == kernel_attn(Q,K,V).
//   * RoPE restated from kernel_test.cpp:451-471, GELU from two_stage_cuda_kernels.cu:1883-1915.
//
// Every function has a float instantiation that follows the reference operation order and a
// double instantiation (inputs still float) used to adjudicate rounding differences.
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <random>
#include <vector>
#include <algorithm>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

// kernel_test.cpp:16-17
template <typename T> inline T phi_elu(T x) { return x > T(0) ? x + T(1) : std::exp(x); }
template <typename T> inline T phi_elu_der(T x) { return x > T(0) ? T(1) : std::exp(x); }

// Element offset of (b, s, h, c) in a (B*S, H*Dh) row-major tensor: kernel_test.cpp:19-22.
inline size_t at(size_t b, size_t s, size_t h, size_t c, size_t S, size_t H, size_t Dh) {
    return ((b * S + s) * H + h) * Dh + c;
}

// Softmax MHA forward, kernel_test.cpp:24-46.  The reference recomputes the score row for each
// output column c; the scores do not depend on c, so one row pass gives the same bits.
template <typename T>
void mha_fwd(const float* Q, const float* K, const float* V, float* O, float* lse,
             size_t B, size_t S, size_t H, size_t Dh) {
    const T scale = T(1) / std::sqrt(T(Dh));
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (size_t b = 0; b < B; b++)
        for (size_t h = 0; h < H; h++) {
            std::vector<T> sc(S), out(Dh);
            for (size_t s = 0; s < S; s++) {
                T m = T(-1e30f);
                for (size_t t = 0; t <= s; t++) {
                    T acc = 0;
                    for (size_t d = 0; d < Dh; d++)
                        acc += T(Q[at(b, s, h, d, S, H, Dh)]) * T(K[at(b, t, h, d, S, H, Dh)]);
                    sc[t] = acc * scale;
                    m = std::max(m, sc[t]);
                }
                T l = 0;
                for (size_t t = 0; t <= s; t++) l += std::exp(sc[t] - m);
                std::fill(out.begin(), out.end(), T(0));
                for (size_t t = 0; t <= s; t++) {
                    T p = std::exp(sc[t] - m) / l;
                    for (size_t c = 0; c < Dh; c++) out[c] += p * T(V[at(b, t, h, c, S, H, Dh)]);
                }
                for (size_t c = 0; c < Dh; c++) O[at(b, s, h, c, S, H, Dh)] = float(out[c]);
                if (lse) lse[(b * H + h) * S + s] = float(m + std::log(l));
            }
        }
}

// Softmax MHA backward, kernel_test.cpp:48-94.  For a fixed (b, h) the reference visits s
// ascending and, inside, t ascending; each (b, h) owns its slice of dQ/dK/dV, so running the
// (b, h) pairs in parallel keeps every accumulation in the reference's order.
template <typename T>
void mha_bwd(const float* Q, const float* K, const float* V, const float* O, const float* dO,
             float* dQ, float* dK, float* dV, size_t B, size_t S, size_t H, size_t Dh) {
    const T scale = T(1) / std::sqrt(T(Dh));
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (size_t b = 0; b < B; b++)
        for (size_t h = 0; h < H; h++) {
            std::vector<T> p(S), aq(S * Dh, T(0)), ak(S * Dh, T(0)), av(S * Dh, T(0));
            for (size_t s = 0; s < S; s++) {
                T m = T(-1e30f);
                for (size_t t = 0; t <= s; t++) {
                    T acc = 0;
                    for (size_t d = 0; d < Dh; d++)
                        acc += T(Q[at(b, s, h, d, S, H, Dh)]) * T(K[at(b, t, h, d, S, H, Dh)]);
                    p[t] = acc * scale;
                    m = std::max(m, p[t]);
                }
                T l = 0;
                for (size_t t = 0; t <= s; t++) { p[t] = std::exp(p[t] - m); l += p[t]; }
                T gs = 0;
                for (size_t c = 0; c < Dh; c++)
                    gs += T(dO[at(b, s, h, c, S, H, Dh)]) * T(O[at(b, s, h, c, S, H, Dh)]);
                for (size_t t = 0; t <= s; t++) {
                    T pv = p[t] / l;
                    T ds = 0;
                    for (size_t c = 0; c < Dh; c++)
                        ds += T(dO[at(b, s, h, c, S, H, Dh)]) * T(V[at(b, t, h, c, S, H, Dh)]);
                    T dscore = pv * (ds - gs);
                    for (size_t c = 0; c < Dh; c++) {
                        aq[s * Dh + c] += scale * dscore * T(K[at(b, t, h, c, S, H, Dh)]);
                        ak[t * Dh + c] += scale * dscore * T(Q[at(b, s, h, c, S, H, Dh)]);
                        av[t * Dh + c] += pv * T(dO[at(b, s, h, c, S, H, Dh)]);
                    }
                }
            }
            for (size_t s = 0; s < S; s++)
                for (size_t c = 0; c < Dh; c++) {
                    dQ[at(b, s, h, c, S, H, Dh)] = float(aq[s * Dh + c]);
                    dK[at(b, s, h, c, S, H, Dh)] = float(ak[s * Dh + c]);
                    dV[at(b, s, h, c, S, H, Dh)] = float(av[s * Dh + c]);
                }
        }
}

// Causal linear attention forward, both flavours.
//   elu = true : two_stage kernel attention, kernel_test.cpp:96-126 (phi fused, state[e*D+d],
//                den stored without eps, O = num / (den + 1e-8)).
//   elu = false: LinearGPT scan, linear_cuda_kernels.cu:10-79 (inputs already mapped,
//                den_cache = q.z + 1e-8 stored, O = num / den_cache).
// z_cache (optional) receives the running z_t, as both reference kernels write it.
template <typename T>
void lin_fwd(const float* Q, const float* K, const float* V, float* O, float* den, float* z_cache,
             size_t B, size_t S, size_t D, size_t E, bool elu) {
#pragma omp parallel for schedule(dynamic, 1)
    for (size_t b = 0; b < B; b++) {
        std::vector<T> z(D, T(0)), state(E * D, T(0)), kp(D), qp(D);
        for (size_t t = 0; t < S; t++) {
            size_t idx = b * S + t;
            for (size_t d = 0; d < D; d++) {
                kp[d] = elu ? phi_elu(T(K[idx * D + d])) : T(K[idx * D + d]);
                qp[d] = elu ? phi_elu(T(Q[idx * D + d])) : T(Q[idx * D + d]);
            }
            for (size_t d = 0; d < D; d++) {
                z[d] += kp[d];
                for (size_t e = 0; e < E; e++) state[e * D + d] += kp[d] * T(V[idx * E + e]);
            }
            if (z_cache)
                for (size_t d = 0; d < D; d++) z_cache[idx * D + d] = float(z[d]);
            T dpart = 0;
            for (size_t d = 0; d < D; d++) dpart += qp[d] * z[d];
            T denom = dpart + T(1e-8f);
            den[idx] = elu ? float(dpart) : float(denom);
            for (size_t e = 0; e < E; e++) {
                T num = 0;
                for (size_t d = 0; d < D; d++) num += qp[d] * state[e * D + d];
                O[idx * E + e] = float(num / denom);
            }
        }
    }
}

// Step 1 of the linear backward: two_stage_cuda_kernels.cu:1190-1219 and
// linear_cuda_kernels.cu:101-134 (same arithmetic; which den is passed decides the flavour).
template <typename T>
void lin_step1(const float* O, const float* dO, const float* den, float* dnum, float* dden,
               size_t N, size_t E) {
#pragma omp parallel for
    for (size_t i = 0; i < N; i++) {
        T inv = T(1) / T(den[i]);
        T sum = 0;
        for (size_t e = 0; e < E; e++) {
            dnum[i * E + e] = float(T(dO[i * E + e]) * inv);
            sum += T(dO[i * E + e]) * T(O[i * E + e]);
        }
        dden[i] = float(-sum * inv);
    }
}

// Linear attention backward from (dnum, dden).  elu = true follows kernel_test.cpp:128-193
// (outputs carry phi'), elu = false follows linear_cuda_kernels.cu:152-197,217-273 (gradients
// with respect to the mapped features).  The reference test rebuilds the prefix state from
// s = 0..t and the suffix state from s = S-1..t for every t; a running forward scan and a
// running reverse scan add the same terms in the same order, so the bits are the same at
// O(S*D*E) cost.
template <typename T>
void lin_bwd(const float* Q, const float* K, const float* V, const float* dnum, const float* dden,
             float* dQ, float* dK, float* dV, size_t B, size_t S, size_t D, size_t E, bool elu) {
#pragma omp parallel for schedule(dynamic, 1)
    for (size_t b = 0; b < B; b++) {
        std::vector<T> z(D, T(0)), state(E * D, T(0));
        for (size_t t = 0; t < S; t++) {
            size_t idx = b * S + t;
            for (size_t d = 0; d < D; d++) {
                T kp = elu ? phi_elu(T(K[idx * D + d])) : T(K[idx * D + d]);
                z[d] += kp;
                for (size_t e = 0; e < E; e++) state[e * D + d] += kp * T(V[idx * E + e]);
            }
            for (size_t d = 0; d < D; d++) {
                T acc = z[d] * T(dden[idx]);
                for (size_t e = 0; e < E; e++) acc += state[e * D + d] * T(dnum[idx * E + e]);
                dQ[idx * D + d] = float(elu ? acc * phi_elu_der(T(Q[idx * D + d])) : acc);
            }
        }
        std::vector<T> zs(D, T(0)), ss(E * D, T(0));
        for (size_t t = S; t-- > 0;) {
            size_t idx = b * S + t;
            for (size_t d = 0; d < D; d++) {
                T qp = elu ? phi_elu(T(Q[idx * D + d])) : T(Q[idx * D + d]);
                zs[d] += qp * T(dden[idx]);
                for (size_t e = 0; e < E; e++) ss[e * D + d] += qp * T(dnum[idx * E + e]);
            }
            for (size_t e = 0; e < E; e++) {
                T acc = 0;
                for (size_t d = 0; d < D; d++) {
                    T kp = elu ? phi_elu(T(K[idx * D + d])) : T(K[idx * D + d]);
                    acc += ss[e * D + d] * kp;
                }
                dV[idx * E + e] = float(acc);
            }
            for (size_t d = 0; d < D; d++) {
                T acc = zs[d];
                for (size_t e = 0; e < E; e++) acc += ss[e * D + d] * T(V[idx * E + e]);
                dK[idx * D + d] = float(elu ? acc * phi_elu_der(T(K[idx * D + d])) : acc);
            }
        }
    }
}

// ELU+1 kernel attention backward straight from (O, dO, den), with the exact expression forms
// of kernel_test.cpp:128-193: the prefix half multiplies by inv_den = 1/den, the suffix half
// divides by den, and dden is accumulated term by term.  Running scans replace the per-t
// recomputation (same terms, same order, same bits).
template <typename T>
void kattn_bwd_ref(const float* Q, const float* K, const float* V, const float* O, const float* dO,
                   const float* den, float* dQ, float* dK, float* dV,
                   size_t B, size_t S, size_t D, size_t E) {
#pragma omp parallel for schedule(dynamic, 1)
    for (size_t b = 0; b < B; b++) {
        std::vector<T> z(D, T(0)), state(E * D, T(0));
        for (size_t t = 0; t < S; t++) {
            size_t idx = b * S + t;
            for (size_t d = 0; d < D; d++) {
                z[d] += phi_elu(T(K[idx * D + d]));
                for (size_t e = 0; e < E; e++)
                    state[e * D + d] += phi_elu(T(K[idx * D + d])) * T(V[idx * E + e]);
            }
            T inv_den = T(1) / T(den[idx]);
            T dden = 0;
            for (size_t e = 0; e < E; e++) dden -= T(dO[idx * E + e]) * T(O[idx * E + e]) * inv_den;
            for (size_t d = 0; d < D; d++) {
                T dnum = z[d] * dden;
                for (size_t e = 0; e < E; e++) dnum += state[e * D + d] * (T(dO[idx * E + e]) * inv_den);
                dQ[idx * D + d] = float(dnum * phi_elu_der(T(Q[idx * D + d])));
            }
        }
        std::vector<T> zs(D, T(0)), ss(E * D, T(0));
        for (size_t t = S; t-- > 0;) {
            size_t j = b * S + t;
            T dd = 0;
            for (size_t e = 0; e < E; e++) dd -= T(dO[j * E + e]) * T(O[j * E + e]) / T(den[j]);
            for (size_t d = 0; d < D; d++) {
                zs[d] += phi_elu(T(Q[j * D + d])) * dd;
                for (size_t e = 0; e < E; e++)
                    ss[e * D + d] += phi_elu(T(Q[j * D + d])) * (T(dO[j * E + e]) / T(den[j]));
            }
            for (size_t e = 0; e < E; e++) {
                T acc = 0;
                for (size_t d = 0; d < D; d++) acc += ss[e * D + d] * phi_elu(T(K[j * D + d]));
                dV[j * E + e] = float(acc);
            }
            for (size_t d = 0; d < D; d++) {
                T acc = zs[d];
                for (size_t e = 0; e < E; e++) acc += ss[e * D + d] * T(V[j * E + e]);
                dK[j * D + d] = float(acc * phi_elu_der(T(K[j * D + d])));
            }
        }
    }
}

}  // namespace

extern "C" {

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void oracle_set_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n < 1 ? 1 : n);
#else
    (void)n;
#endif
}

// kernel_test.cpp:12-14: std::mt19937(1234), uniform in [-1, 1]; `skip` draws are discarded
// first so that a test can reproduce the inputs of any block of the reference test.
void oracle_frand(float* out, size_t n, size_t skip) {
    std::mt19937 g(1234);
    g.discard(skip);
    for (size_t i = 0; i < n; i++) out[i] = (float)g() / (float)g.max() * 2.0f - 1.0f;
}

void oracle_mha_fwd(const float* Q, const float* K, const float* V, float* O, float* lse,
                    size_t B, size_t S, size_t H, size_t Dh, int f64) {
    if (f64) mha_fwd<double>(Q, K, V, O, lse, B, S, H, Dh);
    else mha_fwd<float>(Q, K, V, O, lse, B, S, H, Dh);
}

void oracle_mha_bwd(const float* Q, const float* K, const float* V, const float* O,
                    const float* dO, float* dQ, float* dK, float* dV,
                    size_t B, size_t S, size_t H, size_t Dh, int f64) {
    if (f64) mha_bwd<double>(Q, K, V, O, dO, dQ, dK, dV, B, S, H, Dh);
    else mha_bwd<float>(Q, K, V, O, dO, dQ, dK, dV, B, S, H, Dh);
}

void oracle_linattn_fwd(const float* Q, const float* K, const float* V, float* O, float* den,
                        float* z_cache, size_t B, size_t S, size_t D, size_t E, int elu, int f64) {
    if (f64) lin_fwd<double>(Q, K, V, O, den, z_cache, B, S, D, E, elu != 0);
    else lin_fwd<float>(Q, K, V, O, den, z_cache, B, S, D, E, elu != 0);
}

void oracle_linattn_step1(const float* O, const float* dO, const float* den, float* dnum,
                          float* dden, size_t N, size_t E, int f64) {
    if (f64) lin_step1<double>(O, dO, den, dnum, dden, N, E);
    else lin_step1<float>(O, dO, den, dnum, dden, N, E);
}

void oracle_linattn_bwd(const float* Q, const float* K, const float* V, const float* dnum,
                        const float* dden, float* dQ, float* dK, float* dV,
                        size_t B, size_t S, size_t D, size_t E, int elu, int f64) {
    if (f64) lin_bwd<double>(Q, K, V, dnum, dden, dQ, dK, dV, B, S, D, E, elu != 0);
    else lin_bwd<float>(Q, K, V, dnum, dden, dQ, dK, dV, B, S, D, E, elu != 0);
}

void oracle_kernel_attn_bwd(const float* Q, const float* K, const float* V, const float* O,
                            const float* dO, const float* den, float* dQ, float* dK, float* dV,
                            size_t B, size_t S, size_t D, size_t E, int f64) {
    if (f64) kattn_bwd_ref<double>(Q, K, V, O, dO, den, dQ, dK, dV, B, S, D, E);
    else kattn_bwd_ref<float>(Q, K, V, O, dO, den, dQ, dK, dV, B, S, D, E);
}

// linear_cuda_kernels.cu:305-325: phi[n, d] = ELU(x[n, d]) + 1 for d < E, 0 for E <= d < D.
void oracle_phi_elu_fwd(const float* x, float* phi, size_t N, size_t D, size_t E) {
    for (size_t i = 0; i < N; i++)
        for (size_t j = 0; j < D; j++) {
            if (j < E) {
                float xv = x[i * E + j];
                float elu = xv > 0.0f ? xv : std::exp(xv) - 1.0f;
                phi[i * D + j] = elu + 1.0f;
            } else {
                phi[i * D + j] = 0.0f;
            }
        }
}

// linear_cuda_kernels.cu:347-364.
void oracle_phi_elu_bwd(const float* dphi, const float* x, float* dx, size_t N, size_t D, size_t E) {
    for (size_t i = 0; i < N; i++)
        for (size_t j = 0; j < E; j++) {
            float xv = x[i * E + j];
            dx[i * E + j] = dphi[i * D + j] * (xv > 0.0f ? 1.0f : std::exp(xv));
        }
}

// kernel_test.cpp:451-471: rotate pairs (2i, 2i+1) of each head by sign * (row % S) * base^(-2i/hd).
void oracle_rope(float* X, size_t rows, size_t S, size_t D, size_t head_dim, float sign) {
    const float base = 10000.0f;
    for (size_t r = 0; r < rows; r++) {
        size_t p = r % S;
        for (size_t h = 0; h < D / head_dim; h++)
            for (size_t i = 0; i < head_dim / 2; i++) {
                float w = std::pow(base, -2.0f * (float)i / (float)head_dim);
                float ang = sign * p * w;
                float c = std::cos(ang), s = std::sin(ang);
                float& x0 = X[r * D + h * head_dim + 2 * i];
                float& x1 = X[r * D + h * head_dim + 2 * i + 1];
                float a = x0, bb = x1;
                x0 = a * c - bb * s;
                x1 = a * s + bb * c;
            }
    }
}

// two_stage_cuda_kernels.cu:1883-1915 (erf GELU and its derivative).
void oracle_gelu_exact(const float* A, float* C, size_t n, int deriv) {
    for (size_t i = 0; i < n; i++) {
        float x = A[i];
        float a = x * 0.7071067811865476f;
        C[i] = deriv ? 0.5f * (1.0f + std::erf(a)) + x * std::exp(-0.5f * x * x) * 0.3989422804014327f
                     : 0.5f * x * (1.0f + std::erf(a));
    }
}

}  // extern "C"
