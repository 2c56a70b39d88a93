// Builds the reference's own CPU test functions into a shared object.  TEST INFRASTRUCTURE ONLY.
//
// The translation unit textually includes src/TwoStage/kernel_test.cpp from the reference tree
// (found through -I <reference>/src; nothing is copied into this repository), with main()
// renamed, and exports thin extern "C" callers around its static functions ref_mha_fwd,
// ref_mha_bwd, ref_kernel_attn_fwd, ref_kernel_attn_bwd and frand.  The result,
// oracle/_ref/libref_kernel_test.so, is what oracle.cpp is pinned against.
#define main cxxgpt_reference_kernel_test_main
#include "TwoStage/kernel_test.cpp"
#undef main

// Never called (the renamed main is never run); present so the object links.
namespace two_stage_cuda {
void fused_mha_fwd(In, In, In, Out, size_t, size_t, size_t, size_t) {}
void fused_mha_bwd(In, In, In, In, In, Out, Out, Out, size_t, size_t, size_t, size_t) {}
void kernel_attn_fwd(In, In, In, Out, Out, Out, Out, Out, size_t, size_t, size_t, size_t) {}
void kernel_attn_bwd_step1(In, In, In, Out, Out, size_t, size_t) {}
void kernel_attn_bwd_dQ(In, In, In, In, In, In, Out, Out, size_t, size_t, size_t, size_t) {}
void kernel_attn_bwd_dKdV(In, In, In, In, In, Out, Out, size_t, size_t, size_t, size_t) {}
void rope_fwd(Out, Out, size_t, size_t, size_t, size_t) {}
void rope_bwd(Out, Out, size_t, size_t, size_t, size_t) {}
}  // namespace two_stage_cuda

extern "C" {

// Re-seeds the file's generator (std::mt19937(1234)), skips `skip` draws, then fills n values.
void ref_frand(float* out, size_t n, size_t skip) {
    rgen.seed(1234);
    rgen.discard(skip);
    for (size_t i = 0; i < n; i++) out[i] = frand();
}

void ref_mha_fwd_all(const float* Q, const float* K, const float* V, float* O,
                     size_t B, size_t S, size_t H, size_t Dh) {
    size_t n = B * S * H * Dh;
    std::vector<float> q(Q, Q + n), k(K, K + n), v(V, V + n);
    for (size_t b = 0; b < B; b++)
        for (size_t s = 0; s < S; s++)
            for (size_t h = 0; h < H; h++)
                for (size_t c = 0; c < Dh; c++)
                    O[idx3(b, s, h, c, S, H, Dh)] = ref_mha_fwd(q, k, v, b, s, h, c, B, S, H, Dh);
}

void ref_mha_bwd_all(const float* Q, const float* K, const float* V, const float* O, const float* dO,
                     float* dQ, float* dK, float* dV, size_t B, size_t S, size_t H, size_t Dh) {
    size_t n = B * S * H * Dh;
    std::vector<float> q(Q, Q + n), k(K, K + n), v(V, V + n), o(O, O + n), g(dO, dO + n);
    std::vector<float> rq(n, 0.0f), rk(n, 0.0f), rv(n, 0.0f);
    ref_mha_bwd(q, k, v, o, g, rq, rk, rv, B, S, H, Dh);
    std::copy(rq.begin(), rq.end(), dQ);
    std::copy(rk.begin(), rk.end(), dK);
    std::copy(rv.begin(), rv.end(), dV);
}

void ref_kernel_attn_fwd_all(const float* Q, const float* K, const float* V, float* O, float* den,
                             size_t B, size_t S, size_t D, size_t E) {
    size_t n = B * S;
    std::vector<float> q(Q, Q + n * D), k(K, K + n * D), v(V, V + n * E), o(n * E), dn(n);
    ref_kernel_attn_fwd(q, k, v, o, dn, B, S, D, E);
    std::copy(o.begin(), o.end(), O);
    std::copy(dn.begin(), dn.end(), den);
}

void ref_kernel_attn_bwd_all(const float* Q, const float* K, const float* V, const float* O,
                             const float* dO, const float* den, float* dQ, float* dK, float* dV,
                             size_t B, size_t S, size_t D, size_t E) {
    size_t n = B * S;
    std::vector<float> q(Q, Q + n * D), k(K, K + n * D), v(V, V + n * E), o(O, O + n * E),
        g(dO, dO + n * E), dn(den, den + n), rq(n * D), rk(n * D), rv(n * E);
    ref_kernel_attn_bwd(q, k, v, o, g, dn, rq, rk, rv, B, S, D, E);
    std::copy(rq.begin(), rq.end(), dQ);
    std::copy(rk.begin(), rk.end(), dK);
    std::copy(rv.begin(), rv.end(), dV);
}

}  // extern "C"
