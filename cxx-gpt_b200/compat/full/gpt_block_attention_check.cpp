// GPT::Block (src/GPT/gpt_gpt.hpp:365-380 forward, 420-438 backward) computes its single-head causal
// attention unfused: a [B*S, B*S] score matrix, gpt_cuda::attention_mask, a row softmax and two more
// products, with the transposes and the softmax backward to match.  This program runs that sequence
// (TensorN stand-in products + CXX-GPT's own gpt_cuda kernels) and two_stage_cuda::fused_mha_fwd /
// fused_mha_bwd with H = 1, Dh = n_embd on the same tensors, prints "<name> maxdiff = <x>" per tensor
// and the time of either route: the fused entry points can stand in for the block's attention.
//   gpt_block_attention_check [B] [S] [n_embd]
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "TensorN.hpp"
#include "TwoStage/two_stage_cuda_kernels.cuh"
#include "gpt_cuda_kernels.cuh"

using TensorN::CudaTensor;
using TensorN::Tensor;
namespace ops = TensorN::cuda;

static std::vector<float> seeded(size_t n, unsigned seed) {
    std::vector<float> v(n);
    unsigned long long s = 0x9E3779B97F4A7C15ull * (seed + 1);
    for (size_t i = 0; i < n; i++) {
        s = s * 6364136223846793005ull + 1442695040888963407ull;
        v[i] = (float)((s >> 40) & 0xFFFFFF) / 8388608.0f - 1.0f;
    }
    return v;
}

static float maxdiff(const CudaTensor<float>& a, const CudaTensor<float>& b) {
    Tensor<float> x = a.toTensor(), y = b.toTensor();
    float m = 0.f;
    for (size_t i = 0; i < x.size(); i++) {
        const float d = std::fabs(x[i] - y[i]);
        if (!(d <= m)) m = d;
    }
    return m;
}

struct Timer {
    cudaEvent_t a, b;
    Timer() { cudaEventCreate(&a), cudaEventCreate(&b), cudaEventRecord(a); }
    float ms() {
        cudaEventRecord(b), cudaEventSynchronize(b);
        float t = 0.f;
        cudaEventElapsedTime(&t, a, b);
        return t;
    }
};

int main(int argc, char** argv) {
    auto arg = [&](int i, size_t d) { return argc > i ? (size_t)std::strtoul(argv[i], nullptr, 10) : d; };
    const size_t B = arg(1, 8), S = arg(2, 64), E = arg(3, 128), dim = B * S;
    try {
        std::vector<CudaTensor<float>> in;
        for (unsigned i = 0; i < 4; i++) in.push_back(CudaTensor<float>::fromTensor(Tensor<float>({dim, E}, seeded(dim * E, i))));
        const CudaTensor<float>&Q = in[0], &K = in[1], &V = in[2], &dOut = in[3];
        const float scale = 1.0f / std::sqrt((float)E);

        CudaTensor<float> O1({dim, E}), dQ1({dim, E}), dK1({dim, E}), dV1({dim, E});
        float t_unfused = 0.f;
        for (int rep = 0; rep < 2; rep++) {  // second pass is the timed one
            Timer tm;
            CudaTensor<float> Kt({E, dim}), scores({dim, dim}), w({dim, dim});
            ops::transpose(K, Kt);
            ops::matmul(Q, Kt, scores);
            ops::multiply_scalar(scores, scale, scores);
            gpt_cuda::attention_mask(scores, B, S);
            ops::softmax(scores, w, -1);
            ops::matmul(w, V, O1);
            CudaTensor<float> dw({dim, dim}), Vt({E, dim}), ds({dim, dim}), dsT({dim, dim}), wT({dim, dim});
            ops::transpose(V, Vt);
            ops::matmul(dOut, Vt, dw);
            gpt_cuda::softmax_backward(w, dw, ds);
            ops::multiply_scalar(ds, scale, ds);
            ops::matmul(ds, K, dQ1);
            ops::transpose(ds, dsT);
            ops::matmul(dsT, Q, dK1);
            ops::transpose(w, wT);
            ops::matmul(wT, dOut, dV1);
            t_unfused = tm.ms();
        }

        CudaTensor<float> O2({dim, E}), dQ2({dim, E}), dK2({dim, E}), dV2({dim, E});
        float t_fused = 0.f;
        for (int rep = 0; rep < 2; rep++) {
            Timer tm;
            two_stage_cuda::fused_mha_fwd(Q, K, V, O2, B, S, 1, E);
            two_stage_cuda::fused_mha_bwd(Q, K, V, O2, dOut, dQ2, dK2, dV2, B, S, 1, E);
            t_fused = tm.ms();
        }
        std::printf("gpt block O maxdiff = %g\n", maxdiff(O1, O2));
        std::printf("gpt block dQ maxdiff = %g\n", maxdiff(dQ1, dQ2));
        std::printf("gpt block dK maxdiff = %g\n", maxdiff(dK1, dK2));
        std::printf("gpt block dV maxdiff = %g\n", maxdiff(dV1, dV2));
        std::printf("time unfused_ms = %g\n", t_unfused);
        std::printf("time fused_ms = %g\n", t_fused);
        std::printf("done\n");
    } catch (const std::exception& e) {
        std::fprintf(stderr, "error: %s\n", e.what());
        return 1;
    }
    return 0;
}
