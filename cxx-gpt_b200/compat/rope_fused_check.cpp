// Checks the adapter's rope_fused_mha_fwd / rope_fused_mha_bwd against the sequence of calls they
// stand for in TwoStageGPT's stage 1 (two_stage_gpt.hpp:102-106 and 171-174):
//   rope_fwd(Q, K); fused_mha_fwd(Q, K, V, O);  fused_mha_bwd(...); rope_bwd(dQ, dK)
// on seeded inputs, in whichever precision mode the adapter is switched to.  Prints one
// "<name> maxdiff = <x>" line per tensor in the style of the reference's kernel unit test, plus a
// line that says whether the un-rotated inputs were left untouched.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "cxxgpt_kernels.hpp"

using TensorN::CudaTensor;
using TensorN::Tensor;

static std::vector<float> seeded(size_t n, unsigned seed) {
    std::vector<float> v(n);
    unsigned long long s = 0x9E3779B97F4A7C15ull * (seed + 1);
    for (size_t i = 0; i < n; i++) {
        s = s * 6364136223846793005ull + 1442695040888963407ull;
        v[i] = (float)((s >> 40) & 0xFFFFFF) / 8388608.0f - 1.0f;  // uniform in [-1, 1)
    }
    return v;
}

static float maxdiff(const CudaTensor<float>& a, const CudaTensor<float>& b) {
    Tensor<float> x = a.toTensor(), y = b.toTensor();
    float m = 0.f;
    for (size_t i = 0; i < x.size(); i++) {
        const float d = std::fabs((*x.data)[i] - (*y.data)[i]);
        if (!(d <= m)) m = d;  // keeps a NaN
    }
    return m;
}

int main(int argc, char** argv) {
    const size_t B = argc > 1 ? std::strtoul(argv[1], nullptr, 10) : 2;
    const size_t S = argc > 2 ? std::strtoul(argv[2], nullptr, 10) : 300;
    const size_t H = argc > 3 ? std::strtoul(argv[3], nullptr, 10) : 3;
    const size_t Dh = argc > 4 ? std::strtoul(argv[4], nullptr, 10) : 64;
    const size_t dim = B * S, big = H * Dh, n = dim * big;
    std::vector<CudaTensor<float>> in;
    for (unsigned i = 0; i < 4; i++) in.push_back(CudaTensor<float>::fromTensor(Tensor<float>({dim, big}, seeded(n, i))));
    const CudaTensor<float>&Q = in[0], &K = in[1], &V = in[2], &dO = in[3];

    // the reference's sequence, on copies that the rotation overwrites
    CudaTensor<float> Qr(Q), Kr(K), O1({dim, big}), dQ1({dim, big}), dK1({dim, big}), dV1({dim, big});
    two_stage_cuda::rope_fwd(Qr, Kr, B, S, big, Dh);
    two_stage_cuda::fused_mha_fwd(Qr, Kr, V, O1, B, S, H, Dh);
    two_stage_cuda::fused_mha_bwd(Qr, Kr, V, O1, dO, dQ1, dK1, dV1, B, S, H, Dh);
    two_stage_cuda::rope_bwd(dQ1, dK1, B, S, big, Dh);

    // the folded pair, on the un-rotated projections
    CudaTensor<float> Q0(Q), K0(K), O2({dim, big}), dQ2({dim, big}), dK2({dim, big}), dV2({dim, big});
    cxxattn_compat::rope_fused_mha_fwd(Q0, K0, V, O2, B, S, H, Dh);
    cxxattn_compat::rope_fused_mha_bwd(Q0, K0, V, O2, dO, dQ2, dK2, dV2, B, S, H, Dh);

    std::printf("rope+mha O maxdiff = %g\n", maxdiff(O1, O2));
    std::printf("rope+mha dQ maxdiff = %g\n", maxdiff(dQ1, dQ2));
    std::printf("rope+mha dK maxdiff = %g\n", maxdiff(dK1, dK2));
    std::printf("rope+mha dV maxdiff = %g\n", maxdiff(dV1, dV2));
    std::printf("inputs untouched maxdiff = %g\n", std::fmax(maxdiff(Q, Q0), maxdiff(K, K0)));
    std::printf("rotation applied maxdiff = %g\n", maxdiff(Q, Qr));  // non-zero: the check is not vacuous
    std::printf("done\n");
    return 0;
}
