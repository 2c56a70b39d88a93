// Shared body of two_stage_check.cpp and linear_gpt_check.cpp: runs one of CXX-GPT's models (its
// header included unmodified by the caller) on synthetic token ids and prints
//   * the model's own numerical gradient check,
//   * a digest of one forward + backward: loss, logit checksums, gradient norm per parameter,
//   * the loss of a few AdamW steps (gpt_gpt.hpp:254-286).
// The same program linked against CXX-GPT's attention kernels and against this library's adapter
// must print the same numbers: the attention kernels are the only difference between the two.
#pragma once
#include <cmath>
#include <cstdio>
#include <vector>

template <class Model, class GradCheck>
int run_model_check(Model& model, GradCheck grad_check, RNG& rng, size_t B, size_t S, size_t vocab, size_t steps,
                    float lr) {
    std::vector<int> x(B * S), y(B * S);
    for (size_t i = 0; i < B * S; i++) {
        x[i] = rng.randint(0, (int)vocab - 1);
        y[i] = (x[i] * 7 + 3) % (int)vocab;  // a learnable map
    }
    grad_check(model, x, y, B, S);

    auto logits = model.forward(x, B, S);
    auto [loss, dlogits] = cross_entropy_loss(logits, y);
    model.zero_grad();
    model.backward(dlogits);
    auto lg = logits.toTensor();
    double sum = 0, sumabs = 0;
    for (size_t i = 0; i < lg.size(); i++) sum += lg[i], sumabs += std::fabs(lg[i]);
    std::printf("digest loss = %.7f\n", loss);
    std::printf("digest logits_sum = %.6f\n", sum);
    std::printf("digest logits_abs = %.6f\n", sumabs);
    for (auto& [name, p] : model.named_parameters())
        std::printf("digest gradnorm %s = %.7g\n", name.c_str(), std::sqrt(gpt_cuda::grad_norm_squared(p->grad)));

    AdamW opt(model.parameters(), lr);
    for (size_t s = 0; s < steps; s++) {
        auto lgs = model.forward(x, B, S);
        auto [l, dl] = cross_entropy_loss(lgs, y);
        model.zero_grad();
        model.backward(dl);
        opt.step();
        std::printf("train step %zu loss = %.6f\n", s, l);
    }
    std::printf("done\n");
    return 0;
}
