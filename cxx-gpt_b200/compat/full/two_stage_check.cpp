// CXX-GPT's TwoStageGPT (src/TwoStage/two_stage_gpt.hpp, included unmodified) on synthetic token
// ids, with its numerical gradient check (two_stage_gpt.hpp:547-604); see model_check.hpp.
//   two_stage_check [B] [S] [n_embd] [n_head] [N] [vocab] [steps] [learning rate]
#include <cstdlib>

#include "TwoStage/two_stage_gpt.hpp"
#include "model_check.hpp"

int main(int argc, char** argv) {
    auto arg = [&](int i, size_t d) { return argc > i ? (size_t)std::strtoul(argv[i], nullptr, 10) : d; };
    const size_t B = arg(1, 2), S = arg(2, 48);
    TwoStageConfig cfg;
    cfg.n_embd = arg(3, 64);
    cfg.n_head = arg(4, 2);
    cfg.N = arg(5, 1);
    cfg.vocab_size = arg(6, 96);
    cfg.block_size = S;
    try {
        RNG rng(1234);
        TwoStageGPT model(cfg, rng);
        return run_model_check(model, two_stage_numerical_grad_check, rng, B, S, cfg.vocab_size, arg(7, 8),
                               argc > 8 ? std::strtof(argv[8], nullptr) : 3e-3f);
    } catch (const std::exception& e) {
        std::fprintf(stderr, "error: %s\n", e.what());
        return 1;
    }
}
