// CXX-GPT's LinearGPT (src/LinearAttention/linear_gpt.hpp, included unmodified) on synthetic token
// ids, with its numerical gradient check (linear_gpt.hpp:554-610); see model_check.hpp.
//   linear_gpt_check [B] [S] [n_embd] [n_layer] [vocab] [steps] [learning rate]
#include <cstdlib>

#include "LinearAttention/linear_gpt.hpp"
#include "model_check.hpp"

int main(int argc, char** argv) {
    auto arg = [&](int i, size_t d) { return argc > i ? (size_t)std::strtoul(argv[i], nullptr, 10) : d; };
    const size_t B = arg(1, 2), S = arg(2, 48);
    LinearGPTConfig cfg;
    cfg.n_embd = arg(3, 64);
    cfg.n_layer = arg(4, 2);
    cfg.vocab_size = arg(5, 96);
    cfg.block_size = S;
    try {
        RNG rng(4321);
        LinearGPT model(cfg, rng);
        return run_model_check(model, linear_numerical_grad_check, rng, B, S, cfg.vocab_size, arg(6, 8),
                               argc > 7 ? std::strtof(argv[7], nullptr) : 3e-3f);
    } catch (const std::exception& e) {
        std::fprintf(stderr, "error: %s\n", e.what());
        return 1;
    }
}
