// Found in place of CXX-GPT's src/tokenizer.hpp (which needs nlohmann/json and a tokenizer file)
// when the model headers are compiled for checks that feed synthetic token ids.  gpt_gpt.hpp only
// includes the tokenizer; it never calls it.
#pragma once
#include <string>
#include <vector>

class BPETokenizer {
public:
    bool load(const std::string&) { return false; }
    size_t vocab_size() const { return 0; }
    std::vector<int> encode(const std::string&, bool = false, bool = false) const { return {}; }
    std::string decode(const std::vector<int>&) const { return {}; }
};
