// Found in place of CXX-GPT's src/TwoStage/two_stage_gpt.hpp when its kernel unit test
// (src/TwoStage/kernel_test.cpp, which includes "TwoStage/two_stage_gpt.hpp") is compiled
// unmodified against this library.  The real header pulls in the whole model and with it the parts
// of TensorN (GEMM, GGUF) that are not available; the unit test itself only needs the tensor types
// and the kernel entry points.
#pragma once
#include "../cxxgpt_kernels.hpp"
