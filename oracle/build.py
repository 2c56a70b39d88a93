"""Compile the CPU oracle (oracle.cpp) and, when the reference tree is mounted, the reference's
own CPU test functions (ref_wrap.cpp, which includes src/TwoStage/kernel_test.cpp where it
lies) into oracle/_ref/.  Test infrastructure only; building the checker is not using it.

    python oracle/build.py [--reference /path/to/CXX-GPT]

The CXX-GPT source tree is taken from --reference, else from the environment variable
CXXGPT_REFERENCE, else from a checkout named `reference` beside this repository; without one the
previously built files under oracle/_ref/ are used as they are.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_REFERENCE = os.environ.get("CXXGPT_REFERENCE") or \
    os.path.normpath(os.path.join(HERE, os.pardir, os.pardir, "reference"))


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.exists(s) and os.path.getmtime(s) > t for s in sources)


def build_oracle(force=False):
    src = os.path.join(HERE, "oracle.cpp")
    out = os.path.join(HERE, "liboracle.so")
    if force or _stale(out, [src]):
        subprocess.check_call(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fopenmp",
                               "-o", out, src])
    return out


def build_reference(reference=DEFAULT_REFERENCE, force=False):
    """Returns the path of libref_kernel_test.so, or None when neither the reference tree nor a
    previously built copy is available."""
    out_dir = os.path.join(HERE, "_ref")
    out = os.path.join(out_dir, "libref_kernel_test.so")
    ref_src = os.path.join(reference, "src", "TwoStage", "kernel_test.cpp")
    if not os.path.exists(ref_src):
        return out if os.path.exists(out) else None
    wrap = os.path.join(HERE, "ref_wrap.cpp")
    stub = os.path.join(HERE, "ref_stub")
    if force or _stale(out, [wrap, ref_src, os.path.join(stub, "TwoStage", "two_stage_gpt.hpp")]):
        os.makedirs(out_dir, exist_ok=True)
        subprocess.check_call(["g++", "-O2", "-std=c++17", "-fPIC", "-shared",
                               "-I", stub, "-I", os.path.join(reference, "src"),
                               "-o", out, wrap])
    return out


def build_dropin_kernel_test(reference=DEFAULT_REFERENCE, force=False):
    """Compiles the reference's UNMODIFIED src/TwoStage/kernel_test.cpp against this repository's
    kernels (compat adapter + libcxxattn.so) into oracle/_ref/kernel_test_dropin.  Returns its path,
    or None when neither the reference tree nor a previously built binary is available."""
    root = os.path.dirname(HERE)
    pkg = os.path.join(root, "cxx-gpt_b200")
    out_dir = os.path.join(HERE, "_ref")
    out = os.path.join(out_dir, "kernel_test_dropin")
    ref_src = os.path.join(reference, "src", "TwoStage", "kernel_test.cpp")
    if not os.path.exists(ref_src):
        return out if os.path.exists(out) else None
    adapter = os.path.join(pkg, "compat", "cxxgpt_kernels.cpp")
    lib = os.path.join(pkg, "libcxxattn.so")
    deps = [ref_src, adapter, lib, os.path.join(pkg, "compat", "cxxgpt_kernels.hpp"),
            os.path.join(pkg, "compat", "TensorN.hpp"), os.path.join(root, "include", "cxxattn.h")]
    if force or _stale(out, deps):
        os.makedirs(out_dir, exist_ok=True)
        subprocess.check_call(["nvcc", "-std=c++17", "-O2", "-Wno-deprecated-gpu-targets",
                               "-I", os.path.join(pkg, "compat"), "-I", os.path.join(root, "include"),
                               "-I", os.path.join(reference, "src"), "-o", out, ref_src, adapter,
                               "-L", pkg, "-lcxxattn", "-Xlinker", "-rpath", "-Xlinker",
                               "$ORIGIN/../../cxx-gpt_b200"])
    return out


def build_reference_cuda(reference=DEFAULT_REFERENCE, force=False):
    """Compiles the reference's UNMODIFIED two_stage_cuda_kernels.cu and linear_cuda_kernels.cu for
    sm_100 (with the TensorN stand-in) plus oracle/ref_cuda_wrap.cu into oracle/_ref/libref_cuda.so.
    Returns its path, or None when neither the reference tree nor a previous build is available."""
    root = os.path.dirname(HERE)
    out_dir = os.path.join(HERE, "_ref")
    out = os.path.join(out_dir, "libref_cuda.so")
    srcs = [os.path.join(reference, "src", "TwoStage", "two_stage_cuda_kernels.cu"),
            os.path.join(reference, "src", "LinearAttention", "linear_cuda_kernels.cu")]
    if not all(os.path.exists(s) for s in srcs):
        return out if os.path.exists(out) else None
    wrap = os.path.join(HERE, "ref_cuda_wrap.cu")
    compat = os.path.join(root, "cxx-gpt_b200", "compat")
    if force or _stale(out, srcs + [wrap, os.path.join(compat, "TensorN.hpp")]):
        os.makedirs(out_dir, exist_ok=True)
        subprocess.check_call(["nvcc", "-gencode", "arch=compute_100,code=sm_100", "-O3", "-std=c++17",
                               "-Xcompiler", "-fPIC", "-shared", "-Wno-deprecated-gpu-targets",
                               "-I", compat, "-I", os.path.join(reference, "src"), "-o", out, wrap] + srcs)
    return out

def build_model_checks(reference=DEFAULT_REFERENCE, force=False):
    """Compiles the reference's UNMODIFIED model headers (src/TwoStage/two_stage_gpt.hpp,
    src/LinearAttention/linear_gpt.hpp, src/GPT/gpt_gpt.hpp) and its src/GPT/gpt_cuda_kernels.cu, with
    the wider TensorN stand-in of cxx-gpt_b200/compat/full, into four programs under oracle/_ref/:
      two_stage_check_dropin, linear_gpt_check_dropin   attention kernels = this repository
                                                        (compat adapter + libcxxattn.so)
      two_stage_check_ref, linear_gpt_check_ref         attention kernels = the reference's
                                                        two_stage_cuda_kernels.cu / linear_cuda_kernels.cu
    Returns the dict name -> path, or None when neither the reference tree nor earlier builds are there."""
    root = os.path.dirname(HERE)
    pkg = os.path.join(root, "cxx-gpt_b200")
    full = os.path.join(pkg, "compat", "full")
    out_dir = os.path.join(HERE, "_ref")
    src = os.path.join(reference, "src")
    models = {"two_stage_check": (os.path.join(src, "TwoStage", "two_stage_gpt.hpp"),
                                  os.path.join(src, "TwoStage", "two_stage_cuda_kernels.cu")),
              "linear_gpt_check": (os.path.join(src, "LinearAttention", "linear_gpt.hpp"),
                                   os.path.join(src, "LinearAttention", "linear_cuda_kernels.cu"))}
    outs = {f"{m}_{v}": os.path.join(out_dir, f"{m}_{v}") for m in models for v in ("dropin", "ref")}
    if not all(os.path.exists(h) for h, _ in models.values()):
        return outs if all(os.path.exists(o) for o in outs.values()) else None
    gpt_cu = os.path.join(src, "GPT", "gpt_cuda_kernels.cu")
    ops = os.path.join(full, "tensorn_ops.cu")
    adapter = os.path.join(pkg, "compat", "cxxgpt_kernels.cpp")
    flags = ["nvcc", "-std=c++17", "-O2", "-gencode", "arch=compute_100,code=sm_100", "-Wno-deprecated-gpu-targets",
             "-I", full, "-I", src, "-I", os.path.join(src, "GPT")]
    os.makedirs(out_dir, exist_ok=True)
    for m, (header, kernels_cu) in models.items():
        main = os.path.join(full, m + ".cpp")
        common = [main, ops, gpt_cu, header, os.path.join(src, "GPT", "gpt_gpt.hpp"),
                  os.path.join(full, "model_check.hpp"), os.path.join(full, "TensorN.hpp"),
                  os.path.join(full, "tokenizer.hpp"), os.path.join(pkg, "compat", "TensorN.hpp")]
        dropin, ref = outs[m + "_dropin"], outs[m + "_ref"]
        if force or _stale(dropin, common + [adapter, os.path.join(pkg, "libcxxattn.so"),
                                             os.path.join(root, "include", "cxxattn.h")]):
            subprocess.check_call(flags + ["-I", os.path.join(root, "include"), "-o", dropin, main, ops, gpt_cu,
                                           adapter, "-L", pkg, "-lcxxattn", "-lcublas", "-Xlinker", "-rpath",
                                           "-Xlinker", "$ORIGIN/../../cxx-gpt_b200"])
        if force or _stale(ref, common + [kernels_cu]):
            subprocess.check_call(flags + ["-o", ref, main, ops, gpt_cu, kernels_cu, "-lcublas"])
    return outs


def build_gpt_block_check(reference=DEFAULT_REFERENCE, force=False):
    """Compiles cxx-gpt_b200/compat/full/gpt_block_attention_check.cpp with the reference's
    src/GPT/gpt_cuda_kernels.cu (its mask and softmax-backward kernels, unmodified, where it lies), the
    TensorN stand-in and this repository's adapter into oracle/_ref/gpt_block_attention_check."""
    root = os.path.dirname(HERE)
    pkg = os.path.join(root, "cxx-gpt_b200")
    full = os.path.join(pkg, "compat", "full")
    out = os.path.join(HERE, "_ref", "gpt_block_attention_check")
    src = os.path.join(reference, "src")
    gpt_cu = os.path.join(src, "GPT", "gpt_cuda_kernels.cu")
    if not os.path.exists(gpt_cu):
        return out if os.path.exists(out) else None
    main = os.path.join(full, "gpt_block_attention_check.cpp")
    ops = os.path.join(full, "tensorn_ops.cu")
    adapter = os.path.join(pkg, "compat", "cxxgpt_kernels.cpp")
    deps = [main, ops, gpt_cu, adapter, os.path.join(full, "TensorN.hpp"), os.path.join(pkg, "compat", "TensorN.hpp"),
            os.path.join(pkg, "libcxxattn.so"), os.path.join(root, "include", "cxxattn.h")]
    if force or _stale(out, deps):
        os.makedirs(os.path.dirname(out), exist_ok=True)
        subprocess.check_call(["nvcc", "-std=c++17", "-O2", "-gencode", "arch=compute_100,code=sm_100",
                               "-Wno-deprecated-gpu-targets", "-I", full, "-I", src, "-I", os.path.join(src, "GPT"),
                               "-I", os.path.join(root, "include"), "-o", out, main, ops, gpt_cu, adapter,
                               "-L", pkg, "-lcxxattn", "-lcublas", "-Xlinker", "-rpath", "-Xlinker",
                               "$ORIGIN/../../cxx-gpt_b200"])
    return out


if __name__ == "__main__":
    ref = DEFAULT_REFERENCE
    if "--reference" in sys.argv:
        ref = sys.argv[sys.argv.index("--reference") + 1]
    print(build_oracle(force="--force" in sys.argv))
    print(build_reference(ref, force="--force" in sys.argv))
    print(build_dropin_kernel_test(ref, force="--force" in sys.argv))
    print(build_reference_cuda(ref, force="--force" in sys.argv))
    print(build_model_checks(ref, force="--force" in sys.argv))
    print(build_gpt_block_check(ref, force="--force" in sys.argv))
