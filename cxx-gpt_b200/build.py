"""Builds libcxxattn.so (all CUDA kernels + the C-ABI) in-tree for sm_100a with nvcc.

    python cxx-gpt_b200/build.py [--force] [--verbose]

nvcc cross-compiles without a GPU.  The shared object lands next to this file so that it
travels with the source tree.
"""
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
LIB = os.path.join(HERE, "libcxxattn.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def sources():
    return sorted(glob.glob(os.path.join(HERE, "csrc", "*.cu")))


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = sources() + glob.glob(os.path.join(HERE, "csrc", "*.cuh")) + \
        glob.glob(os.path.join(ROOT, "include", "*.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    if not force and not _stale():
        return LIB
    objs = []
    procs = []
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    for src in sources():
        obj = os.path.join(HERE, "build", os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        cmd = ["nvcc"] + NVCC_FLAGS + \
              (["-Xptxas", "-v"] if verbose else []) + \
              ["-I", os.path.join(ROOT, "include"), "-I", os.path.join(HERE, "csrc"), "-c", src, "-o", obj]
        procs.append((cmd, subprocess.Popen(cmd)))
    for cmd, p in procs:
        if p.wait() != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
    subprocess.check_call(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB] + objs + ["-lcuda"])
    return LIB


COMPAT_CHECK = os.path.join(HERE, "build", "rope_fused_check")


def build_compat_check(force=False):
    """Compiles compat/rope_fused_check.cpp with the adapter against libcxxattn.so: the program that
    compares the adapter's rope-folded attention pair with the reference's sequence of calls."""
    compat = os.path.join(HERE, "compat")
    srcs = [os.path.join(compat, "rope_fused_check.cpp"), os.path.join(compat, "cxxgpt_kernels.cpp")]
    deps = srcs + [os.path.join(compat, "cxxgpt_kernels.hpp"), os.path.join(compat, "TensorN.hpp"),
                   os.path.join(ROOT, "include", "cxxattn.h"), LIB]
    if force or not os.path.exists(COMPAT_CHECK) or \
            any(os.path.getmtime(d) > os.path.getmtime(COMPAT_CHECK) for d in deps):
        os.makedirs(os.path.dirname(COMPAT_CHECK), exist_ok=True)
        subprocess.check_call(["nvcc", "-std=c++17", "-O2", "-Wno-deprecated-gpu-targets", "-I", compat,
                               "-I", os.path.join(ROOT, "include"), "-o", COMPAT_CHECK] + srcs +
                              ["-L", HERE, "-lcxxattn", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/.."])
    return COMPAT_CHECK


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    print(build_compat_check(force="--force" in sys.argv))
