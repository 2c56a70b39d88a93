"""The reference's own kernel unit test, compiled UNMODIFIED against this library (TensorN shim +
adapter that implements two_stage_cuda::* on the C-ABI), run on the GPU.  The reference program
only prints max|gpu - cpu| per tensor and never fails (kernel_test.cpp:239, 501-502); this test
turns its printout into assertions."""
import os
import re
import subprocess

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu


def test_reference_kernel_test_program_passes_on_this_library():
    exe = os.path.join(ROOT, "oracle", "_ref", "kernel_test_dropin")
    if not os.path.exists(exe):
        import oracle
        if oracle.build.build_dropin_kernel_test() is None:
            pytest.skip("kernel_test_dropin not built and reference tree not mounted")
    out = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = re.findall(r"^(.*\S)\s+maxdiff\s*=\s*([-+0-9.eE]+|nan|inf)\s*$", out.stdout, flags=re.M)
    # 4 + 7 + 4 + 5 + 4 + 5 attention lines and 5 RoPE lines (kernel_test.cpp:239-498)
    assert len(lines) == 34, out.stdout
    assert out.stdout.strip().endswith("done")
    bad = []
    for name, val in lines:
        v = float(val)
        # The program prints ABSOLUTE differences.  The reference README expects ~1e-7 for values of
        # order one; the S=300, Dh=128 block sums 300 terms per element, and the denominators of the
        # D=E=256 block are of order 1e4 (sum over 256 features and up to 32 keys), so for the "den"
        # lines 1e-2 absolute is 1e-6 relative.
        limit = 1e-2 if name.split()[-1] == "den" else 2e-5
        if not (v == v and v < limit):
            bad.append((name, val))
    assert not bad, (bad, out.stdout)


def test_reference_kernel_test_program_in_tensorcore_mode():
    """The same unmodified program with the adapter's opt-in switch: the fp32 signatures run on the bf16
    tensor-core kernels where those exist — the softmax attention with head dimension 64 (the "big
    S=256" block) and the linear attention with one wide head (the "chunk" block, D = E = 256);
    everything else stays on the exact path.  Inputs are uniform in [-1, 1] (outputs and gradients of
    order one), so 2e-2 absolute is the bf16 bar; the denominators of the chunk block are sums of up to
    32 x 256 products of order one, so theirs is 2e-2 of 1e4."""
    exe = os.path.join(ROOT, "oracle", "_ref", "kernel_test_dropin")
    if not os.path.exists(exe):
        import oracle
        if oracle.build.build_dropin_kernel_test() is None:
            pytest.skip("kernel_test_dropin not built and reference tree not mounted")
    env = dict(os.environ, CXXATTN_COMPAT_PRECISION="tensorcore")
    out = subprocess.run([exe], capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = re.findall(r"^(.*\S)\s+maxdiff\s*=\s*([-+0-9.eE]+|nan|inf)\s*$", out.stdout, flags=re.M)
    assert len(lines) == 34, out.stdout
    big = [(n, float(v)) for n, v in lines if n.startswith("big S=256")]
    assert len(big) == 4, lines
    for name, v in big:
        # above the fp32 path's error (so the tensor-core kernels really ran), below the bf16 bar
        assert 2e-5 < v < 2e-2, (name, v)
    chunk = [(n, float(v)) for n, v in lines if n.startswith("chunk")]
    assert len(chunk) == 5, lines
    for name, v in chunk:
        assert v == v and v < (2e2 if name.split()[-1] == "den" else 2e-2), (name, v)
    assert max(v for n, v in chunk if n.split()[-1] != "den") > 2e-6  # the tensor-core kernels really ran
    for name, val in lines:
        if name.startswith("big S=256") or name.startswith("chunk"):
            continue
        v = float(val)
        limit = 1e-2 if name.split()[-1] == "den" else 2e-5
        assert v == v and v < limit, (name, val)


def _rope_fused_lines(env=None, args=()):
    exe = os.path.join(ROOT, "cxx-gpt_b200", "build", "rope_fused_check")
    if not os.path.exists(exe):
        import importlib.util
        spec = importlib.util.spec_from_file_location("cxx_gpt_b200_build", os.path.join(ROOT, "cxx-gpt_b200", "build.py"))
        b = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(b)
        b.build_compat_check()
    out = subprocess.run([exe, *map(str, args)], capture_output=True, text=True, timeout=600,
                         env=dict(os.environ, **(env or {})))
    assert out.returncode == 0, out.stderr[-2000:]
    assert out.stdout.strip().endswith("done")
    return {n: float(v) for n, v in
            re.findall(r"^(.*\S)\s+maxdiff\s*=\s*([-+0-9.eE]+|nan|inf)\s*$", out.stdout, flags=re.M)}


@pytest.mark.parametrize("shape", [(2, 300, 3, 64), (1, 129, 2, 32)])
def test_rope_folded_attention_pair_equals_the_reference_call_sequence(shape):
    """cxxattn_compat::rope_fused_mha_fwd / _bwd against rope_fwd; fused_mha_fwd; fused_mha_bwd; rope_bwd
    (two_stage_gpt.hpp:102-106, 171-174) on the exact path: same arithmetic, inputs left un-rotated."""
    d = _rope_fused_lines(args=shape)
    assert len(d) == 6, d
    for k in ("rope+mha O", "rope+mha dQ", "rope+mha dK", "rope+mha dV"):
        assert d[k] < 1e-6, d
    assert d["inputs untouched"] == 0.0
    assert d["rotation applied"] > 0.1


def test_rope_folded_attention_pair_in_tensorcore_mode():
    """Both sides on the bf16 tensor-core kernels: the folded pair rounds the rotated fp32 values to
    bf16 exactly as the separate rotation + conversion does, so the results still agree closely."""
    d = _rope_fused_lines(env={"CXXATTN_COMPAT_PRECISION": "tensorcore"}, args=(2, 300, 3, 64))
    for k in ("rope+mha O", "rope+mha dQ", "rope+mha dK", "rope+mha dV"):
        assert d[k] < 1e-6, d
    assert d["inputs untouched"] == 0.0
