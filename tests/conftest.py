import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def orc():
    import oracle
    return oracle.Oracle()


@pytest.fixture(scope="session")
def ref():
    """The reference's own kernel_test.cpp functions; skipped when neither the reference tree nor
    a prebuilt oracle/_ref is present."""
    import oracle
    if not oracle.Reference.available():
        pytest.skip("reference functions not built and reference tree not mounted")
    return oracle.Reference()


@pytest.fixture(scope="session")
def pkg():
    import __graft_entry__ as g
    return g.load_package()


@pytest.fixture(scope="session")
def dev():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    return torch.device("cuda:0")


def rel_err(a, b, floor=1e-30):
    """max|a-b| / max|b| — the per-tensor error measure used for every tolerance in this suite.
    `floor` bounds the denominator from below for tensors whose exact value is zero by
    cancellation (e.g. dQ of a length-1 sequence)."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), floor))


def assert_parity(name, got, want32, want64=None, tol=1e-5, floor=1e-30):
    """Parity rule of this suite.  A tensor passes when it is within `tol` (max|a-b|/max|b|) of the
    fp32 oracle.  Where the quantity is dominated by cancellation (e.g. dQ of linear attention on
    N(0, 0.02^2) inputs) the fp32 oracle itself is further than `tol` from the exact value; the
    double-accumulating oracle `want64` (array or zero-argument callable) then adjudicates: the
    tensor passes when its distance to the fp64 result is within 3x the fp32 oracle's own."""
    e32 = rel_err(got, want32, floor)
    if e32 < tol:
        return e32
    if want64 is not None:
        w64 = want64() if callable(want64) else want64
        eg, eo = rel_err(got, w64, floor), rel_err(want32, w64, floor)
        if eg <= max(tol, 3 * eo):
            return eg
        raise AssertionError(f"{name}: vs fp32 oracle {e32:.3e}, vs fp64 oracle {eg:.3e}, "
                             f"fp32 oracle vs fp64 oracle {eo:.3e}, tol {tol:.1e}")
    raise AssertionError(f"{name}: {e32:.3e} >= {tol:.1e}")


# Draw counts of the blocks of the reference kernel test (src/TwoStage/kernel_test.cpp:215-441),
# in file order; each block draws Q, K, V, dO from one std::mt19937(1234) stream.
KT_BLOCKS = [
    ("mha", dict(B=2, S=6, H=2, Dh=8)),       # :217
    ("lin", dict(B=2, S=6, D=8, E=8)),        # :254
    ("mha", dict(B=2, S=300, H=1, Dh=128)),   # :303
    ("lin", dict(B=2, S=5, D=7, E=6)),        # :337
    ("mha", dict(B=2, S=256, H=2, Dh=64)),    # :378
    ("lin", dict(B=2, S=32, D=256, E=256)),   # :412
]


def kt_block_inputs(frand, index):
    """Inputs of block `index` of the reference kernel test, drawn with `frand(n, skip)`."""
    skip = 0
    for i, (kind, d) in enumerate(KT_BLOCKS):
        if kind == "mha":
            n = d["B"] * d["S"] * d["H"] * d["Dh"]
            sizes = [n, n, n, n]
            shapes = [(d["B"] * d["S"], d["H"] * d["Dh"])] * 4
        else:
            N = d["B"] * d["S"]
            sizes = [N * d["D"], N * d["D"], N * d["E"], N * d["E"]]
            shapes = [(N, d["D"]), (N, d["D"]), (N, d["E"]), (N, d["E"])]
        if i == index:
            x = frand(sum(sizes), skip)
            out, o = [], 0
            for s, sh in zip(sizes, shapes):
                out.append(x[o:o + s].reshape(sh).copy())
                o += s
            return kind, d, out
        skip += sum(sizes)
    raise IndexError(index)


def seeded_normal(seed, shapes, std=1.0):
    rng = np.random.default_rng(seed)
    return [(rng.standard_normal(s) * std).astype(np.float32) for s in shapes]
