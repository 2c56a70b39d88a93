"""GPU parity of the tcgen05 (bf16) linear attention forward against the CPU oracle, through the
C-ABI.  Inputs are rounded to bf16 first and the same rounded values go to the oracle (double
accumulation).  Tolerance for the bf16 tensor-core path: 2e-2 as max|a-b| / max|b|."""
import numpy as np
import pytest
import torch

from conftest import rel_err

pytestmark = pytest.mark.gpu
TOL_BF16 = 2e-2


def inputs(seed, B, S, D, E, positive=False):
    g = torch.Generator().manual_seed(seed)
    Q, K = (torch.randn(B * S, D, generator=g) for _ in range(2))
    V = torch.randn(B * S, E, generator=g)
    if positive:  # pre-mapped features of the LinearGPT flavour are positive
        Q, K = Q.abs() + 0.1, K.abs() + 0.1
    return Q.bfloat16(), K.bfloat16(), V.bfloat16()


def run(pkg, dev, Q, K, V, B, S, fmap, eps):
    tq, tk, tv = (x.to(dev) for x in (Q, K, V))
    O = torch.full_like(tv, float("nan"))
    den = torch.full((B * S,), float("nan"), device=dev)
    pkg.linattn_fwd(tq, tk, tv, O, den, None, B, S, 64, 64, fmap, eps)
    pkg.sync_status()
    return O.float().cpu().numpy(), den.cpu().numpy()


@pytest.mark.parametrize("B,S", [(1, 128), (2, 256), (3, 384), (2, 1000), (1, 77), (5, 2048)])
def test_elu_forward_matches_oracle(pkg, dev, orc, B, S):
    Q, K, V = inputs(3 + S, B, S, 64, 64)
    O, den = run(pkg, dev, Q, K, V, B, S, pkg.MAP_ELU1, 0)
    rO, rden, _ = orc.linattn_fwd(Q.float().numpy(), K.float().numpy(), V.float().numpy(), B, S, 64, 64,
                                  elu=True, f64=True)
    assert np.all(np.isfinite(O)) and np.all(np.isfinite(den))
    assert rel_err(O, rO) < TOL_BF16, rel_err(O, rO)
    assert rel_err(den, rden) < TOL_BF16, rel_err(den, rden)


@pytest.mark.parametrize("B,S", [(2, 256), (2, 700)])
def test_premapped_forward_matches_oracle(pkg, dev, orc, B, S):
    """LinearGPT flavour: features already mapped, den stored with the 1e-8."""
    Q, K, V = inputs(11 + S, B, S, 64, 64, positive=True)
    O, den = run(pkg, dev, Q, K, V, B, S, pkg.MAP_NONE, 1)
    rO, rden, _ = orc.linattn_fwd(Q.float().numpy(), K.float().numpy(), V.float().numpy(), B, S, 64, 64,
                                  elu=False, f64=True)
    assert rel_err(O, rO) < TOL_BF16 and rel_err(den, rden) < TOL_BF16


def test_long_sequence_causality_and_subset_parity(pkg, dev, orc):
    B, S = 6, 4096
    Q, K, V = inputs(5, B, S, 64, 64)
    O1, d1 = run(pkg, dev, Q, K, V, B, S, pkg.MAP_ELU1, 0)
    cut = 3000
    K2, V2 = K.clone(), V.clone()
    K2.view(B, S, 64)[:, cut:] *= -1
    V2.view(B, S, 64)[:, cut:] += 2
    O2, d2 = run(pkg, dev, Q, K2, V2, B, S, pkg.MAP_ELU1, 0)
    a, b = O1.reshape(B, S, 64), O2.reshape(B, S, 64)
    assert np.array_equal(a[:, :cut], b[:, :cut]) and not np.array_equal(a[:, cut:], b[:, cut:])
    rO, rden, _ = orc.linattn_fwd(Q[:S].float().numpy(), K[:S].float().numpy(), V[:S].float().numpy(), 1, S, 64, 64,
                                  elu=True, f64=True)
    assert rel_err(O1[:S], rO) < TOL_BF16 and rel_err(d1[:S], rden) < TOL_BF16


def test_unsupported_bf16_requests_are_refused(pkg, dev):
    import ctypes as C
    lib = pkg.lib()
    t = torch.zeros(64 * 32, dtype=torch.bfloat16, device=dev)
    d = pkg.lin_desc(1, 64, 32, 32, pkg.BF16, pkg.MAP_ELU1, 0)
    f = torch.zeros(64, device=dev)
    rc = lib.cxxattn_linattn_fwd(C.byref(d), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), f.data_ptr(), None,
                                 None, 0, None)
    assert rc == -2  # D = E = 32 has no bf16 kernel: an error, not a detour through another path
