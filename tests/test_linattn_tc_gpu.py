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


def run_fwd_bwd(pkg, dev, Q, K, V, dO, B, S, fmap, eps):
    tq, tk, tv, tg = (x.to(dev) for x in (Q, K, V, dO))
    O = torch.full_like(tv, float("nan"))
    den = torch.full((B * S,), float("nan"), device=dev)
    pkg.linattn_fwd(tq, tk, tv, O, den, None, B, S, 64, 64, fmap, eps)
    dQ, dK, dV = (torch.full_like(tq, float("nan")) for _ in range(3))
    pkg.linattn_bwd(tq, tk, tv, O, tg, den, dQ, dK, dV, B, S, 64, 64, fmap, eps)
    pkg.sync_status()
    return [t.float().cpu().numpy() for t in (O, den, dQ, dK, dV)]


@pytest.mark.parametrize("B,S", [(1, 128), (2, 256), (2, 1000), (1, 77), (3, 2048)])
def test_elu_backward_matches_oracle(pkg, dev, orc, B, S):
    Q, K, V = inputs(21 + S, B, S, 64, 64)
    dO = torch.randn(B * S, 64, generator=torch.Generator().manual_seed(S)).bfloat16()
    O, den, dQ, dK, dV = run_fwd_bwd(pkg, dev, Q, K, V, dO, B, S, pkg.MAP_ELU1, 0)
    f = [x.float().numpy() for x in (Q, K, V, dO)]
    # the reference backward consumes the stored O and den of the forward under test
    rdQ, rdK, rdV = orc.kernel_attn_bwd(f[0], f[1], f[2], O, f[3], den, B, S, 64, 64, f64=True)
    for name, a, b in (("dQ", dQ, rdQ), ("dK", dK, rdK), ("dV", dV, rdV)):
        assert np.all(np.isfinite(a)), name
        assert rel_err(a, b) < TOL_BF16, (name, rel_err(a, b))


def test_premapped_backward_matches_oracle(pkg, dev, orc):
    B, S = 2, 700
    Q, K, V = inputs(31, B, S, 64, 64, positive=True)
    dO = torch.randn(B * S, 64, generator=torch.Generator().manual_seed(7)).bfloat16()
    O, den, dQ, dK, dV = run_fwd_bwd(pkg, dev, Q, K, V, dO, B, S, pkg.MAP_NONE, 1)
    f = [x.float().numpy() for x in (Q, K, V, dO)]
    dnum, dden = orc.linattn_step1(O, f[3], den, f64=True)
    rdQ, rdK, rdV = orc.linattn_bwd(f[0], f[1], f[2], dnum, dden, B, S, 64, 64, elu=False, f64=True)
    for name, a, b in (("dQ", dQ, rdQ), ("dK", dK, rdK), ("dV", dV, rdV)):
        assert rel_err(a, b) < TOL_BF16, (name, rel_err(a, b))


def test_backward_long_sequence_linearity_and_subset_parity(pkg, dev, orc):
    """S=4096: dX(4*dO) == 4*dX(dO) (a power of two is exact in bf16/fp32 up to the bf16 roundings
    it moves), and parity on one unit."""
    B, S = 4, 4096
    Q, K, V = inputs(41, B, S, 64, 64)
    dO = torch.randn(B * S, 64, generator=torch.Generator().manual_seed(9)).bfloat16()
    O, den, dQ, dK, dV = run_fwd_bwd(pkg, dev, Q, K, V, dO, B, S, pkg.MAP_ELU1, 0)
    _, _, dQ4, dK4, dV4 = run_fwd_bwd(pkg, dev, Q, K, V, dO * 4, B, S, pkg.MAP_ELU1, 0)
    for a, b in ((dQ4, dQ), (dK4, dK), (dV4, dV)):
        assert rel_err(a, 4 * b) < 1e-2
    f = [x[:S].float().numpy() for x in (Q, K, V, dO)]
    rdQ, rdK, rdV = orc.kernel_attn_bwd(f[0], f[1], f[2], O[:S], f[3], den[:S], 1, S, 64, 64, f64=True)
    for name, a, b in (("dQ", dQ, rdQ), ("dK", dK, rdK), ("dV", dV, rdV)):
        assert rel_err(a[:S], b) < TOL_BF16, (name, rel_err(a[:S], b))


def test_sequence_groups_agree_with_single_pass(pkg, dev, orc):
    """Few units: the sequence is cut into groups of chunks that run as separate CTAs, seeded by a
    state pre-pass (the workspace holds the group states).  Without a workspace one CTA walks the
    whole unit.  Both must match the oracle, and each other closely; 11 chunks give groups of
    unequal length, the last chunk is ragged."""
    import ctypes as C
    B, S = 3, 1300
    Q, K, V = inputs(51, B, S, 64, 64)
    dO = torch.randn(B * S, 64, generator=torch.Generator().manual_seed(3)).bfloat16()
    d = pkg.lin_desc(B, S, 64, 64, pkg.BF16, pkg.MAP_ELU1, 0)
    assert pkg.lib().cxxattn_linattn_workspace_bytes(C.byref(d)) > 0  # groups are planned for this shape
    grouped = run_fwd_bwd(pkg, dev, Q, K, V, dO, B, S, pkg.MAP_ELU1, 0)

    tq, tk, tv, tg = (x.to(dev) for x in (Q, K, V, dO))
    O = torch.full_like(tv, float("nan"))
    den = torch.full((B * S,), float("nan"), device=dev)
    dQ, dK, dV = (torch.full_like(tq, float("nan")) for _ in range(3))
    lib = pkg.lib()
    assert lib.cxxattn_linattn_fwd(C.byref(d), tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), O.data_ptr(),
                                   den.data_ptr(), None, None, 0, None) == 0
    torch.cuda.synchronize()
    assert lib.cxxattn_linattn_bwd(C.byref(d), tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), O.data_ptr(),
                                   tg.data_ptr(), den.data_ptr(), dQ.data_ptr(), dK.data_ptr(), dV.data_ptr(),
                                   None, 0, None) == 0
    pkg.sync_status()
    single = [t.float().cpu().numpy() for t in (O, den, dQ, dK, dV)]
    for name, a, b in zip(("O", "den", "dQ", "dK", "dV"), grouped, single):
        assert np.all(np.isfinite(a)) and np.all(np.isfinite(b)), name
        assert rel_err(a, b) < 1e-2, (name, rel_err(a, b))
    f = [x.float().numpy() for x in (Q, K, V, dO)]
    rO, rden, _ = orc.linattn_fwd(f[0], f[1], f[2], B, S, 64, 64, elu=True, f64=True)
    for got in (grouped, single):
        assert rel_err(got[0], rO) < TOL_BF16 and rel_err(got[1], rden) < TOL_BF16
        rdQ, rdK, rdV = orc.kernel_attn_bwd(f[0], f[1], f[2], got[0], f[3], got[1], B, S, 64, 64, f64=True)
        for name, a, b in (("dQ", got[2], rdQ), ("dK", got[3], rdK), ("dV", got[4], rdV)):
            assert rel_err(a, b) < TOL_BF16, (name, rel_err(a, b))


def test_many_units_take_one_group(pkg, dev, orc):
    """With more units than SMs nothing is cut (no workspace is asked for) and the results are the
    single-pass ones."""
    import ctypes as C
    B, S = 320, 256
    d = pkg.lin_desc(B, S, 64, 64, pkg.BF16, pkg.MAP_ELU1, 0)
    assert pkg.lib().cxxattn_linattn_workspace_bytes(C.byref(d)) == 0
    Q, K, V = inputs(61, B, S, 64, 64)
    O, den = run(pkg, dev, Q, K, V, B, S, pkg.MAP_ELU1, 0)
    n = 4 * S
    rO, rden, _ = orc.linattn_fwd(Q[:n].float().numpy(), K[:n].float().numpy(), V[:n].float().numpy(), 4, S, 64, 64,
                                  elu=True, f64=True)
    assert rel_err(O[:n], rO) < TOL_BF16 and rel_err(den[:n], rden) < TOL_BF16


def check_units(orc, Q, K, V, dO, res, S, units):
    O, den, dQ, dK, dV = res
    for u in units:
        r = slice(u * S, (u + 1) * S)
        f = [x[r].float().numpy() for x in (Q, K, V, dO)]
        rO, rden, _ = orc.linattn_fwd(f[0], f[1], f[2], 1, S, 64, 64, elu=True, f64=True)
        assert rel_err(O[r], rO) < TOL_BF16, ("O", u, rel_err(O[r], rO))
        assert rel_err(den[r], rden) < TOL_BF16, ("den", u)
        rdQ, rdK, rdV = orc.kernel_attn_bwd(f[0], f[1], f[2], O[r], f[3], den[r], 1, S, 64, 64, f64=True)
        for name, a, b in (("dQ", dQ, rdQ), ("dK", dK, rdK), ("dV", dV, rdV)):
            # the floor matters for a single token only: its dQ and dK are zero by cancellation
            floor = 0.2 if S == 1 else 1e-30  # absolute bar 4e-3 on terms of order one
            assert rel_err(a[r], b, floor=floor) < TOL_BF16, (name, u, rel_err(a[r], b, floor=floor))


def test_long_sequence_sweep_shape_s16384(pkg, dev, orc):
    """48 units x S=16384 (B=4 x 12 heads folded) — the longest point of the sequence sweep at full
    size: fewer units than SMs, so every unit is cut into sequence groups seeded by the state
    pre-passes (the backward's suffix pre-pass on the side stream).  Parity on the first and last unit."""
    import ctypes as C
    B, S = 48, 16384
    d = pkg.lin_desc(B, S, 64, 64, pkg.BF16, pkg.MAP_ELU1, 0)
    assert pkg.lib().cxxattn_linattn_workspace_bytes(C.byref(d)) > 0  # groups are planned
    Q, K, V = inputs(71, B, S, 64, 64)
    dO = torch.randn(B * S, 64, generator=torch.Generator().manual_seed(11)).bfloat16()
    res = run_fwd_bwd(pkg, dev, Q, K, V, dO, B, S, pkg.MAP_ELU1, 0)
    for a in res:
        assert np.all(np.isfinite(a))
    check_units(orc, Q, K, V, dO, res, S, [0, 47])


def test_long_sequence_sweep_shape_s1024(pkg, dev, orc):
    """768 units x S=1024 (B=64 x 12 heads folded): more units than SMs, one group, several waves."""
    B, S = 768, 1024
    Q, K, V = inputs(73, B, S, 64, 64)
    dO = torch.randn(B * S, 64, generator=torch.Generator().manual_seed(13)).bfloat16()
    res = run_fwd_bwd(pkg, dev, Q, K, V, dO, B, S, pkg.MAP_ELU1, 0)
    for a in res:
        assert np.all(np.isfinite(a))
    check_units(orc, Q, K, V, dO, res, S, [0, 400, 767])


@pytest.mark.parametrize("groups", [1, 2, 5])
def test_group_count_option(pkg, dev, orc, groups):
    """CXXATTN_OPT_LIN_GROUPS forces the number of sequence groups; every setting meets the oracle."""
    B, S = 3, 1300
    Q, K, V = inputs(81, B, S, 64, 64)
    dO = torch.randn(B * S, 64, generator=torch.Generator().manual_seed(5)).bfloat16()
    with pkg.forced_option(pkg.OPT_LIN_GROUPS, groups):
        res = run_fwd_bwd(pkg, dev, Q, K, V, dO, B, S, pkg.MAP_ELU1, 0)
    check_units(orc, Q, K, V, dO, res, S, [0, 2])


def test_side_stream_option_both_settings(pkg, dev):
    """The suffix-state pre-pass of the backward runs on the library's side stream or in line
    (CXXATTN_OPT_LIN_SIDE_STREAM); the results are the same bits either way."""
    B, S = 3, 1300
    Q, K, V = inputs(83, B, S, 64, 64)
    dO = torch.randn(B * S, 64, generator=torch.Generator().manual_seed(7)).bfloat16()
    out = []
    for setting in (1, 0):
        with pkg.forced_option(pkg.OPT_LIN_SIDE_STREAM, setting):
            out.append(run_fwd_bwd(pkg, dev, Q, K, V, dO, B, S, pkg.MAP_ELU1, 0))
    for a, b in zip(*out):
        assert np.array_equal(a, b)


def test_host_entry_point_matches_device_entry_points(pkg, dev):
    """cxxattn_linattn_fwd_bwd_host (host tensors in and out, chunked over the units) gives the bits of
    the device-pointer entry points on the same chunks."""
    B, S = 12, 512
    Q, K, V = inputs(91, B, S, 64, 64)
    dO = torch.randn(B * S, 64, generator=torch.Generator().manual_seed(17)).bfloat16()
    hO, hdQ, hdK, hdV = (torch.empty(B * S, 64, dtype=torch.bfloat16) for _ in range(4))
    hden = torch.empty(B * S)
    plan = pkg.LinHostPlan(B, S, 64, 64, pkg.BF16, 5)  # chunks of 5, 5, 2 units
    plan.fwd_bwd(Q, K, V, dO, hO, hden, hdQ, hdK, hdV)
    plan.close()
    for lo, hi in ((0, 5), (5, 10), (10, 12)):
        r = slice(lo * S, hi * S)
        want = run_fwd_bwd(pkg, dev, Q[r], K[r], V[r], dO[r], hi - lo, S, pkg.MAP_ELU1, 0)
        got = [t[r].float().numpy() for t in (hO, hden, hdQ, hdK, hdV)]
        for name, a, b in zip(("O", "den", "dQ", "dK", "dV"), got, want):
            assert np.array_equal(a, b), (name, lo)


@pytest.mark.parametrize("B,S", [(1, 1), (2, 129), (300, 130)])
def test_edge_shapes(pkg, dev, orc, B, S):
    """A single token, one row past a chunk border, more units than SMs with a ragged second chunk."""
    Q, K, V = inputs(95 + S, B, S, 64, 64)
    dO = torch.randn(B * S, 64, generator=torch.Generator().manual_seed(S)).bfloat16()
    res = run_fwd_bwd(pkg, dev, Q, K, V, dO, B, S, pkg.MAP_ELU1, 0)
    for a in res:
        assert np.all(np.isfinite(a))
    check_units(orc, Q, K, V, dO, res, S, [0, B - 1])
