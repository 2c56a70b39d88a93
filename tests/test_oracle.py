"""CPU tests of the oracle: against the committed golden vectors (made from the reference's own
kernel_test.cpp functions), against those functions directly when they are built, and against
mathematical identities that pin the LinearGPT flavour, which the reference never tests."""
import os

import numpy as np
import pytest

from conftest import KT_BLOCKS, kt_block_inputs, rel_err, seeded_normal

GOLD = os.path.join(os.path.dirname(__file__), "golden")
STRIDE = 61


def check_packed(gold, name, a):
    a = np.asarray(a, np.float32).ravel()
    if name in gold:
        np.testing.assert_array_equal(a, gold[name])
    else:
        np.testing.assert_array_equal(a[::STRIDE], gold[name + "__sub"])
        sums = gold[name + "__sum"]
        assert np.isclose(a.astype(np.float64).sum(), sums[0], rtol=0, atol=1e-9 * max(1.0, abs(sums[1])))
        assert np.isclose(np.abs(a.astype(np.float64)).sum(), sums[1], rtol=1e-12)


def test_frand_matches_reference_stream(orc):
    gold = np.load(os.path.join(GOLD, "kernel_test_blocks.npz"))
    np.testing.assert_array_equal(orc.frand(64, 0), gold["frand_head"])
    np.testing.assert_array_equal(orc.frand(10, 54), gold["frand_head"][54:])


@pytest.mark.parametrize("index", range(len(KT_BLOCKS)))
def test_oracle_bit_exact_on_kernel_test_blocks(orc, index):
    gold = np.load(os.path.join(GOLD, "kernel_test_blocks.npz"))
    kind, d, (Q, K, V, dO) = kt_block_inputs(orc.frand, index)
    if kind == "mha":
        O = orc.mha_fwd(Q, K, V, **d)
        dQ, dK, dV = orc.mha_bwd(Q, K, V, O, dO, **d)
        outs = dict(O=O, dQ=dQ, dK=dK, dV=dV)
    else:
        O, den, _ = orc.linattn_fwd(Q, K, V, **d)
        dQ, dK, dV = orc.kernel_attn_bwd(Q, K, V, O, dO, den, **d)
        outs = dict(O=O, den=den, dQ=dQ, dK=dK, dV=dV)
    for k, v in outs.items():
        check_packed(gold, f"b{index}_{k}", v)


def test_oracle_bit_exact_on_seeded_cases(orc):
    gold = np.load(os.path.join(GOLD, "seeded_cases.npz"))
    B, S, H, Dh = 8, 64, 4, 32
    Q, K, V, dO = seeded_normal(0, [(B * S, H * Dh)] * 4)
    O = orc.mha_fwd(Q, K, V, B, S, H, Dh)
    dQ, dK, dV = orc.mha_bwd(Q, K, V, O, dO, B, S, H, Dh)
    for k, v in dict(O=O, dQ=dQ, dK=dK, dV=dV).items():
        check_packed(gold, "cfg1_" + k, v)
    B, S, D, E = 32, 64, 32, 32
    Q, K, V, dO = seeded_normal(1, [(B * S, D), (B * S, D), (B * S, E), (B * S, E)])
    O, den, _ = orc.linattn_fwd(Q, K, V, B, S, D, E)
    dQ, dK, dV = orc.kernel_attn_bwd(Q, K, V, O, dO, den, B, S, D, E)
    for k, v in dict(O=O, den=den, dQ=dQ, dK=dK, dV=dV).items():
        check_packed(gold, "cfg2_" + k, v)


@pytest.mark.parametrize("index", [0, 1, 3])
def test_oracle_equals_reference_functions(orc, ref, index):
    """Direct comparison with the reference's compiled functions (small blocks; the large ones are
    covered through the golden file)."""
    kind, d, (Q, K, V, dO) = kt_block_inputs(ref.frand, index)
    if kind == "mha":
        O = ref.mha_fwd(Q, K, V, **d)
        np.testing.assert_array_equal(orc.mha_fwd(Q, K, V, **d), O)
        for a, b in zip(orc.mha_bwd(Q, K, V, O, dO, **d), ref.mha_bwd(Q, K, V, O, dO, **d)):
            np.testing.assert_array_equal(a, b)
    else:
        O, den = ref.kernel_attn_fwd(Q, K, V, **d)
        O2, den2, _ = orc.linattn_fwd(Q, K, V, **d)
        np.testing.assert_array_equal(O2, O)
        np.testing.assert_array_equal(den2, den)
        for a, b in zip(orc.kernel_attn_bwd(Q, K, V, O, dO, den, **d),
                        ref.kernel_attn_bwd(Q, K, V, O, dO, den, **d)):
            np.testing.assert_array_equal(a, b)


def test_stepwise_backward_matches_fused_form(orc):
    """step1 + (dQ, dK, dV from dnum/dden) is the reference CUDA decomposition; it must agree with
    the kernel_test form up to rounding of 1/den."""
    B, S, D, E = 3, 40, 16, 12
    Q, K, V, dO = seeded_normal(5, [(B * S, D), (B * S, D), (B * S, E), (B * S, E)])
    O, den, _ = orc.linattn_fwd(Q, K, V, B, S, D, E)
    want = orc.kernel_attn_bwd(Q, K, V, O, dO, den, B, S, D, E)
    dnum, dden = orc.linattn_step1(O, dO, den)
    got = orc.linattn_bwd(Q, K, V, dnum, dden, B, S, D, E)
    for a, b in zip(got, want):
        assert rel_err(a, b) < 1e-6


def test_linear_gpt_flavour_identity(orc):
    """linear_cuda(phi(Q), phi(K), V) equals kernel_attn(Q, K, V): same O, den differs by the
    stored 1e-8, and the gradients differ by the phi' factor only.  Also checks D > E zero padding
    through phi_elu_fwd (linear_cuda_kernels.cu:316-323)."""
    B, S, E = 2, 50, 24
    D = 32  # next power of two, as LinearGPT pads
    x_q, x_k, V, dO = seeded_normal(7, [(B * S, E)] * 4)
    Qp, Kp = orc.phi_elu_fwd(x_q, D), orc.phi_elu_fwd(x_k, D)
    assert np.all(Qp[:, E:] == 0) and np.all(Qp[:, :E] > 0)
    O1, den1, zc1 = orc.linattn_fwd(Qp, Kp, V, B, S, D, E, elu=False)
    O2, den2, zc2 = orc.linattn_fwd(x_q, x_k, V, B, S, E, E, elu=True)
    assert rel_err(O1, O2) < 1e-6
    assert rel_err(den1, den2 + 1e-8) < 1e-6
    assert rel_err(zc1[:, :E], zc2) < 1e-6
    dnum, dden = orc.linattn_step1(O1, dO, den1)
    dQp, dKp, dV1 = orc.linattn_bwd(Qp, Kp, V, dnum, dden, B, S, D, E, elu=False)
    dQ1, dK1 = orc.phi_elu_bwd(dQp, x_q), orc.phi_elu_bwd(dKp, x_k)
    dnum2, dden2 = orc.linattn_step1(O2, dO, den2)
    dQ2, dK2, dV2 = orc.linattn_bwd(x_q, x_k, V, dnum2, dden2, B, S, E, E, elu=True)
    assert rel_err(dQ1, dQ2) < 1e-5 and rel_err(dK1, dK2) < 1e-5 and rel_err(dV1, dV2) < 1e-5


def test_f32_and_f64_oracles_agree(orc):
    B, S, H, Dh = 2, 48, 2, 16
    Q, K, V, dO = seeded_normal(9, [(B * S, H * Dh)] * 4)
    O32 = orc.mha_fwd(Q, K, V, B, S, H, Dh)
    O64, lse = orc.mha_fwd(Q, K, V, B, S, H, Dh, f64=True, want_lse=True)
    assert rel_err(O32, O64) < 1e-6 and np.all(np.isfinite(lse))
    for a, b in zip(orc.mha_bwd(Q, K, V, O32, dO, B, S, H, Dh),
                    orc.mha_bwd(Q, K, V, O32, dO, B, S, H, Dh, f64=True)):
        assert rel_err(a, b) < 1e-6


def _num_grad(f, x, eps=1e-3):
    g = np.zeros_like(x, dtype=np.float64)
    flat = x.reshape(-1)
    for i in range(flat.size):
        old = flat[i]
        flat[i] = old + eps
        hi = f()
        flat[i] = old - eps
        lo = f()
        flat[i] = old
        g.reshape(-1)[i] = (hi - lo) / (2 * eps)
    return g


def test_oracle_gradients_against_finite_differences(orc):
    """The reference validates its models with central differences (gpt_gpt.hpp:751-803); the same
    check pins the backward formulas of the oracle (double accumulation, tiny shapes)."""
    B, S, H, Dh = 1, 5, 1, 4
    Q, K, V, dO = seeded_normal(11, [(B * S, H * Dh)] * 4)
    O = orc.mha_fwd(Q, K, V, B, S, H, Dh, f64=True)
    dQ, dK, dV = orc.mha_bwd(Q, K, V, O, dO, B, S, H, Dh, f64=True)

    def loss():
        return float((orc.mha_fwd(Q, K, V, B, S, H, Dh, f64=True).astype(np.float64) * dO).sum())
    for x, g in ((Q, dQ), (K, dK), (V, dV)):
        assert rel_err(g, _num_grad(loss, x)) < 2e-3

    B, S, D, E = 1, 6, 3, 4
    Q, K, V, dO = seeded_normal(12, [(B * S, D), (B * S, D), (B * S, E), (B * S, E)])
    O, den, _ = orc.linattn_fwd(Q, K, V, B, S, D, E, f64=True)
    dQ, dK, dV = orc.kernel_attn_bwd(Q, K, V, O, dO, den, B, S, D, E, f64=True)

    def loss2():
        return float((orc.linattn_fwd(Q, K, V, B, S, D, E, f64=True)[0].astype(np.float64) * dO).sum())
    for x, g in ((Q, dQ), (K, dK), (V, dV)):
        assert rel_err(g, _num_grad(loss2, x)) < 2e-3


def test_rope_is_orthogonal_and_gelu_matches_closed_form(orc):
    X, = seeded_normal(13, [(12, 16)])
    Y = orc.rope(X, S=6, head_dim=8, sign=1.0)
    np.testing.assert_allclose(orc.rope(Y, S=6, head_dim=8, sign=-1.0), X, atol=1e-6)
    np.testing.assert_allclose((Y ** 2).sum(1), (X ** 2).sum(1), rtol=1e-5)
    np.testing.assert_array_equal(Y[0], X[0])  # position 0 is not rotated
    from math import erf, sqrt
    x = np.linspace(-4, 4, 33).astype(np.float32)
    want = np.array([0.5 * v * (1 + erf(v / sqrt(2))) for v in x])
    np.testing.assert_allclose(orc.gelu_exact(x), want, atol=1e-6)
    num = (orc.gelu_exact(x + 1e-3).astype(np.float64) - orc.gelu_exact(x - 1e-3)) / 2e-3
    np.testing.assert_allclose(orc.gelu_exact(x, deriv=True), num, atol=2e-3)
