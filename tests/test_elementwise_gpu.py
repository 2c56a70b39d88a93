"""GPU parity of the elementwise neighbours (RoPE, erf-GELU, phi) against the CPU oracle."""
import numpy as np
import pytest
import torch

from conftest import rel_err, seeded_normal

pytestmark = pytest.mark.gpu


def test_rope_block_of_reference_kernel_test(pkg, dev, orc):
    """B=2, S=6, D=16, head_dim=8, forward, backward and the aliased round trip
    (kernel_test.cpp:445-498)."""
    B, S, D, hd = 2, 6, 16, 8
    skip = sum(4 * d["B"] * d["S"] * d["H"] * d["Dh"] if k == "mha"
               else d["B"] * d["S"] * (2 * d["D"] + 2 * d["E"])
               for k, d in __import__("conftest").KT_BLOCKS)
    x = orc.frand(4 * B * S * D, skip)
    Q, K, dQ, dK = (x[i * B * S * D:(i + 1) * B * S * D].reshape(B * S, D) for i in range(4))
    ts = pkg.two_stage_cuda
    tq, tk = torch.from_numpy(Q.copy()).to(dev), torch.from_numpy(K.copy()).to(dev)
    ts.rope_fwd(tq, tk, B, S, D, hd)
    assert np.abs(tq.cpu().numpy() - orc.rope(Q, S, hd, 1.0)).max() < 2e-6
    assert np.abs(tk.cpu().numpy() - orc.rope(K, S, hd, 1.0)).max() < 2e-6
    tdq, tdk = torch.from_numpy(dQ.copy()).to(dev), torch.from_numpy(dK.copy()).to(dev)
    ts.rope_bwd(tdq, tdk, B, S, D, hd)
    assert np.abs(tdq.cpu().numpy() - orc.rope(dQ, S, hd, -1.0)).max() < 2e-6
    assert np.abs(tdk.cpu().numpy() - orc.rope(dK, S, hd, -1.0)).max() < 2e-6
    t2 = torch.from_numpy(Q.copy()).to(dev)
    ts.rope_fwd(t2, t2, B, S, D, hd)   # same tensor twice: rotated twice
    ts.rope_bwd(t2, t2, B, S, D, hd)
    assert np.abs(t2.cpu().numpy() - Q).max() < 2e-6


def test_rope_whole_vector_and_long_positions(pkg, dev, orc):
    B, S, D = 2, 256, 64
    X, = seeded_normal(61, [(B * S, D)])
    t = torch.from_numpy(X.copy()).to(dev)
    pkg.two_stage_cuda.rope_fwd(t, None, B, S, D, D)
    assert rel_err(t.cpu().numpy(), orc.rope(X, S, D, 1.0)) < 1e-4   # fp32 angle at p ~ 255


def _bf16_round(a):
    return torch.from_numpy(a).bfloat16().float().numpy()


@pytest.mark.parametrize("B,S,D,hd", [(2, 6, 16, 8), (3, 130, 768, 64), (1, 33, 64, 64)])
def test_rope_cast_all_type_pairs(pkg, dev, orc, B, S, D, hd):
    """The one-pass rotary + conversion gives what rope followed by the conversion gives: equal to
    the in-place kernel bit for bit in fp32, and to the bf16 rounding of the oracle's rotation up to
    the rounding of a value that sits on a bf16 tie (one bf16 ulp = 2^-8 relative)."""
    X, = seeded_normal(63 + S, [(B * S, D)])
    want_f = orc.rope(X, S, hd, 1.0)
    src = torch.from_numpy(X.copy()).to(dev)
    # fp32 -> fp32: the same arithmetic as the in-place kernel
    out = torch.empty_like(src)
    pkg.rope_cast(src, out, B, S, D, hd, 1.0)
    inplace = src.clone()
    pkg.two_stage_cuda.rope_fwd(inplace, None, B, S, D, hd)
    assert torch.equal(out, inplace)
    assert rel_err(out.cpu().numpy(), want_f) < 1e-5
    # fp32 -> bf16 (forward side of the tensor-core kernels)
    outb = torch.empty(B * S, D, dtype=torch.bfloat16, device=dev)
    pkg.rope_cast(src, outb, B, S, D, hd, 1.0)
    assert torch.equal(outb, inplace.bfloat16())
    assert np.abs(outb.float().cpu().numpy() - _bf16_round(want_f)).max() <= 2.0 ** -8 * np.abs(want_f).max()
    # bf16 -> fp32 with the inverse rotation (gradient side): exact on the bf16 input values
    g = outb.clone()
    back = torch.empty_like(src)
    pkg.rope_cast(g, back, B, S, D, hd, -1.0)
    want_b = orc.rope(g.float().cpu().numpy(), S, hd, -1.0)
    assert rel_err(back.cpu().numpy(), want_b) < 1e-5
    assert rel_err(back.cpu().numpy(), X) < 2.0 ** -7   # the round trip loses only the bf16 rounding
    # bf16 -> bf16
    bb = torch.empty_like(g)
    pkg.rope_cast(g, bb, B, S, D, hd, -1.0)
    assert torch.equal(bb, back.bfloat16())


@pytest.mark.parametrize("src_dtype,dst_dtype", [(torch.float32, torch.bfloat16), (torch.bfloat16, torch.bfloat16),
                                                 (torch.bfloat16, torch.float32)])
def test_rope_cast_pair_is_two_single_calls(pkg, dev, src_dtype, dst_dtype):
    B, S, D, hd = 3, 130, 768, 64
    X0, X1 = seeded_normal(71, [(B * S, D), (B * S, D)])
    a, b = (torch.from_numpy(x).to(dev).to(src_dtype) for x in (X0, X1))
    for sign in (1.0, -1.0):
        want = [torch.empty(B * S, D, dtype=dst_dtype, device=dev) for _ in range(2)]
        got = [torch.full((B * S, D), 9.0, dtype=dst_dtype, device=dev) for _ in range(2)]
        pkg.rope_cast(a, want[0], B, S, D, hd, sign)
        pkg.rope_cast(b, want[1], B, S, D, hd, sign)
        pkg.rope_cast_pair(a, b, got[0], got[1], B, S, D, hd, sign)
        assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
    lib = pkg.lib()
    assert lib.cxxattn_rope_cast_pair(a.data_ptr(), None, 0, want[0].data_ptr(), want[1].data_ptr(), 1, B, S, D, hd, 1.0,
                                      None) == -1


def test_rope_cast_rejects_unaligned_and_unknown_types(pkg, dev):
    src = torch.zeros(64, 64, device=dev)
    dst = torch.zeros(64, 64, device=dev)
    with pytest.raises(pkg.CxxAttnError):
        pkg.rope_cast(src.view(-1)[1:65], dst, 1, 1, 64, 64, 1.0)
    lib = pkg.lib()
    assert lib.cxxattn_rope_cast(src.data_ptr(), 5, dst.data_ptr(), 0, 1, 64, 64, 64, 1.0, None) == -2


def test_gelu_exact_and_derivative(pkg, dev, orc):
    X, = seeded_normal(62, [(1000, 37)])
    X *= 3
    t = torch.from_numpy(X).to(dev)
    out = torch.empty_like(t)
    pkg.two_stage_cuda.gelu_exact(t, out)
    assert np.abs(out.cpu().numpy() - orc.gelu_exact(X)).max() < 1e-6
    pkg.two_stage_cuda.gelu_exact_deriv(t, out)
    assert np.abs(out.cpu().numpy() - orc.gelu_exact(X, deriv=True)).max() < 1e-6


def test_phi_elu_padding(pkg, dev, orc):
    N, D, E = 77, 128, 100
    X, G = seeded_normal(63, [(N, E), (N, D)])
    tx, tg = torch.from_numpy(X).to(dev), torch.from_numpy(G).to(dev)
    phi = torch.full((N, D), float("nan"), device=dev)
    pkg.linear_cuda.phi_elu_forward(tx, phi, D, E)
    assert rel_err(phi.cpu().numpy(), orc.phi_elu_fwd(X, D)) < 1e-6
    dx = torch.empty(N, E, device=dev)
    pkg.linear_cuda.phi_elu_backward(tg, tx, dx, D, E)
    assert rel_err(dx.cpu().numpy(), orc.phi_elu_bwd(G, X)) < 1e-6
