"""GPU parity of the tcgen05 (bf16) linear attention with one wide head — the widths the models call
(TwoStageGPT stage 2: D = E = n_embd; LinearGPT: D = next_pow2(n_embd), E = n_embd, pre-mapped
features) — against the CPU oracle, through the C-ABI.  Inputs are rounded to bf16 first and the same
rounded values go to the oracle (double accumulation).  Tolerance of the bf16 path: 2e-2."""
import ctypes as C

import numpy as np
import pytest
import torch

from conftest import rel_err

pytestmark = pytest.mark.gpu
TOL_BF16 = 2e-2


def inputs(seed, B, S, D, E, positive, scale):
    g = torch.Generator().manual_seed(seed)
    Q, K = (torch.randn(B * S, D, generator=g) * scale for _ in range(2))
    V, dO = (torch.randn(B * S, E, generator=g) for _ in range(2))
    if positive:  # pre-mapped features of the LinearGPT flavour are positive
        Q, K = Q.abs() + 0.1, K.abs() + 0.1
    return [t.bfloat16() for t in (Q, K, V, dO)]


def run(pkg, dev, Q, K, V, dO, B, S, D, E, fmap, eps):
    tq, tk, tv, tg = (x.to(dev) for x in (Q, K, V, dO))
    O = torch.full_like(tv, float("nan"))
    den = torch.full((B * S,), float("nan"), device=dev)
    pkg.linattn_fwd(tq, tk, tv, O, den, None, B, S, D, E, fmap, eps)
    dQ, dK = torch.full_like(tq, float("nan")), torch.full_like(tq, float("nan"))
    dV = torch.full_like(tv, float("nan"))
    pkg.linattn_bwd(tq, tk, tv, O, tg, den, dQ, dK, dV, B, S, D, E, fmap, eps)
    pkg.sync_status()
    return [t.float().cpu().numpy() for t in (O, den, dQ, dK, dV)]


@pytest.mark.parametrize("B,S,D,E", [(2, 256, 128, 128), (3, 200, 256, 256), (1, 256, 768, 768), (2, 77, 128, 320),
                                     (1, 600, 192, 128), (8, 256, 768, 768)])
def test_elu_flavour_matches_oracle(pkg, dev, orc, B, S, D, E):
    """two_stage_cuda::kernel_attn_* semantics (ELU+1 fused, den stored without the 1e-8), one head of
    width D -> E; ragged last tiles, result widths that are not a multiple of the column group, several
    row tiles per unit."""
    Q, K, V, dO = inputs(5 + S + D, B, S, D, E, False, 0.5)
    O, den, dQ, dK, dV = run(pkg, dev, Q, K, V, dO, B, S, D, E, pkg.MAP_ELU1, 0)
    f = [x.float().numpy() for x in (Q, K, V, dO)]
    rO, rden, _ = orc.linattn_fwd(f[0], f[1], f[2], B, S, D, E, elu=True, f64=True)
    assert np.all(np.isfinite(O)) and np.all(np.isfinite(den))
    assert rel_err(O, rO) < TOL_BF16, rel_err(O, rO)
    assert rel_err(den, rden) < TOL_BF16, rel_err(den, rden)
    # the reference backward consumes the stored O and den of the forward under test
    rdQ, rdK, rdV = orc.kernel_attn_bwd(f[0], f[1], f[2], O, f[3], den, B, S, D, E, f64=True)
    for name, a, b in (("dQ", dQ, rdQ), ("dK", dK, rdK), ("dV", dV, rdV)):
        assert np.all(np.isfinite(a)), name
        assert rel_err(a, b) < TOL_BF16, (name, rel_err(a, b))


@pytest.mark.parametrize("B,S,D,E", [(2, 256, 1024, 768), (2, 130, 256, 128)])
def test_premapped_flavour_matches_oracle(pkg, dev, orc, B, S, D, E):
    """linear_cuda::causal_linear_attention_* semantics: features already mapped, den stored with the
    1e-8, gradients with respect to the mapped features; D = 1024, E = 768 is LinearGPT at n_embd 768."""
    Q, K, V, dO = inputs(7 + S, B, S, D, E, True, 1.0)
    O, den, dQ, dK, dV = run(pkg, dev, Q, K, V, dO, B, S, D, E, pkg.MAP_NONE, 1)
    f = [x.float().numpy() for x in (Q, K, V, dO)]
    rO, rden, _ = orc.linattn_fwd(f[0], f[1], f[2], B, S, D, E, elu=False, f64=True)
    assert rel_err(O, rO) < TOL_BF16 and rel_err(den, rden) < TOL_BF16
    dnum, dden = orc.linattn_step1(O, f[3], den, f64=True)
    rdQ, rdK, rdV = orc.linattn_bwd(f[0], f[1], f[2], dnum, dden, B, S, D, E, elu=False, f64=True)
    for name, a, b in (("dQ", dQ, rdQ), ("dK", dK, rdK), ("dV", dV, rdV)):
        assert rel_err(a, b) < TOL_BF16, (name, rel_err(a, b))


def test_zero_padded_feature_columns_give_the_unpadded_result(pkg, dev):
    """LinearGPT pads its mapped features with zero columns from E to D (phi_elu_forward,
    linear_cuda_kernels.cu:316-323).  The padded call and the call on the first E columns alone agree
    bit for bit in O, den and dV, and the padded gradient columns are exactly zero."""
    B, S, D, E = 2, 256, 256, 192
    Q, K, V, dO = inputs(11, B, S, E, E, True, 1.0)
    pad = torch.zeros(B * S, D - E, dtype=torch.bfloat16)
    Qp, Kp = torch.cat([Q, pad], 1).contiguous(), torch.cat([K, pad], 1).contiguous()
    a = run(pkg, dev, Q, K, V, dO, B, S, E, E, pkg.MAP_NONE, 1)
    b = run(pkg, dev, Qp, Kp, V, dO, B, S, D, E, pkg.MAP_NONE, 1)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1]) and np.array_equal(a[4], b[4])
    assert np.array_equal(a[2], b[2][:, :E]) and np.array_equal(a[3], b[3][:, :E])
    assert not b[2][:, E:].any() and not b[3][:, E:].any()


def test_workspace_is_required_and_widths_off_the_grid_are_refused(pkg, dev):
    lib = pkg.lib()
    t = torch.zeros(256 * 128, dtype=torch.bfloat16, device=dev)
    f = torch.zeros(256, device=dev)
    d = pkg.lin_desc(1, 256, 128, 128, pkg.BF16, pkg.MAP_ELU1, 0)
    assert lib.cxxattn_linattn_workspace_bytes(C.byref(d)) > 0
    p = t.data_ptr()
    assert lib.cxxattn_linattn_fwd(C.byref(d), p, p, p, p, f.data_ptr(), None, None, 0, None) == -3
    odd = pkg.lin_desc(1, 256, 96, 96, pkg.BF16, pkg.MAP_ELU1, 0)  # not a multiple of 64: no bf16 kernel
    assert lib.cxxattn_linattn_fwd(C.byref(odd), p, p, p, p, f.data_ptr(), None, p, 1 << 20, None) == -2


def test_split_backward_entry_points_and_z_cache(pkg, dev, orc):
    """The reference cuts the backward into step 1, dQ and dK/dV calls and hands a z_cache from the
    forward to the dQ call.  In bf16 the same cut (cxxattn_linattn_bwd_dq / _bwd_dkdv with dnum in bf16)
    gives the bits of the fused call, and the forward fills z_cache = running sum of phi(K)."""
    lib = pkg.lib()
    B, S, D, E = 2, 200, 128, 192
    Q, K, V, dO = inputs(23, B, S, D, E, False, 0.5)
    fused = run(pkg, dev, Q, K, V, dO, B, S, D, E, pkg.MAP_ELU1, 0)
    tq, tk, tv, tg = (x.to(dev) for x in (Q, K, V, dO))
    d = pkg.lin_desc(B, S, D, E, pkg.BF16, pkg.MAP_ELU1, 0)
    n = lib.cxxattn_linattn_workspace_bytes(C.byref(d))
    ws = torch.empty(n, dtype=torch.uint8, device=dev)
    O = torch.empty_like(tv)
    den = torch.empty(B * S, device=dev)
    zc = torch.full((B * S, D), float("nan"), device=dev)
    st = torch.cuda.current_stream().cuda_stream
    assert lib.cxxattn_linattn_fwd(C.byref(d), tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), O.data_ptr(), den.data_ptr(),
                                   zc.data_ptr(), ws.data_ptr(), n, st) == 0
    # step 1 on the stored (bf16-rounded) O, as the fused call does, with dnum rounded to bf16
    inv = 1.0 / den
    dnum = (tg.float() * inv[:, None]).bfloat16()
    dden = -(tg.float() * O.float()).sum(1) * inv
    dQ, dK, dV = torch.empty_like(tq), torch.empty_like(tq), torch.empty_like(tv)
    assert lib.cxxattn_linattn_bwd_dq(C.byref(d), tk.data_ptr(), tv.data_ptr(), dnum.data_ptr(), dden.data_ptr(), None,
                                      tq.data_ptr(), dQ.data_ptr(), ws.data_ptr(), n, st) == 0
    assert lib.cxxattn_linattn_bwd_dkdv(C.byref(d), tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), dnum.data_ptr(),
                                        dden.data_ptr(), dK.data_ptr(), dV.data_ptr(), ws.data_ptr(), n, st) == 0
    pkg.sync_status()
    for name, a, b in (("dQ", dQ, fused[2]), ("dK", dK, fused[3]), ("dV", dV, fused[4])):
        assert rel_err(a.float().cpu().numpy(), b) < 5e-3, name  # dden summed in another order, dnum the same bits
    f = [x.float().numpy() for x in (Q, K, V)]
    _, _, rzc = orc.linattn_fwd(f[0], f[1], f[2], B, S, D, E, elu=True, f64=True)
    assert rel_err(zc.cpu().numpy(), rzc) < TOL_BF16


@pytest.mark.parametrize("B,S,D,E", [(1, 1, 128, 128), (2, 128, 64, 128), (2, 100, 128, 64), (3, 257, 192, 320)])
def test_edge_shapes(pkg, dev, orc, B, S, D, E):
    """A single token, exactly one tile, widths where only one of D, E is 64 (these take the wide-head
    kernel too), one row past a tile border with a result width that is not a multiple of the column group."""
    Q, K, V, dO = inputs(31 + S + D, B, S, D, E, False, 0.5)
    O, den, dQ, dK, dV = run(pkg, dev, Q, K, V, dO, B, S, D, E, pkg.MAP_ELU1, 0)
    f = [x.float().numpy() for x in (Q, K, V, dO)]
    rO, rden, _ = orc.linattn_fwd(f[0], f[1], f[2], B, S, D, E, elu=True, f64=True)
    assert rel_err(O, rO) < TOL_BF16 and rel_err(den, rden) < TOL_BF16
    rdQ, rdK, rdV = orc.kernel_attn_bwd(f[0], f[1], f[2], O, f[3], den, B, S, D, E, f64=True)
    # A single token: dQ and dK are a difference of two equal terms (O = v), so what is left of them is the
    # bf16 rounding of O and dnum; they are held to an absolute bar there.
    floor = 5e-2 if S == 1 else 1e-30
    for name, a, b in (("dQ", dQ, rdQ), ("dK", dK, rdK), ("dV", dV, rdV)):
        assert np.all(np.isfinite(a)), name
        assert rel_err(a, b, floor=floor) < TOL_BF16, (name, rel_err(a, b, floor=floor))
