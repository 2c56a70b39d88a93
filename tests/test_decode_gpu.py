"""Decoding with carried state against the CPU oracle: T single-token steps must reproduce the rows
of the oracle's full forward pass on the same sequence (the reference's generate() obtains them by
re-running the whole context, two_stage_gpt.hpp:458-474)."""
import numpy as np
import pytest
import torch

from conftest import rel_err, seeded_normal

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,T,D,E,fmap,eps", [(3, 40, 32, 32, "elu1", 0), (2, 33, 7, 6, "elu1", 0),
                                              (4, 20, 64, 64, "none", 1), (2, 25, 128, 96, "none", 1),
                                              (1, 12, 300, 260, "elu1", 0)])
def test_linear_stage_steps_equal_forward_rows(pkg, dev, orc, B, T, D, E, fmap, eps):
    Q, K, V = seeded_normal(300 + D, [(B * T, D), (B * T, D), (B * T, E)])
    if fmap == "none":   # the LinearGPT flavour takes mapped (positive) features
        Q, K = (np.abs(Q) + 0.1).astype(np.float32), (np.abs(K) + 0.1).astype(np.float32)
        O, den, _ = orc.linattn_fwd(Q, K, V, B, T, D, E, elu=False)
    else:
        O, den, _ = orc.linattn_fwd(Q, K, V, B, T, D, E)
    tq, tk, tv = (torch.from_numpy(x.reshape(B, T, -1)).to(dev) for x in (Q, K, V))
    S = torch.zeros(B, D, E, device=dev)
    z = torch.zeros(B, D, device=dev)
    outs, dens = [], []
    for t in range(T):
        o = torch.empty(B, E, device=dev)
        dn = torch.empty(B, device=dev)
        pkg.linattn_decode_step(tq[:, t].contiguous(), tk[:, t].contiguous(), tv[:, t].contiguous(), S, z, o, dn,
                                B, D, E, pkg.MAP_ELU1 if fmap == "elu1" else pkg.MAP_NONE, eps)
        outs.append(o)
        dens.append(dn)
    got = torch.stack(outs, 1).reshape(B * T, E).cpu().numpy()
    got_den = torch.stack(dens, 1).reshape(B * T).cpu().numpy()
    assert rel_err(got, O) < 1e-5
    assert rel_err(got_den, den) < 1e-5


@pytest.mark.parametrize("B,T,H,Dh,cap", [(2, 40, 4, 32, 64), (1, 70, 2, 64, 70), (3, 17, 1, 128, 32),
                                          (2, 9, 3, 40, 16)])
def test_softmax_stage_steps_equal_forward_rows(pkg, dev, orc, B, T, H, Dh, cap):
    Q, K, V = seeded_normal(400 + Dh, [(B * T, H * Dh)] * 3)
    O = orc.mha_fwd(Q, K, V, B, T, H, Dh)
    tq, tk, tv = (torch.from_numpy(x.reshape(B, T, H * Dh)).to(dev) for x in (Q, K, V))
    Kc = torch.full((B, cap, H * Dh), float("nan"), device=dev)   # unwritten rows must never be read
    Vc = torch.full((B, cap, H * Dh), float("nan"), device=dev)
    outs = []
    for t in range(T):
        o = torch.empty(B, H * Dh, device=dev)
        pkg.mha_decode_step(tq[:, t].contiguous(), tk[:, t].contiguous(), tv[:, t].contiguous(), Kc, Vc, t, o,
                            B, cap, H, Dh)
        outs.append(o)
    got = torch.stack(outs, 1).reshape(B * T, H * Dh).cpu().numpy()
    assert rel_err(got, O) < 1e-5
    assert torch.equal(Kc[:, :T], tk) and torch.equal(Vc[:, :T], tv)


def test_softmax_stage_long_cache_takes_key_splits(pkg, dev, orc):
    """Few (batch, head) units and a long prefix: the keys are cut over several CTAs and merged.  The
    cache is filled directly; six steps at the end are compared with the oracle's last rows."""
    B, T, H, Dh = 1, 3003, 2, 64
    Q, K, V = seeded_normal(77, [(B * T, H * Dh)] * 3)
    O = orc.mha_fwd(Q, K, V, B, T, H, Dh)
    d = pkg.mha_desc(B, T, H, Dh)
    import ctypes as C
    assert pkg.lib().cxxattn_mha_decode_workspace_bytes(C.byref(d)) > 0
    tq, tk, tv = (torch.from_numpy(x.reshape(B, T, H * Dh)).to(dev) for x in (Q, K, V))
    Kc, Vc = torch.zeros(B, T, H * Dh, device=dev), torch.zeros(B, T, H * Dh, device=dev)
    Kc[:, :T - 6], Vc[:, :T - 6] = tk[:, :T - 6], tv[:, :T - 6]
    for t in range(T - 6, T):   # about 3000 keys over 12 splits
        o = torch.empty(B, H * Dh, device=dev)
        pkg.mha_decode_step(tq[:, t].contiguous(), tk[:, t].contiguous(), tv[:, t].contiguous(), Kc, Vc, t, o,
                            B, T, H, Dh)
        assert rel_err(o.cpu().numpy(), O.reshape(B, T, H * Dh)[:, t]) < 1e-5


def test_softmax_stage_unaligned_rows_take_the_scalar_loads(pkg, dev, orc):
    """Head dimension 64 normally uses 8-byte loads; a query that does not start on a 16-byte
    boundary must give the same numbers through the scalar path."""
    B, T, H, Dh = 2, 21, 2, 64
    Q, K, V = seeded_normal(91, [(B * T, H * Dh)] * 3)
    O = orc.mha_fwd(Q, K, V, B, T, H, Dh).reshape(B, T, H * Dh)
    tq, tk, tv = (torch.from_numpy(x.reshape(B, T, H * Dh)).to(dev) for x in (Q, K, V))
    Kc, Vc = torch.zeros(B, T, H * Dh, device=dev), torch.zeros(B, T, H * Dh, device=dev)
    Kc[:, :T - 1], Vc[:, :T - 1] = tk[:, :T - 1], tv[:, :T - 1]
    pad = torch.zeros(B * H * Dh + 1, device=dev)
    q_off = pad[1:]                      # 4 bytes past a 16-byte boundary
    q_off.copy_(tq[:, T - 1].reshape(-1))
    assert q_off.data_ptr() % 16 == 4
    o = torch.empty(B, H * Dh, device=dev)
    pkg.mha_decode_step(q_off, tk[:, T - 1].contiguous(), tv[:, T - 1].contiguous(), Kc, Vc, T - 1, o, B, T, H, Dh)
    assert rel_err(o.cpu().numpy(), O[:, T - 1]) < 1e-5
