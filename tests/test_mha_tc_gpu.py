"""GPU parity of the tcgen05 (bf16) softmax MHA kernels against the CPU oracle, through the C-ABI.
Inputs are generated in fp32, rounded to bf16, and the SAME rounded values are given to the oracle
(double accumulation).  Tolerance for the bf16 tensor-core path: 2e-2 as max|a-b| / max|b|."""
import numpy as np
import pytest
import torch

from conftest import rel_err

pytestmark = pytest.mark.gpu
TOL_BF16 = 2e-2


def test_umma_operand_conventions(pkg, dev):
    """Single-tile products that pin the shared-memory / tensor-memory operand layouts the attention
    kernels assume (K-major x K-major, TMEM x MN-major, MN-major x MN-major)."""
    g = torch.Generator().manual_seed(1)
    A64 = torch.randn(128, 64, generator=g).bfloat16()
    A128 = torch.randn(128, 128, generator=g).bfloat16()
    B = torch.randn(128, 64, generator=g).bfloat16()
    cases = [(0, A64, (128, 128), A64.float() @ B.float().T),
             (1, A128, (128, 64), A128.float() @ B.float()),
             (2, A128, (128, 64), A128.float().T @ B.float())]
    for mode, A, shape, want in cases:
        D = torch.full(shape, float("nan"), device=dev)
        pkg.selftest_umma(mode, A.to(dev), B.to(dev), D)
        pkg.sync_status()
        err = rel_err(D.cpu().numpy(), want.numpy())
        assert err < 1e-5, (mode, err)


def bf16_inputs(seed, B, S, H, Dh, n=4, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(B * S, H * Dh, generator=g) * scale).bfloat16() for _ in range(n)]


def run_fwd(pkg, dev, Q, K, V, B, S, H, Dh):
    tq, tk, tv = (x.to(dev) for x in (Q, K, V))
    O = torch.full_like(tq, float("nan"))
    lse = torch.full((B * H * S,), float("nan"), device=dev)
    pkg.mha_fwd(tq, tk, tv, O, B, S, H, Dh, lse=lse)
    pkg.sync_status()
    return O, lse


@pytest.mark.parametrize("B,S,H,Dh", [(1, 128, 1, 64), (1, 256, 1, 64), (2, 512, 3, 64), (1, 384, 2, 64),
                                      (2, 1024, 2, 64), (1, 200, 2, 64), (1, 77, 1, 64), (1, 2048, 1, 64)])
def test_forward_matches_oracle(pkg, dev, orc, B, S, H, Dh):
    Q, K, V = bf16_inputs(7 + S, B, S, H, Dh, n=3)
    O, lse = run_fwd(pkg, dev, Q, K, V, B, S, H, Dh)
    rO, rl = orc.mha_fwd(Q.float().numpy(), K.float().numpy(), V.float().numpy(), B, S, H, Dh,
                         f64=True, want_lse=True)
    got = O.float().cpu().numpy()
    assert np.all(np.isfinite(got))
    assert rel_err(got, rO) < TOL_BF16, rel_err(got, rO)
    assert np.abs(lse.cpu().numpy() - rl).max() < 2e-2


def test_forward_long_sequence_properties(pkg, dev, orc):
    """S=4096 with 12 heads of 64 (the long-sequence shape): causality (bit-identical prefix when
    later keys/values change) and parity on one (batch, head) slice."""
    B, S, H, Dh = 1, 4096, 12, 64
    Q, K, V = bf16_inputs(3, B, S, H, Dh, n=3)
    O1, _ = run_fwd(pkg, dev, Q, K, V, B, S, H, Dh)
    cut = 3000
    K2, V2 = K.clone(), V.clone()
    K2[cut:] = -K2[cut:]
    V2[cut:] = V2[cut:] + 1
    O2, _ = run_fwd(pkg, dev, Q, K2, V2, B, S, H, Dh)
    assert torch.equal(O1[:cut], O2[:cut]) and not torch.equal(O1[cut:], O2[cut:])
    h = 5
    sl = slice(h * Dh, (h + 1) * Dh)
    rO = orc.mha_fwd(Q[:, sl].float().numpy(), K[:, sl].float().numpy(), V[:, sl].float().numpy(),
                     1, S, 1, Dh, f64=True)
    assert rel_err(O1[:, sl].float().cpu().numpy(), rO) < TOL_BF16


def run_fwd_bwd(pkg, dev, Q, K, V, dO, B, S, H, Dh, use_lse=True):
    tq, tk, tv, tg = (x.to(dev) for x in (Q, K, V, dO))
    O = torch.full_like(tq, float("nan"))
    lse = torch.full((B * H * S,), float("nan"), device=dev)
    pkg.mha_fwd(tq, tk, tv, O, B, S, H, Dh, lse=lse)
    dQ, dK, dV = (torch.full_like(tq, float("nan")) for _ in range(3))
    pkg.mha_bwd(tq, tk, tv, O, tg, dQ, dK, dV, B, S, H, Dh, lse=lse if use_lse else None)
    pkg.sync_status()
    return O, dQ, dK, dV


@pytest.mark.parametrize("B,S,H,Dh", [(1, 128, 1, 64), (1, 256, 1, 64), (2, 512, 3, 64), (1, 384, 2, 64),
                                      (2, 1024, 2, 64), (1, 200, 2, 64), (1, 77, 1, 64)])
def test_backward_matches_oracle(pkg, dev, orc, B, S, H, Dh):
    Q, K, V, dO = bf16_inputs(17 + S, B, S, H, Dh)
    O, dQ, dK, dV = run_fwd_bwd(pkg, dev, Q, K, V, dO, B, S, H, Dh)
    f = [x.float().numpy() for x in (Q, K, V, dO)]
    # the reference backward consumes the stored (here bf16-rounded) O of the forward under test
    rdQ, rdK, rdV = orc.mha_bwd(f[0], f[1], f[2], O.float().cpu().numpy(), f[3], B, S, H, Dh, f64=True)
    for name, a, b in (("dQ", dQ, rdQ), ("dK", dK, rdK), ("dV", dV, rdV)):
        got = a.float().cpu().numpy()
        assert np.all(np.isfinite(got)), name
        assert rel_err(got, b) < TOL_BF16, (name, rel_err(got, b))


def test_backward_without_lse_recomputes_statistics(pkg, dev):
    """The kept reference signature carries no row statistics: passing lse=NULL must give the same
    gradients as reusing the forward's (dK and dV bit-identical; dQ is summed with atomics)."""
    B, S, H, Dh = 2, 640, 2, 64
    Q, K, V, dO = bf16_inputs(5, B, S, H, Dh)
    a = run_fwd_bwd(pkg, dev, Q, K, V, dO, B, S, H, Dh, use_lse=True)
    b = run_fwd_bwd(pkg, dev, Q, K, V, dO, B, S, H, Dh, use_lse=False)
    assert torch.equal(a[2], b[2]) and torch.equal(a[3], b[3])
    assert rel_err(a[1].float().cpu().numpy(), b[1].float().cpu().numpy()) < 1e-2


def test_backward_long_sequence_properties(pkg, dev, orc):
    """S=4096, 12 heads x 64: gradients of one (batch, head) slice against the oracle, and
    linearity in dO (dX(a*dO) == a*dX(dO) for a power of two, exact in bf16/fp32)."""
    B, S, H, Dh = 1, 4096, 12, 64
    Q, K, V, dO = bf16_inputs(9, B, S, H, Dh)
    O, dQ, dK, dV = run_fwd_bwd(pkg, dev, Q, K, V, dO, B, S, H, Dh)
    _, dQ2, dK2, dV2 = run_fwd_bwd(pkg, dev, Q, K, V, dO * 4, B, S, H, Dh)
    assert torch.equal(dK2.float(), dK.float() * 4) and torch.equal(dV2.float(), dV.float() * 4)
    assert rel_err(dQ2.float().cpu().numpy(), 4 * dQ.float().cpu().numpy()) < 1e-2
    h = 7
    sl = slice(h * Dh, (h + 1) * Dh)
    f = [x[:, sl].float().numpy() for x in (Q, K, V, dO)]
    rdQ, rdK, rdV = orc.mha_bwd(f[0], f[1], f[2], O[:, sl].float().cpu().numpy(), f[3], 1, S, 1, Dh, f64=True)
    for name, a, b in (("dQ", dQ, rdQ), ("dK", dK, rdK), ("dV", dV, rdV)):
        assert rel_err(a[:, sl].float().cpu().numpy(), b) < TOL_BF16, name


def test_persistent_schedule_many_ragged_items(pkg, dev, orc):
    """More work items than SMs, of unequal length, with a ragged last query-tile pair (5 tiles):
    every persistent CTA walks several items in both kernels.  Parity on two (batch, head) slices."""
    B, S, H, Dh = 9, 640, 12, 64
    Q, K, V, dO = bf16_inputs(23, B, S, H, Dh)
    O, dQ, dK, dV = run_fwd_bwd(pkg, dev, Q, K, V, dO, B, S, H, Dh)
    for b, h in ((0, 0), (8, 11)):
        rows = slice(b * S, (b + 1) * S)
        cols = slice(h * Dh, (h + 1) * Dh)
        f = [x[rows, cols].float().numpy() for x in (Q, K, V, dO)]
        rO = orc.mha_fwd(f[0], f[1], f[2], 1, S, 1, Dh, f64=True)
        got_O = O[rows, cols].float().cpu().numpy()
        assert rel_err(got_O, rO) < TOL_BF16
        rdQ, rdK, rdV = orc.mha_bwd(f[0], f[1], f[2], got_O, f[3], 1, S, 1, Dh, f64=True)
        for name, a, ref in (("dQ", dQ, rdQ), ("dK", dK, rdK), ("dV", dV, rdV)):
            got = a[rows, cols].float().cpu().numpy()
            assert np.all(np.isfinite(got)), name
            assert rel_err(got, ref) < TOL_BF16, (name, rel_err(got, ref))


def test_backward_beyond_32_tiles_takes_one_cta_per_item(pkg, dev, orc):
    """33 query tiles: the backward leaves its persistent schedule (one CTA per (key tile, batch*head)
    item instead); same parity bar."""
    B, S, H, Dh = 1, 4224, 2, 64
    Q, K, V, dO = bf16_inputs(29, B, S, H, Dh)
    O, dQ, dK, dV = run_fwd_bwd(pkg, dev, Q, K, V, dO, B, S, H, Dh)
    cols = slice(Dh, 2 * Dh)
    f = [x[:, cols].float().numpy() for x in (Q, K, V, dO)]
    got_O = O[:, cols].float().cpu().numpy()
    rO = orc.mha_fwd(f[0], f[1], f[2], 1, S, 1, Dh, f64=True)
    assert rel_err(got_O, rO) < TOL_BF16
    rdQ, rdK, rdV = orc.mha_bwd(f[0], f[1], f[2], got_O, f[3], 1, S, 1, Dh, f64=True)
    for name, a, ref in (("dQ", dQ, rdQ), ("dK", dK, rdK), ("dV", dV, rdV)):
        got = a[:, cols].float().cpu().numpy()
        assert np.all(np.isfinite(got)), name
        assert rel_err(got, ref) < TOL_BF16, (name, rel_err(got, ref))


def check_slices(orc, Q, K, V, dO, O, dQ, dK, dV, S, H, Dh, slices):
    """Parity of chosen (batch, head) slices against the fp64 oracle; O of the kernel under test is
    what the oracle's backward consumes, as in the reference."""
    for b, h in slices:
        rows = slice(b * S, (b + 1) * S)
        cols = slice(h * Dh, (h + 1) * Dh)
        f = [x[rows, cols].float().numpy() for x in (Q, K, V, dO)]
        got_O = O[rows, cols].float().cpu().numpy()
        rO = orc.mha_fwd(f[0], f[1], f[2], 1, S, 1, Dh, f64=True)
        assert np.all(np.isfinite(got_O))
        assert rel_err(got_O, rO) < TOL_BF16, ("O", b, h, rel_err(got_O, rO))
        rdQ, rdK, rdV = orc.mha_bwd(f[0], f[1], f[2], got_O, f[3], 1, S, 1, Dh, f64=True)
        for name, a, ref in (("dQ", dQ, rdQ), ("dK", dK, rdK), ("dV", dV, rdV)):
            got = a[rows, cols].float().cpu().numpy()
            assert np.all(np.isfinite(got)), (name, b, h)
            # the floor matters for a single token only: its dQ and dK are zero by cancellation
            assert rel_err(got, ref, floor=1e-3) < TOL_BF16, (name, b, h, rel_err(got, ref, floor=1e-3))


def test_long_sequence_sweep_shape_s16384(pkg, dev, orc):
    """B=4, S=16384, 12 heads x 64 — the longest point of the sequence sweep, at full size.  128 key
    tiles per row: the forward in its default (late-wait) instantiation and the backward with one CTA
    per (key tile, batch*head) item of 128 query tiles.  Parity on the last (batch, head) slice, the
    one whose items are scheduled last."""
    B, S, H, Dh = 4, 16384, 12, 64
    assert pkg.get_option(pkg.OPT_FWD_LATE_WAIT) == -1 and pkg.get_option(pkg.OPT_BWD_PERSISTENT) == -1
    Q, K, V, dO = bf16_inputs(31, B, S, H, Dh)
    O, dQ, dK, dV = run_fwd_bwd(pkg, dev, Q, K, V, dO, B, S, H, Dh)
    for t in (O, dQ, dK, dV):
        assert bool(torch.isfinite(t.float()).all())
    check_slices(orc, Q, K, V, dO, O, dQ, dK, dV, S, H, Dh, [(3, 11)])


def test_long_sequence_sweep_shape_s1024(pkg, dev, orc):
    """B=64, S=1024, 12 heads x 64 — the shortest point of the sweep at full size: 768 (batch, head)
    units of 8 tiles, every persistent CTA walks dozens of items.  Parity on three slices."""
    B, S, H, Dh = 64, 1024, 12, 64
    Q, K, V, dO = bf16_inputs(37, B, S, H, Dh)
    O, dQ, dK, dV = run_fwd_bwd(pkg, dev, Q, K, V, dO, B, S, H, Dh)
    for t in (O, dQ, dK, dV):
        assert bool(torch.isfinite(t.float()).all())
    check_slices(orc, Q, K, V, dO, O, dQ, dK, dV, S, H, Dh, [(0, 0), (31, 5), (63, 11)])


@pytest.mark.parametrize("S", [77, 200, 640, 1024])
def test_forward_wait_placement_option_both_settings(pkg, dev, orc, S):
    """CXXATTN_OPT_FWD_LATE_WAIT forces either instantiation of the forward kernel (where a softmax
    warp waits for the previous PV product); both must meet the oracle on ragged last tile pairs and
    with several items per CTA, and give the same O and lse bit for bit (the arithmetic is the
    same, only the order of waits differs)."""
    B, H, Dh = 3, 2, 64
    Q, K, V = bf16_inputs(41 + S, B, S, H, Dh, n=3)
    rO, rl = orc.mha_fwd(Q.float().numpy(), K.float().numpy(), V.float().numpy(), B, S, H, Dh, f64=True, want_lse=True)
    out = []
    for setting in (0, 1):
        with pkg.forced_option(pkg.OPT_FWD_LATE_WAIT, setting):
            O, lse = run_fwd(pkg, dev, Q, K, V, B, S, H, Dh)
        assert rel_err(O.float().cpu().numpy(), rO) < TOL_BF16, setting
        assert np.abs(lse.cpu().numpy() - rl).max() < 2e-2, setting
        out.append((O, lse))
    assert pkg.get_option(pkg.OPT_FWD_LATE_WAIT) == -1
    assert torch.equal(out[0][0], out[1][0]) and torch.equal(out[0][1], out[1][1])


def test_backward_schedule_option_both_settings(pkg, dev, orc):
    """CXXATTN_OPT_BWD_PERSISTENT forces the persistent or the CTA-per-item schedule of the backward;
    both meet the oracle, dK and dV agree bit for bit (each key tile is summed in the same order by
    one CTA either way; dQ is summed in arrival order)."""
    B, S, H, Dh = 2, 640, 2, 64
    Q, K, V, dO = bf16_inputs(43, B, S, H, Dh)
    res = []
    for setting in (0, 1):
        with pkg.forced_option(pkg.OPT_BWD_PERSISTENT, setting):
            O, dQ, dK, dV = run_fwd_bwd(pkg, dev, Q, K, V, dO, B, S, H, Dh)
        check_slices(orc, Q, K, V, dO, O, dQ, dK, dV, S, H, Dh, [(0, 0), (1, 1)])
        res.append((dQ, dK, dV))
    assert torch.equal(res[0][1], res[1][1]) and torch.equal(res[0][2], res[1][2])
    assert rel_err(res[0][0].float().cpu().numpy(), res[1][0].float().cpu().numpy()) < 1e-2


def test_bounded_wait_gives_up_and_reports(pkg, dev):
    """A device-side wait that can never be satisfied (one CTA waiting on a barrier nothing arrives
    on, limit 1 ms) returns by itself: the status call reports the timeout and the wait site, the
    flag is cleared, and a normal launch right after it is correct."""
    import ctypes as C
    pkg.sync_status()  # clean slate
    pkg.selftest_wait_limit(1_000_000)
    rc = pkg.lib().cxxattn_sync_status(C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -5 and "timed out" in pkg.strerror(rc)
    assert pkg.lib().cxxattn_last_timeout_site() == 990
    pkg.sync_status()  # cleared: no exception
    g = torch.Generator().manual_seed(1)
    A = torch.randn(128, 64, generator=g).bfloat16()
    Bm = torch.randn(128, 64, generator=g).bfloat16()
    D = torch.full((128, 128), float("nan"), device=dev)
    pkg.selftest_umma(0, A.to(dev), Bm.to(dev), D)
    pkg.sync_status()
    assert rel_err(D.cpu().numpy(), (A.float() @ Bm.float().T).numpy()) < 1e-5


def test_head_range_inside_full_width_rows_matches_the_dense_call(pkg, dev):
    """What a rank of the 8-GPU split of the S=16384 point does: heads 6..11 of a batch item are
    addressed in place inside rows of 12 heads through the descriptor's strides (stride_b = S*H*Dh,
    stride_s = H*Dh, stride_h = Dh, base pointer moved by 6*Dh elements).  Same bits as the dense call on
    compact copies for O, lse, dK, dV; dQ within its arrival-order noise; the other heads' columns of the
    output tensors are not written."""
    B, S, H, Dh, h0, nh = 2, 640, 12, 64, 6, 6
    Q, K, V, dO = (t.to(dev) for t in bf16_inputs(53, B, S, H, Dh))
    cols = slice(h0 * Dh, (h0 + nh) * Dh)
    strides = (S * H * Dh, H * Dh, Dh)

    def outputs():
        return [torch.full_like(Q, 9.0) for _ in range(4)]
    O, dQ, dK, dV = outputs()
    lse = torch.empty(B * nh * S, device=dev)
    view = lambda t: t[:, cols]
    pkg.mha_fwd(view(Q), view(K), view(V), view(O), B, S, nh, Dh, lse=lse, strides=strides)
    pkg.mha_bwd(view(Q), view(K), view(V), view(O), view(dO), view(dQ), view(dK), view(dV), B, S, nh, Dh, lse=lse,
                strides=strides)
    cq, ck, cv, cg = (view(t).contiguous() for t in (Q, K, V, dO))
    cO, cdQ, cdK, cdV = (torch.empty_like(cq) for _ in range(4))
    clse = torch.empty_like(lse)
    pkg.mha_fwd(cq, ck, cv, cO, B, S, nh, Dh, lse=clse)
    pkg.mha_bwd(cq, ck, cv, cO, cg, cdQ, cdK, cdV, B, S, nh, Dh, lse=clse)
    pkg.sync_status()
    assert torch.equal(view(O), cO) and torch.equal(lse, clse)
    assert torch.equal(view(dK), cdK) and torch.equal(view(dV), cdV)
    assert rel_err(view(dQ).float().cpu().numpy(), cdQ.float().cpu().numpy()) < 1e-2
    for t in (O, dQ, dK, dV):  # heads 0..5 untouched
        assert bool((t[:, :h0 * Dh] == 9.0).all())


@pytest.mark.parametrize("B,S,H", [(1, 1, 1), (2, 129, 3), (40, 130, 12)])
def test_edge_shapes_forward_and_backward(pkg, dev, orc, B, S, H):
    """A single token, one row past a tile border, and 480 short (batch, head) units (more items than SMs
    in both kernels, each with a ragged second tile)."""
    Dh = 64
    Q, K, V, dO = bf16_inputs(59 + S, B, S, H, Dh)
    O, dQ, dK, dV = run_fwd_bwd(pkg, dev, Q, K, V, dO, B, S, H, Dh)
    check_slices(orc, Q, K, V, dO, O, dQ, dK, dV, S, H, Dh, [(0, 0), (B - 1, H - 1)])
