"""GPU parity against the reference's OWN CUDA kernels (compiled unmodified for sm_100 into
oracle/_ref/libref_cuda.so): same inputs, same GPU, this library's fp32 kernels vs
two_stage_cuda::* / linear_cuda::* of the reference.  Tolerance 1e-5 as max|a-b|/max|b| per
tensor (the reference uses __expf where this library uses expf)."""
import numpy as np
import pytest
import torch

from conftest import rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-5


@pytest.fixture(scope="module")
def refcuda():
    import oracle
    if not oracle.ReferenceCuda.available():
        pytest.skip("reference CUDA kernels not built and reference tree not mounted")
    return oracle.ReferenceCuda()


def rnd(dev, seed, *shape, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dev)


@pytest.mark.parametrize("B,S,H,Dh", [(8, 64, 4, 32), (2, 300, 1, 128), (2, 256, 2, 64), (2, 6, 2, 8)])
def test_softmax_mha_matches_reference_kernels(pkg, dev, refcuda, B, S, H, Dh):
    Q, K, V, dO = (rnd(dev, 10 + i, B * S, H * Dh) for i in range(4))
    O, dQ, dK, dV = (torch.empty_like(Q) for _ in range(4))
    rO, rdQ, rdK, rdV = (torch.empty_like(Q) for _ in range(4))
    pkg.two_stage_cuda.fused_mha_fwd(Q, K, V, O, B, S, H, Dh)
    refcuda.mha_fwd(Q, K, V, rO, B, S, H, Dh)
    pkg.two_stage_cuda.fused_mha_bwd(Q, K, V, rO, dO, dQ, dK, dV, B, S, H, Dh)
    refcuda.mha_bwd(Q, K, V, rO, dO, rdQ, rdK, rdV, B, S, H, Dh)
    torch.cuda.synchronize()
    for name, a, b in (("O", O, rO), ("dQ", dQ, rdQ), ("dK", dK, rdK), ("dV", dV, rdV)):
        assert rel_err(a.cpu().numpy(), b.cpu().numpy()) < TOL, name


@pytest.mark.parametrize("B,S,D,E", [(32, 64, 32, 32), (32, 1024, 32, 32), (8, 64, 128, 128), (2, 5, 7, 6),
                                     (2, 32, 256, 256), (6, 512, 64, 64)])
def test_elu_kernel_attention_matches_reference_kernels(pkg, dev, refcuda, B, S, D, E):
    N = B * S
    Q, K = rnd(dev, 1, N, D), rnd(dev, 2, N, D)
    V, dO = rnd(dev, 3, N, E), rnd(dev, 4, N, E)
    buf = refcuda.scan_buffers(B, S, D, E, dev)
    refcuda.kernel_attn(Q, K, V, dO, buf, B, S, D, E)
    mine = refcuda.scan_buffers(B, S, D, E, dev)
    ts = pkg.two_stage_cuda
    ts.kernel_attn_fwd(Q, K, V, mine["O"], mine["den"], mine["zc"], mine["Sbuf"], mine["zbuf"], B, S, D, E)
    # backward from the reference's O / den, so both sides differentiate the same forward
    ts.kernel_attn_bwd_step1(buf["O"], dO, buf["den"], mine["dnum"], mine["dden"], N, E)
    ts.kernel_attn_bwd_dQ(K, V, mine["dnum"], mine["dden"], buf["zc"], Q, mine["dQ"], mine["Sbuf"], B, S, D, E)
    ts.kernel_attn_bwd_dKdV(Q, K, V, mine["dnum"], mine["dden"], mine["dK"], mine["dV"], B, S, D, E)
    torch.cuda.synchronize()
    for k in ("O", "den", "zc", "dnum", "dden", "dQ", "dK", "dV"):
        assert rel_err(mine[k].cpu().numpy(), buf[k].cpu().numpy(), floor=1e-3) < TOL, k


@pytest.mark.parametrize("B,S,D,E", [(96, 256, 64, 64), (2, 128, 1024, 768), (3, 70, 32, 16)])
def test_linear_gpt_scan_matches_reference_kernels(pkg, dev, refcuda, B, S, D, E):
    """The LinearGPT flavour has no CPU code in the reference; its CUDA kernels are the only pin.
    E is kept a power of two: the reference's step-1 kernel reduces over min(E, 256) threads with a
    halving tree (linear_cuda_kernels.cu:127-131, 142), which drops terms for other block sizes."""
    N = B * S
    x_q, x_k = rnd(dev, 5, N, E, std=0.5), rnd(dev, 6, N, E, std=0.5)
    V, dO = rnd(dev, 7, N, E), rnd(dev, 8, N, E)
    lc = pkg.linear_cuda
    Qp, Kp = torch.empty(N, D, device=dev), torch.empty(N, D, device=dev)
    lc.phi_elu_forward(x_q, Qp, D, E)
    lc.phi_elu_forward(x_k, Kp, D, E)
    buf = refcuda.scan_buffers(B, S, D, E, dev)
    refcuda.linear(Qp, Kp, V, dO, buf, B, S, D, E)
    mine = refcuda.scan_buffers(B, S, D, E, dev)
    lc.causal_linear_attention_fwd(Qp, Kp, V, mine["O"], mine["den"], mine["zc"], mine["Sbuf"], mine["zbuf"], B, S, D, E)
    lc.causal_linear_attention_bwd_step1(buf["O"], dO, buf["den"], mine["dnum"], mine["dden"], N, E)
    lc.causal_linear_attention_bwd_dQ(Kp, V, mine["dnum"], mine["dden"], buf["zc"], mine["dQ"], mine["Sbuf"], B, S, D, E)
    lc.causal_linear_attention_bwd_dKdV(Qp, Kp, V, mine["dnum"], mine["dden"], mine["dK"], mine["dV"], B, S, D, E)
    torch.cuda.synchronize()
    for k in ("O", "den", "zc", "dnum", "dden", "dQ", "dK", "dV"):
        assert rel_err(mine[k].cpu().numpy(), buf[k].cpu().numpy(), floor=1e-3) < 2e-5, k
