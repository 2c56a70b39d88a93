"""GPU tests of the data-parallel training step: the fused optimiser kernel against a restatement of
the reference's AdamW, the model on the library's kernels against the same model on the CPU oracle,
training progress on the tensor-core kernels, and (with two or more GPUs) NCCL ranks against one rank."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT, rel_err
from test_hybrid_gpt import OracleKernels, load_hybrid, make_batch, reference_adamw

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,world", [(4096, 1), (1_000_003, 8), (7, 2)])
def test_fused_adamw_matches_the_reference_formula(pkg, dev, n, world):
    g = torch.Generator().manual_seed(n)
    param, grad = torch.randn(n, generator=g), torch.randn(n, generator=g) * world
    m, v = torch.randn(n, generator=g) * 0.1, torch.rand(n, generator=g) * 0.1
    want = [t.clone().double() for t in (param, grad, m, v)]
    nsq_want = torch.zeros(1, dtype=torch.float64)
    dp, dg, dm, dv = (t.to(dev) for t in (param, grad, m, v))
    nsq = torch.zeros(1, device=dev)
    for step in (1, 2, 3):
        reference_adamw(want[0], want[1], want[2], want[3], step, 1e-3, 0.9, 0.999, 0.01, 1e-8, 1.0 / world, nsq_want)
        pkg.adamw_step(dp, dg, dm, dv, step, 1e-3, grad_scale=1.0 / world, grad_norm_sq=nsq)
    torch.cuda.synchronize()
    assert torch.equal(dg.cpu(), grad)  # the gradient buffer is read, not rescaled in place
    for name, a, b in (("param", dp, want[0]), ("m", dm, want[2]), ("v", dv, want[3])):
        assert rel_err(a.cpu().numpy(), b.numpy()) < 1e-5, name  # fp32 kernel against the fp64 restatement
    assert abs(float(nsq) - float(nsq_want)) < 1e-5 * float(nsq_want)


def test_mixed_precision_adamw_matches_the_reference_formula(pkg, dev):
    """bf16 gradient in, fp32 master and moments updated as by the fp32 kernel on the same (bf16-valued)
    gradient, bf16 working copy = the rounded master."""
    n, world = 100_003, 4
    g = torch.Generator().manual_seed(3)
    param, grad = torch.randn(n, generator=g), (torch.randn(n, generator=g) * world).bfloat16()
    m, v = torch.randn(n, generator=g) * 0.1, torch.rand(n, generator=g) * 0.1
    a = [t.clone().to(dev) for t in (param, grad.float(), m, v)]
    b = [t.clone().to(dev) for t in (param, grad, m, v)]
    copy = torch.zeros(n, dtype=torch.bfloat16, device=dev)
    na, nb = torch.zeros(1, device=dev), torch.zeros(1, device=dev)
    for step in (1, 2):
        pkg.adamw_step(a[0], a[1], a[2], a[3], step, 1e-3, grad_scale=1.0 / world, grad_norm_sq=na)
        pkg.adamw_step(b[0], b[1], b[2], b[3], step, 1e-3, grad_scale=1.0 / world, grad_norm_sq=nb, param_copy=copy)
    torch.cuda.synchronize()
    for x, y in zip(a[:1] + a[2:], b[:1] + b[2:]):
        assert torch.equal(x, y)
    assert torch.equal(copy, b[0].bfloat16())
    assert abs(float(na) - float(nb)) < 1e-5 * float(na)  # one atomic per CTA: the order of the sum varies


def test_model_on_the_exact_kernels_matches_the_oracle_model(pkg, dev):
    """fp32 compute: every custom autograd function runs the library's exact kernels; loss and the
    whole flat gradient agree with the same model computed by the CPU oracle."""
    hy = load_hybrid()
    cfg = hy.HybridConfig(vocab_size=50, block_size=32, n_embd=64, n_head=2, n_layer=2, compute_dtype=torch.float32)
    idx, tgt = make_batch(3, 2, 24, 50)
    ref = hy.HybridGPT(cfg, OracleKernels(), torch.device("cpu"), seed=7)
    lr = ref.loss(idx, tgt)
    lr.backward()
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        model = hy.HybridGPT(cfg, hy.CudaKernels(pkg), dev, seed=7)
        assert torch.equal(model.flat_param.cpu(), ref.flat_param)
        lg = model.loss(idx.to(dev), tgt.to(dev))
        lg.backward()
        torch.cuda.synchronize()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    assert abs(float(lg.detach()) - float(lr.detach())) < 1e-5 * abs(float(lr.detach()))
    assert rel_err(model.flat_grad.cpu().numpy(), ref.flat_grad.numpy()) < 1e-4


def test_training_on_the_tensor_core_kernels_learns_and_tracks_fp32(pkg, dev):
    """bf16 compute, heads of 64, width 128 (both stages on their tcgen05 kernels): the first gradient
    is close to the fp32 oracle model's, and a dozen steps on one batch lower the loss."""
    hy = load_hybrid()
    cfg = hy.HybridConfig(vocab_size=64, block_size=128, n_embd=128, n_head=2, n_layer=2, compute_dtype=torch.bfloat16)
    idx, tgt = make_batch(5, 2, 128, 64)
    model = hy.HybridGPT(cfg, hy.CudaKernels(pkg), dev, seed=9)
    step = hy.DataParallelStep(model, lr=1e-3)
    cfg32 = hy.HybridConfig(vocab_size=64, block_size=128, n_embd=128, n_head=2, n_layer=2, compute_dtype=torch.float32)
    ref = hy.HybridGPT(cfg32, OracleKernels(), torch.device("cpu"), seed=9)
    ref.loss(idx, tgt).backward()
    losses = []
    for i in range(12):
        loss, nsq = step.step(idx.to(dev), tgt.to(dev))
        losses.append(float(loss))
        if i == 0:
            g, r = model.flat_grad.float().cpu(), ref.flat_grad  # bf16 gradient buffer in mixed precision
            cos = float((g @ r) / (g.norm() * r.norm()))
            assert cos > 0.995 and abs(float(g.norm() / r.norm()) - 1) < 3e-2, (cos, float(g.norm() / r.norm()))
            assert abs(float(nsq) - float(g.norm() ** 2)) < 1e-3 * float(nsq)
    pkg.sync_status()
    assert all(np.isfinite(losses)) and losses[-1] < losses[0] - 0.3, losses


def _nccl_rank(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import __graft_entry__ as g
    pkg = g.load_package()
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    torch.backends.cuda.matmul.allow_tf32 = False
    hy = load_hybrid()
    cfg = hy.HybridConfig(vocab_size=50, block_size=32, n_embd=64, n_head=2, n_layer=2, compute_dtype=torch.float32)
    model = hy.HybridGPT(cfg, hy.CudaKernels(pkg), dev, seed=13)
    step = hy.DataParallelStep(model, lr=1e-2, n_buckets=3)
    idx, tgt = make_batch(17, 2 * world, 24, 50)
    lo, hi = 2 * rank, 2 * rank + 2
    losses = []
    for _ in range(5):
        loss, _ = step.step(idx[lo:hi].to(dev), tgt[lo:hi].to(dev))
        t = loss.clone()
        dist.all_reduce(t)  # mean of the ranks' losses = loss of the whole batch
        losses.append(float(t) / world)
    if rank == 0:
        torch.save({"losses": losses, "param": model.flat_param.cpu()}, out)
    dist.destroy_process_group()


def test_nccl_ranks_follow_the_single_rank_loss_curve(pkg, dev, tmp_path):
    """Two NCCL ranks with half the batch each against one rank with the whole batch, fp32 compute on
    the exact (deterministic) kernels: the same loss curve and parameters to 1e-5."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = str(tmp_path / "nccl.pt")
    mp.spawn(_nccl_rank, args=(2, 29531, out), nprocs=2, join=True)
    got = torch.load(out)
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        hy = load_hybrid()
        cfg = hy.HybridConfig(vocab_size=50, block_size=32, n_embd=64, n_head=2, n_layer=2, compute_dtype=torch.float32)
        model = hy.HybridGPT(cfg, hy.CudaKernels(pkg), dev, seed=13)
        step = hy.DataParallelStep(model, lr=1e-2, n_buckets=3)
        idx, tgt = make_batch(17, 4, 24, 50)
        losses = [float(step.step(idx.to(dev), tgt.to(dev))[0]) for _ in range(5)]
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    assert np.allclose(got["losses"], losses, rtol=1e-5), (got["losses"], losses)
    # parameters: AdamW divides by sqrt(v), which magnifies the last-bit differences between the mean of two
    # half-batch gradients and the whole-batch gradient wherever a gradient is tiny
    assert rel_err(got["param"].numpy(), model.flat_param.cpu().numpy()) < 1e-4


def test_cuda_graph_replay_follows_the_eager_steps(pkg, dev):
    """Forward + backward captured in a CUDA graph after three eager steps and replayed give the loss
    curve of launching every kernel (fp32 compute on the exact kernels, which are deterministic)."""
    hy = load_hybrid()
    cfg = hy.HybridConfig(vocab_size=50, block_size=32, n_embd=64, n_head=2, n_layer=2, compute_dtype=torch.float32)
    batches = [tuple(t.to(dev) for t in make_batch(40 + i, 2, 24, 50)) for i in range(7)]
    curves = []
    for graph in (False, True):
        model = hy.HybridGPT(cfg, hy.CudaKernels(pkg), dev, seed=21)
        step = hy.DataParallelStep(model, lr=1e-2, cuda_graph=graph)
        curves.append([float(step.step(i, t)[0]) for i, t in batches])
        assert (step.graph is not None) == graph
    torch.cuda.synchronize()
    assert np.allclose(curves[0], curves[1], rtol=1e-6), curves
