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


@pytest.mark.parametrize("world,dtype", [(1, torch.bfloat16), (2, torch.bfloat16), (4, torch.bfloat16),
                                         (8, torch.bfloat16), (3, torch.float32), (16, torch.float32)])
def test_exchange_step_on_emulated_ranks_is_mean_then_adamw(pkg, dev, world, dtype):
    """cxxattn_adamw_step_exchange with every rank's buffers on ONE GPU and the ranks' calls made in turn (the
    kernel waits for nothing, so that is a faithful run of the multi-GPU data flow): afterwards every rank's
    parameter buffer holds the same bits, the masters follow the fp64 restatement of mean + AdamW, and the
    ranks' norm shares add up."""
    n = 8 * 12_347
    mixed = dtype == torch.bfloat16
    g = torch.Generator().manual_seed(world)
    param0 = torch.randn(n, generator=g)
    per = (n // 8 + world - 1) // world * 8
    bounds = [(min(n, r * per), min(n, r * per + per)) for r in range(world)]
    copies = [(param0.to(dtype)).to(dev) for _ in range(world)]
    masters = [param0[lo:hi].clone().to(dev) if mixed else copies[r][lo:hi] for r, (lo, hi) in enumerate(bounds)]
    m0, v0 = torch.randn(n, generator=g) * 0.1, torch.rand(n, generator=g) * 0.1
    ms = [m0[lo:hi].clone().to(dev) for lo, hi in bounds]
    vs = [v0[lo:hi].clone().to(dev) for lo, hi in bounds]
    want = [param0.clone().double(), None, m0.double(), v0.double()]
    nsq_want = torch.zeros(1, dtype=torch.float64)
    for step in (1, 2, 3):
        grads = [(torch.randn(n, generator=g) * (1 + r)).to(dtype) for r in range(world)]
        dgrads = [x.to(dev) for x in grads]
        want[1] = sum(x.double() for x in grads)
        nsq_want.zero_()
        reference_adamw(want[0], want[1], want[2], want[3], step, 1e-3, 0.9, 0.999, 0.01, 1e-8, 1.0 / world, nsq_want)
        shares = []
        for r, (lo, hi) in enumerate(bounds):
            nsq = torch.zeros(1, device=dev)
            pkg.adamw_step_exchange(masters[r], ms[r], vs[r], [x.data_ptr() for x in dgrads],
                                    [x.data_ptr() for x in copies], dtype, r, lo, step, 1e-3,
                                    grad_scale=1.0 / world, grad_norm_sq=nsq)
            shares.append(nsq)
        torch.cuda.synchronize()
        for x, y in zip(dgrads, grads):
            assert torch.equal(x.cpu(), y)  # gradients are read only
        for r in range(1, world):
            assert torch.equal(copies[0], copies[r]), (step, r)
        master = torch.cat([x.float() for x in masters]).cpu()
        assert rel_err(master.numpy(), want[0].numpy()) < 1e-5, step
        if mixed:
            assert torch.equal(copies[0].cpu(), master.bfloat16())
        assert abs(sum(float(x) for x in shares) - float(nsq_want)) < 1e-5 * float(nsq_want)
    assert rel_err(torch.cat(ms).cpu().numpy(), want[2].numpy()) < 1e-5
    assert rel_err(torch.cat(vs).cpu().numpy(), want[3].numpy()) < 1e-5


@pytest.mark.parametrize("rows,cols,dtype", [(2048, 768, torch.bfloat16), (2048, 3072, torch.bfloat16),
                                             (1, 8, torch.bfloat16), (333, 200, torch.bfloat16), (100, 4, torch.float32),
                                             (5000, 1028, torch.float32), (129, 65544, torch.bfloat16)])
def test_column_sums_match_fp64_and_leave_the_workspace_zero(pkg, dev, rows, cols, dtype):
    g = torch.Generator().manual_seed(rows + cols)
    X = torch.randn(rows, cols, generator=g).to(dtype)
    want = X.double().sum(0)
    ws = torch.zeros(pkg.colsum_workspace_bytes(cols), dtype=torch.uint8, device=dev)
    dX = X.to(dev)
    for _ in range(3):  # the same workspace, never cleared again
        out = torch.full((cols,), 7.0, dtype=dtype, device=dev)
        pkg.colsum(dX, out, ws)
        torch.cuda.synchronize()
        tol = 2 ** -8 if dtype == torch.bfloat16 else 1e-6  # the output rounding; sums are fp32
        assert rel_err(out.double().cpu().numpy(), want.numpy()) < tol
        assert int(ws.count_nonzero()) == 0
    assert torch.equal(dX.cpu(), X)


@pytest.mark.parametrize("rows,cols,dtype", [(2048, 768, torch.bfloat16), (7, 8, torch.bfloat16), (300, 1000, torch.bfloat16),
                                             (129, 260, torch.float32), (2048, 3072, torch.float32)])
def test_layernorm_backward_matches_autograd_in_fp64(pkg, dev, rows, cols, dtype):
    g = torch.Generator().manual_seed(rows * 7 + cols)
    x = (torch.randn(rows, cols, generator=g) * 2 + 0.5).to(dtype)
    gamma = (torch.randn(cols, generator=g) * 0.5 + 1).to(dtype)
    dy = torch.randn(rows, cols, generator=g).to(dtype)
    xd = x.double().requires_grad_(True)
    gd = gamma.double().requires_grad_(True)
    bd = torch.zeros(cols, dtype=torch.float64, requires_grad=True)
    y = torch.nn.functional.layer_norm(xd, (cols,), gd, bd, 1e-5)
    y.backward(dy.double())
    mean = x.double().mean(1)
    rstd = 1.0 / torch.sqrt(x.double().var(1, unbiased=False) + 1e-5)
    ws = torch.zeros(pkg.layernorm_bwd_workspace_bytes(cols), dtype=torch.uint8, device=dev)
    args = [t.to(dev) for t in (dy, x, gamma, mean.float(), rstd.float())]
    tol = 2 ** -7 if dtype == torch.bfloat16 else 2e-5  # output rounding of bf16; fp32 sums against fp64
    for _ in range(2):  # the workspace is left clean for the second call
        dx = torch.full((rows, cols), 3.0, dtype=dtype, device=dev)
        dg = torch.full((cols,), 3.0, dtype=dtype, device=dev)
        db = torch.full((cols,), 3.0, dtype=dtype, device=dev)
        pkg.layernorm_bwd(*args, dx, dg, db, ws)
        torch.cuda.synchronize()
        assert rel_err(dx.double().cpu().numpy(), xd.grad.numpy()) < tol
        assert rel_err(dg.double().cpu().numpy(), gd.grad.numpy()) < tol
        assert rel_err(db.double().cpu().numpy(), bd.grad.numpy()) < tol
        assert int(ws.count_nonzero()) == 0


def test_peer_buffer_is_a_zeroed_torch_view_with_an_exportable_handle(pkg, dev):
    buf = pkg.PeerBuffer(1000, torch.bfloat16, dev)
    assert buf.tensor.dtype == torch.bfloat16 and buf.tensor.numel() == 1000 and buf.tensor.data_ptr() == buf.ptr.value
    assert float(buf.tensor.float().abs().sum()) == 0.0
    buf.tensor.fill_(1.5)
    assert float(buf.tensor.float().sum()) == 1500.0
    h = buf.handle()
    assert len(h) == 64 and any(h)
    del buf.tensor
    buf.close()
    buf.close()  # idempotent


def _peer_rank(rank, world, port, out):
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
    result = {}
    # (a) fp32 compute on the exact kernels, eager: against one rank on the whole batch
    cfg = hy.HybridConfig(vocab_size=50, block_size=32, n_embd=64, n_head=2, n_layer=2, compute_dtype=torch.float32)
    model = hy.HybridGPT(cfg, hy.CudaKernels(pkg), dev, seed=13, peer=True)
    step = hy.DataParallelStep(model, lr=1e-2, exchange="peer")
    idx, tgt = make_batch(17, 2 * world, 24, 50)
    lo, hi = 2 * rank, 2 * rank + 2
    losses = []
    for _ in range(5):
        loss, _ = step.step(idx[lo:hi].to(dev), tgt[lo:hi].to(dev))
        t = loss.clone()
        dist.all_reduce(t)
        losses.append(float(t) / world)
    result.update(losses=losses, param=step.gather_master().cpu(), work=model.flat_work.cpu())
    step.close()
    # (b) mixed precision with graph replay: the peer exchange against the NCCL all-reduce on the same batches
    cfg = hy.HybridConfig(vocab_size=50, block_size=32, n_embd=128, n_head=2, n_layer=2)
    curves, norms = {}, {}
    for mode in ("nccl", "peer"):
        model = hy.HybridGPT(cfg, hy.CudaKernels(pkg), dev, seed=5, peer=mode == "peer")
        step = hy.DataParallelStep(model, lr=1e-2, cuda_graph=True, exchange=mode)
        curves[mode], norms[mode] = [], []
        for i in range(7):
            idx, tgt = make_batch(100 + i, 2 * world, 24, 50)
            loss, nsq = step.step(idx[lo:hi].to(dev), tgt[lo:hi].to(dev))
            t = loss.clone()
            dist.all_reduce(t)
            curves[mode].append(float(t) / world)
            norms[mode].append(float(nsq))
        assert step.graph is not None
        if mode == "peer":
            # every rank reads the same parameter bits
            mine = model.flat_work.view(torch.int16).to(torch.int64)
            both = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(both, mine)
            result["same_bits"] = all(torch.equal(both[0], b) for b in both)
            step.close()
    pkg.sync_status()
    result.update(curves=curves, norms=norms)
    dist.barrier()
    if rank == 0:
        torch.save(result, out)
    dist.destroy_process_group()


def test_peer_exchange_ranks_follow_the_single_rank_loss_curve(pkg, dev, tmp_path):
    """Two ranks, one process per GPU, with the exchange + optimiser kernel over peer memory in place of the
    all-reduce: fp32 compute gives one rank's loss curve and parameters on the whole batch; in mixed precision
    with graph replay it follows the NCCL variant, and all ranks hold the same parameter bits."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = str(tmp_path / "peer.pt")
    mp.spawn(_peer_rank, args=(2, 29533, out), nprocs=2, join=True)
    got = torch.load(out)
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        hy = load_hybrid()
        cfg = hy.HybridConfig(vocab_size=50, block_size=32, n_embd=64, n_head=2, n_layer=2, compute_dtype=torch.float32)
        model = hy.HybridGPT(cfg, hy.CudaKernels(pkg), dev, seed=13)
        step = hy.DataParallelStep(model, lr=1e-2)
        idx, tgt = make_batch(17, 4, 24, 50)
        losses = [float(step.step(idx.to(dev), tgt.to(dev))[0]) for _ in range(5)]
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    assert np.allclose(got["losses"], losses, rtol=1e-5), (got["losses"], losses)
    assert rel_err(got["param"].numpy(), model.flat_param.cpu().numpy()) < 1e-4
    assert torch.equal(got["work"], got["param"])  # fp32 compute: the buffer the passes read IS the master
    assert got["same_bits"]
    assert np.allclose(got["curves"]["peer"], got["curves"]["nccl"], rtol=2e-2), got["curves"]
    assert np.allclose(got["norms"]["peer"], got["norms"]["nccl"], rtol=5e-2), got["norms"]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_peer_exchange_on_one_rank_equals_the_plain_step(pkg, dev, dtype):
    """world = 1: the exchange kernel reads and writes only this rank's buffers and must give the plain step.
    fp32 compute runs on the exact kernels, which are deterministic: the two variants agree to rounding of the
    optimiser arithmetic.  In bf16 the tensor-core backward sums dQ tiles in the order they arrive and AdamW
    turns a last-bit difference of a tiny gradient into a different step, so single parameters may differ by a
    step; the curves and the bulk of the parameters agree."""
    hy = load_hybrid()
    mixed = dtype == torch.bfloat16
    cfg = hy.HybridConfig(vocab_size=50, block_size=32, n_embd=128 if mixed else 64, n_head=2, n_layer=2, compute_dtype=dtype)
    batches = [tuple(t.to(dev) for t in make_batch(60 + i, 2, 24, 50)) for i in range(2 if mixed else 5)]
    curves, works = [], []
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        for mode in ("nccl", "peer"):
            model = hy.HybridGPT(cfg, hy.CudaKernels(pkg), dev, seed=8, peer=mode == "peer")
            step = hy.DataParallelStep(model, lr=1e-2, exchange=mode)
            curves.append([float(step.step(i, t)[0]) for i, t in batches])
            works.append(model.flat_work.float().cpu())
            master = step.gather_master()
            assert torch.equal(master.to(dtype), model.flat_work)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    torch.cuda.synchronize()
    if mixed:
        # after two steps of at most lr each, a parameter whose tiny gradient changed sign between the runs is
        # up to 4 lr apart; they must be few
        assert np.allclose(curves[0][:2], curves[1][:2], rtol=1e-3), curves
        delta = (works[0] - works[1]).abs()
        assert float(delta.max()) <= 4.2e-2, float(delta.max())
        assert float((delta > 2e-3).float().mean()) < 0.05, float((delta > 2e-3).float().mean())
    else:
        assert np.allclose(curves[0], curves[1], rtol=1e-6), curves
        assert rel_err(works[1].numpy(), works[0].numpy()) < 1e-5


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
