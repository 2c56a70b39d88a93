"""CPU tests of the data-parallel training step (cxx-gpt_b200/hybrid_gpt.py): the host logic around
the kernels — flat parameter/gradient buffers, gradient buckets, the all-reduce started from autograd
hooks, the mean + AdamW step — on `gloo` ranks, with the CPU oracle standing in for the attention
kernels and a plain restatement of the reference's AdamW for the optimiser kernel (test
infrastructure only; the product's kernel set refuses to run without a CUDA device)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def load_hybrid():
    import __graft_entry__ as g
    g.load_package()
    import importlib
    return importlib.import_module("cxx_gpt_b200.hybrid_gpt")


class OracleKernels:
    """The interface of hybrid_gpt.CudaKernels on CPU tensors, computed by the CPU oracle."""

    def __init__(self):
        import oracle
        self.orc = oracle.Oracle()
        self.orc.set_threads(1)

    def rope_cast(self, x, B, S, D, head_dim, sign, out_dtype):
        y = self.orc.rope(x.detach().float().numpy().copy(), S, head_dim, sign)
        return torch.from_numpy(np.ascontiguousarray(y)).to(out_dtype)

    def mha_fwd(self, q, k, v, B, S, H, Dh):
        o = self.orc.mha_fwd(q.numpy(), k.numpy(), v.numpy(), B, S, H, Dh)
        return torch.from_numpy(o), torch.zeros(1)

    def mha_bwd(self, q, k, v, o, do, lse, B, S, H, Dh):
        return tuple(torch.from_numpy(t) for t in
                     self.orc.mha_bwd(q.numpy(), k.numpy(), v.numpy(), o.numpy(), do.contiguous().numpy(), B, S, H, Dh))

    def lin_fwd(self, q, k, v, B, S, D, E):
        o, den, _ = self.orc.linattn_fwd(q.numpy(), k.numpy(), v.numpy(), B, S, D, E)
        return torch.from_numpy(o), torch.from_numpy(den)

    def lin_bwd(self, q, k, v, o, do, den, B, S, D, E):
        return tuple(torch.from_numpy(t) for t in
                     self.orc.kernel_attn_bwd(q.numpy(), k.numpy(), v.numpy(), o.numpy(), do.contiguous().numpy(),
                                              den.numpy(), B, S, D, E))

    def adamw(self, param, grad, m, v, step, lr, beta1, beta2, weight_decay, eps, grad_scale, norm_sq, param_copy=None):
        reference_adamw(param, grad.float(), m, v, step, lr, beta1, beta2, weight_decay, eps, grad_scale, norm_sq)
        if param_copy is not None:
            param_copy.copy_(param)


def reference_adamw(param, grad, m, v, step, lr, beta1, beta2, wd, eps, grad_scale, norm_sq):
    """The reference's optimiser step (src/GPT/gpt_cuda_kernels.cu:488-501 with the host factors of
    src/GPT/gpt_gpt.hpp:273-278) on the mean gradient, in torch."""
    g = grad * grad_scale
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    corr1, corr2 = 1 - beta1 ** step, 1 - beta2 ** step
    alpha, eps_hat = lr * corr2 ** 0.5 / corr1, eps * corr2 ** 0.5
    param.sub_(alpha * m / (v.sqrt() + eps_hat) + lr * wd * param)
    if norm_sq is not None:
        norm_sq.add_((g * g).sum())


def small_config(hy):
    return hy.HybridConfig(vocab_size=50, block_size=16, n_embd=16, n_head=2, n_layer=2, compute_dtype=torch.float32)


def make_batch(seed, B, S, vocab):
    g = torch.Generator().manual_seed(seed)
    idx = torch.randint(0, vocab, (B, S), generator=g)
    tgt = torch.randint(0, vocab, (B, S), generator=g)
    return idx, tgt


def test_parameter_layout_and_count():
    hy = load_hybrid()
    full = hy.HybridConfig()
    table = hy.parameter_table(full)
    n = sum(int(np.prod(s)) for _, s, _ in table)
    E, V = 768, 6400
    per_block = 2 * 2 * E + 3 * (E * E + E) + 3 * E * E + (E * E + E) + (4 * E * E + 4 * E) + (4 * E * E + E)
    assert n == V * E + 256 * E + 12 * per_block + 2 * E == 111_401_472
    model = hy.HybridGPT(small_config(hy), OracleKernels(), torch.device("cpu"))
    for name, (off, cnt, shape) in model.offsets.items():
        assert off % 8 == 0 and model.p[name].data_ptr() == model.flat_param.data_ptr() + 4 * off
        assert model.p[name].grad.data_ptr() == model.flat_grad.data_ptr() + 4 * off
    # buckets partition the buffer at parameter borders
    st = hy.DataParallelStep(model, n_buckets=3)
    assert st.buckets[0]["lo"] == 0 and st.buckets[-1]["hi"] == model.numel
    assert all(a["hi"] == b["lo"] for a, b in zip(st.buckets, st.buckets[1:]))
    assert sum(b["params"] for b in st.buckets) == len(model.order)


def test_model_gradients_match_finite_differences():
    """The autograd wiring of the two attention stages and the rotary/conversion pass: directional
    derivative of the loss along a random direction against central differences (fp32, oracle kernels)."""
    hy = load_hybrid()
    model = hy.HybridGPT(small_config(hy), OracleKernels(), torch.device("cpu"), seed=1)
    idx, tgt = make_batch(2, 2, 8, 50)
    model.flat_grad.zero_()
    model.loss(idx, tgt).backward()
    g = model.flat_grad.clone()
    d = torch.randn(model.numel, generator=torch.Generator().manual_seed(3))
    d /= d.norm()
    eps = 1e-2
    with torch.no_grad():
        base = model.flat_param.clone()
        model.flat_param.copy_(base + eps * d)
        lp = float(model.loss(idx, tgt))
        model.flat_param.copy_(base - eps * d)
        lm = float(model.loss(idx, tgt))
        model.flat_param.copy_(base)
    fd, an = (lp - lm) / (2 * eps), float(g @ d)
    assert abs(fd - an) < 2e-2 * max(abs(an), 1e-3) + 2e-4, (fd, an)


def _rank_main(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    hy = load_hybrid()
    model = hy.HybridGPT(small_config(hy), OracleKernels(), torch.device("cpu"), seed=5)  # same weights on every rank
    step = hy.DataParallelStep(model, lr=1e-2, n_buckets=3)
    idx, tgt = make_batch(11, 4, 8, 50)  # the global batch; each rank takes its half
    lo, hi = rank * 2, rank * 2 + 2
    losses = []
    for _ in range(2):
        loss, nsq = step.step(idx[lo:hi], tgt[lo:hi])
        losses.append(float(loss))
    if rank == 0:
        torch.save({"param": model.flat_param.clone(), "grad": model.flat_grad.clone(), "nsq": float(nsq),
                    "losses": losses}, out)
    dist.destroy_process_group()


def test_two_ranks_reproduce_the_single_rank_step_on_the_whole_batch(tmp_path):
    """Two gloo ranks, half the batch each: after the bucketed all-reduce the gradient buffer holds
    the SUM of the ranks' gradients, whose mean is the single-rank gradient on the whole batch, and
    two optimiser steps leave the same parameters (same weights on every rank, no data-path collective
    other than the gradient all-reduce)."""
    out = str(tmp_path / "rank0.pt")
    mp.spawn(_rank_main, args=(2, 29517, out), nprocs=2, join=True)
    got = torch.load(out)
    hy = load_hybrid()
    model = hy.HybridGPT(small_config(hy), OracleKernels(), torch.device("cpu"), seed=5)
    step = hy.DataParallelStep(model, lr=1e-2, n_buckets=3)
    idx, tgt = make_batch(11, 4, 8, 50)
    for _ in range(2):
        loss, nsq = step.step(idx, tgt)
    # the ranks' buffer holds the sum over 2 ranks of half-batch gradients = 2 x the whole-batch gradient
    assert torch.allclose(got["grad"] / 2, model.flat_grad, rtol=1e-4, atol=1e-6)
    assert torch.allclose(got["param"], model.flat_param, rtol=1e-4, atol=1e-6)
    assert abs(got["nsq"] - float(nsq)) < 1e-4 * float(nsq)


def test_product_kernel_set_refuses_to_run_without_a_device():
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    hy = load_hybrid()
    with pytest.raises(RuntimeError):
        hy.CudaKernels(None)
