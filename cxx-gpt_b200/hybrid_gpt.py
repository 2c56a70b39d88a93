"""The data-parallel training step around the attention kernels (full-model configuration of the
baseline: vocab 6400, block 256, n_embd 768, 12 heads x 64, 12 pre-LN blocks, batch 8 per GPU,
AdamW lr 1e-3).

No single reference file implements this model; it is the reference's GPT skeleton
(src/GPT/gpt_gpt.hpp:333-399 block, :480-511 model: token + position embedding, pre-LN blocks with
residuals, GELU MLP, final LayerNorm) whose attention is TwoStageGPT's pair of stages
(src/TwoStage/two_stage_gpt.hpp:101-122 forward, :149-174 backward): q/k/v projections -> rotary
embedding per head -> fused causal softmax MHA -> lq/lk/lv projections (bias-free) -> rotary
embedding over the whole width -> ELU+1 linear attention with ONE head of width n_embd -> output
projection; and TwoStageGPT's weight-tied lm_head (two_stage_gpt.hpp:272-276, 304-313).  With these
layers the model has 111.4 M parameters (111,401,472) at the full size (the baseline's "~95 M" is the plain GPT).

What runs where:
  * the two attention stages, the rotary embedding fused with the type conversion, and the
    optimiser step are this library's kernels, called through its C-ABI (`CudaKernels`);
  * the dense glue (linear layers, LayerNorm, GELU, embedding, cross-entropy) is plain torch, i.e.
    cuBLAS and library kernels: it is outside the attention path and is not tuned here;
  * gradients live in ONE flat buffer (fp32, or bf16 in mixed precision) that the autograd engine accumulates into in place; after
    the backward pass of a bucket of it, `torch.distributed.all_reduce` (NCCL, sum) is started on
    that bucket while the rest of the backward pass runs; the kernel after the collective,
    cxxattn_adamw_step, turns the sum into the mean, applies AdamW as the reference's optimiser
    does (src/GPT/gpt_cuda_kernels.cu:488-501) and accumulates the gradient norm, in one pass;
  * or (`exchange="peer"`, one process per GPU of one machine) exchange and optimiser are ONE kernel over
    peer memory, cxxattn_adamw_step_exchange: every rank owns a contiguous shard of the flat buffers,
    reads all ranks' gradients of it over NVLink, keeps master parameters and moments for the shard only
    and writes the updated parameters into every rank's buffer; two one-element all-reduces order it
    against the backward pass before and the forward pass after.

There is no CPU path in the product: `CudaKernels` refuses to run without a CUDA device.  The model
code takes the kernel set as an argument so that the multi-rank host logic (bucketing, the
all-reduce, the step) can be tested on CPU ranks with a stand-in that the tests supply.
"""
import math

import torch
import torch.distributed as dist
import torch.nn.functional as F


class HybridConfig:
    def __init__(self, vocab_size=6400, block_size=256, n_embd=768, n_head=12, n_layer=12, ln_eps=1e-5,
                 compute_dtype=torch.bfloat16):
        assert n_embd % n_head == 0
        self.vocab_size, self.block_size, self.n_embd = vocab_size, block_size, n_embd
        self.n_head, self.n_layer, self.ln_eps = n_head, n_layer, ln_eps
        self.head_dim = n_embd // n_head
        self.compute_dtype = compute_dtype


class CudaKernels:
    """The library's kernels behind the interface the model uses.  Tensors are CUDA tensors; outputs
    are allocated with torch (plumbing), everything else happens inside libcxxattn.so."""

    def __init__(self, pkg):
        if not torch.cuda.is_available():
            raise RuntimeError("the training step needs a CUDA device: there is no CPU path in the product")
        self.pkg = pkg
        self.colsum_ws = {}  # per device: the zeroed workspace of cxxattn_colsum (it leaves it zeroed)
        self.ln_ws = {}      # the same for cxxattn_layernorm_bwd

    COLSUM_MAX_COLS = 1 << 16

    def colsum(self, x, out):
        """out[c] = sum of column c of the 2-D bf16 tensor x; False if the shape is not covered."""
        if x.dtype != torch.bfloat16 or x.shape[1] % 8 or x.shape[1] > self.COLSUM_MAX_COLS or not x.is_contiguous():
            return False
        ws = self.colsum_ws.get(x.device)
        if ws is None:
            ws = torch.zeros(self.pkg.colsum_workspace_bytes(self.COLSUM_MAX_COLS), dtype=torch.uint8, device=x.device)
            self.colsum_ws[x.device] = ws
        self.pkg.colsum(x, out, ws)
        return True

    def rope_cast(self, x, B, S, D, head_dim, sign, out_dtype):
        out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
        self.pkg.rope_cast(x.contiguous(), out, B, S, D, head_dim, sign)
        return out

    def rope_cast_pair(self, x0, x1, B, S, D, head_dim, sign, out_dtype):
        y0 = torch.empty(x0.shape, dtype=out_dtype, device=x0.device)
        y1 = torch.empty(x1.shape, dtype=out_dtype, device=x1.device)
        self.pkg.rope_cast_pair(x0.contiguous(), x1.contiguous(), y0, y1, B, S, D, head_dim, sign)
        return y0, y1

    def mha_fwd(self, q, k, v, B, S, H, Dh):
        o = torch.empty_like(q)
        lse = torch.empty(B * H * S, dtype=torch.float32, device=q.device)
        self.pkg.mha_fwd(q, k, v, o, B, S, H, Dh, lse=lse)
        return o, lse

    def mha_bwd(self, q, k, v, o, do, lse, B, S, H, Dh):
        dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
        self.pkg.mha_bwd(q, k, v, o, do.contiguous(), dq, dk, dv, B, S, H, Dh, lse=lse)
        return dq, dk, dv

    def lin_fwd(self, q, k, v, B, S, D, E):
        o = torch.empty_like(v)
        den = torch.empty(B * S, dtype=torch.float32, device=q.device)
        self.pkg.linattn_fwd(q, k, v, o, den, None, B, S, D, E, self.pkg.MAP_ELU1, 0)
        return o, den

    def lin_bwd(self, q, k, v, o, do, den, B, S, D, E):
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        self.pkg.linattn_bwd(q, k, v, o, do.contiguous(), den, dq, dk, dv, B, S, D, E, self.pkg.MAP_ELU1, 0)
        return dq, dk, dv

    def adamw(self, param, grad, m, v, step, lr, beta1, beta2, weight_decay, eps, grad_scale, norm_sq, param_copy=None):
        self.pkg.adamw_step(param, grad, m, v, step, lr, beta1, beta2, weight_decay, eps, grad_scale, norm_sq,
                            param_copy=param_copy)

    def layernorm_bwd(self, dy, x, gamma, mean, rstd, dgamma, dbeta):
        """dx of a LayerNorm over the rows of the 2-D bf16 tensor x; dgamma and dbeta are written in place.
        None if the shape is not covered."""
        if x.dtype != torch.bfloat16 or x.shape[1] % 8 or x.shape[1] > self.COLSUM_MAX_COLS:
            return None
        ws = self.ln_ws.get(x.device)
        if ws is None:
            ws = torch.zeros(self.pkg.layernorm_bwd_workspace_bytes(self.COLSUM_MAX_COLS), dtype=torch.uint8, device=x.device)
            self.ln_ws[x.device] = ws
        dx = torch.empty_like(x)
        self.pkg.layernorm_bwd(dy.contiguous(), x, gamma, mean, rstd, dx, dgamma, dbeta, ws)
        return dx

    def peer_buffer(self, numel, dtype, device):
        """A zeroed flat buffer that the other ranks' GPUs can map."""
        return self.pkg.PeerBuffer(numel, dtype, device)

    def open_peer(self, handle, numel, dtype, device):
        return self.pkg.PeerBuffer.open(handle, numel, dtype, device)

    def adamw_exchange(self, param_shard, m_shard, v_shard, grad_ptrs, param_ptrs, dtype, rank, lo, step, lr, beta1,
                       beta2, weight_decay, eps, grad_scale, norm_sq):
        self.pkg.adamw_step_exchange(param_shard, m_shard, v_shard, grad_ptrs, param_ptrs, dtype, rank, lo, step, lr,
                                     beta1, beta2, weight_decay, eps, grad_scale, norm_sq)


class _RopeCast(torch.autograd.Function):
    """y = rope(x) in `out_dtype` (two_stage_cuda::rope_fwd + the conversion the next kernel wants);
    backward = rope with the opposite sign back to x's type (rope_bwd, two_stage_gpt.hpp:160,174)."""

    @staticmethod
    def forward(ctx, x, kernels, B, S, D, head_dim, out_dtype):
        ctx.kernels, ctx.dims, ctx.in_dtype = kernels, (B, S, D, head_dim), x.dtype
        return kernels.rope_cast(x, B, S, D, head_dim, 1.0, out_dtype)

    @staticmethod
    def backward(ctx, g):
        B, S, D, hd = ctx.dims
        return ctx.kernels.rope_cast(g, B, S, D, hd, -1.0, ctx.in_dtype), None, None, None, None, None, None


class _RopeCastPair(torch.autograd.Function):
    """_RopeCast on the query and the key tensor in one launch each way (rope_fwd / rope_bwd take both)."""

    @staticmethod
    def forward(ctx, x0, x1, kernels, B, S, D, head_dim, out_dtype):
        ctx.kernels, ctx.dims, ctx.in_dtype = kernels, (B, S, D, head_dim), x0.dtype
        return kernels.rope_cast_pair(x0, x1, B, S, D, head_dim, 1.0, out_dtype)

    @staticmethod
    def backward(ctx, g0, g1):
        B, S, D, hd = ctx.dims
        d0, d1 = ctx.kernels.rope_cast_pair(g0, g1, B, S, D, hd, -1.0, ctx.in_dtype)
        return d0, d1, None, None, None, None, None, None


def _rope_pair(x0, x1, kernels, B, S, D, head_dim, out_dtype):
    if hasattr(kernels, "rope_cast_pair") and x0.dtype == x1.dtype:
        return _RopeCastPair.apply(x0, x1, kernels, B, S, D, head_dim, out_dtype)
    return (_RopeCast.apply(x0, kernels, B, S, D, head_dim, out_dtype),
            _RopeCast.apply(x1, kernels, B, S, D, head_dim, out_dtype))


class _SoftmaxStage(torch.autograd.Function):
    """Stage 1: fused causal softmax MHA (fused_mha_fwd / fused_mha_bwd, two_stage_gpt.hpp:106,171)."""

    @staticmethod
    def forward(ctx, q, k, v, kernels, B, S, H, Dh):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        o, lse = kernels.mha_fwd(q, k, v, B, S, H, Dh)
        ctx.kernels, ctx.dims = kernels, (B, S, H, Dh)
        ctx.save_for_backward(q, k, v, o, lse)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = ctx.kernels.mha_bwd(q, k, v, o, do, lse, *ctx.dims)
        return dq, dk, dv, None, None, None, None, None


class _LinearStage(torch.autograd.Function):
    """Stage 2: ELU+1 causal linear attention, one head of width D = E (kernel_attn_fwd and the
    step1 / dQ / dKdV backward, two_stage_gpt.hpp:121,149-156)."""

    @staticmethod
    def forward(ctx, q, k, v, kernels, B, S, D, E):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        o, den = kernels.lin_fwd(q, k, v, B, S, D, E)
        ctx.kernels, ctx.dims = kernels, (B, S, D, E)
        ctx.save_for_backward(q, k, v, o, den)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, den = ctx.saved_tensors
        dq, dk, dv = ctx.kernels.lin_bwd(q, k, v, o, do, den, *ctx.dims)
        return dq, dk, dv, None, None, None, None, None


class _Linear(torch.autograd.Function):
    """y = x W^T (+ b) whose backward pass writes dW and db straight into the parameters' views of the flat
    gradient buffer.  Left to the autograd engine, each would be produced in a temporary and then added into
    its view by one more launch per parameter (some 220 launches of a few microseconds per step)."""

    @staticmethod
    def forward(ctx, x, w, b, model, name):
        ctx.save_for_backward(x, w)
        ctx.model, ctx.name, ctx.has_bias = model, name, b is not None
        return F.linear(x, w, b)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        model, name = ctx.model, ctx.name
        dy = dy.contiguous()
        dx = dy @ w
        torch.mm(dy.t(), x, out=model.p[name + ".w"].grad)
        model.grad_ready(name + ".w")
        if ctx.has_bias:
            gb = model.p[name + ".b"].grad
            colsum = getattr(model.kernels, "colsum", None)
            # bf16: one pass of the library's column-sum kernel; fp32 stays on torch's deterministic reduction
            if colsum is None or not colsum(dy, gb):
                torch.sum(dy, 0, out=gb)
            model.grad_ready(name + ".b")
        return dx, None, None, None, None


class _LayerNorm(torch.autograd.Function):
    """LayerNorm over the rows of a 2-D bf16 tensor: torch's forward kernel (which returns the row statistics),
    the library's backward (cxxattn_layernorm_bwd: two launches, dgamma and dbeta written straight into their views
    of the flat gradient buffer)."""

    @staticmethod
    def forward(ctx, x, g, b, model, name):
        y, mean, rstd = torch.native_layer_norm(x, (x.shape[1],), g, b, model.cfg.ln_eps)
        ctx.save_for_backward(x, g, mean.reshape(-1).float(), rstd.reshape(-1).float())
        ctx.model, ctx.name = model, name
        return y

    @staticmethod
    def backward(ctx, dy):
        x, g, mean, rstd = ctx.saved_tensors
        model, name = ctx.model, ctx.name
        dx = model.kernels.layernorm_bwd(dy, x, g, mean, rstd, model.p[name + ".g"].grad, model.p[name + ".b"].grad)
        model.grad_ready(name + ".g")
        model.grad_ready(name + ".b")
        return dx, None, None, None, None


def parameter_table(cfg):
    """(name, shape, init std or None for ones / 0.0 for zeros) in the order the forward pass uses them,
    which is the reverse of the order in which the backward pass finishes their gradients."""
    E, V = cfg.n_embd, cfg.vocab_size
    t = [("wte", (V, E), 0.02), ("wpe", (cfg.block_size, E), 0.02)]
    for i in range(cfg.n_layer):
        p = f"h{i}."
        t += [(p + "ln_1.g", (E,), None), (p + "ln_1.b", (E,), 0.0)]
        for n in ("attn_q", "attn_k", "attn_v"):
            t += [(p + n + ".w", (E, E), 0.02), (p + n + ".b", (E,), 0.0)]
        for n in ("lq_proj", "lk_proj", "lv_proj"):
            t += [(p + n + ".w", (E, E), 0.02)]
        t += [(p + "attn_proj.w", (E, E), 0.02), (p + "attn_proj.b", (E,), 0.0),
              (p + "ln_2.g", (E,), None), (p + "ln_2.b", (E,), 0.0),
              (p + "mlp_fc.w", (4 * E, E), 0.02), (p + "mlp_fc.b", (4 * E,), 0.0),
              (p + "mlp_proj.w", (E, 4 * E), 0.02), (p + "mlp_proj.b", (E,), 0.0)]
    t += [("ln_f.g", (E,), None), ("ln_f.b", (E,), 0.0)]
    return t


class HybridGPT:
    """Parameters, gradients and AdamW moments in flat buffers; `p[name]` are views.

    fp32 compute: the leaves of the autograd graph are views of the fp32 parameter buffer and their gradients
    views of an fp32 gradient buffer.  bf16 compute (mixed precision): the fp32 buffer is the optimiser's
    master copy; the leaves are views of a bf16 working copy that the optimiser kernel rewrites in the pass
    that updates the master, and the gradient buffer is bf16 too (half the bytes through the all-reduce, no
    per-layer conversions in either pass).  `peer`: the buffer the passes read and the gradient buffer are
    allocated so that the other ranks' GPUs can map them (DataParallelStep with exchange="peer")."""

    def __init__(self, cfg, kernels, device, seed=0, peer=False):
        self.cfg, self.kernels, self.device = cfg, kernels, device
        table = parameter_table(cfg)
        self.offsets, off = {}, 0
        for name, shape, _ in table:
            n = math.prod(shape)
            self.offsets[name] = (off, n, shape)
            off += (n + 7) // 8 * 8  # every view starts on a 16-byte boundary, in bf16 too
        self.numel = off
        self.mixed = cfg.compute_dtype == torch.bfloat16
        work_dtype = torch.bfloat16 if self.mixed else torch.float32
        self.peer = None
        if peer:
            self.peer = {"work": kernels.peer_buffer(off, work_dtype, device),
                         "grad": kernels.peer_buffer(off, work_dtype, device)}
        self.flat_param = self.peer["work"].tensor if peer and not self.mixed else \
            torch.zeros(off, dtype=torch.float32, device=device)
        g = torch.Generator(device="cpu").manual_seed(seed)
        for name, shape, std in table:
            o, n, _ = self.offsets[name]
            view = self.flat_param[o:o + n].view(shape)
            if std is None:
                view.fill_(1.0)
            elif std > 0:
                view.copy_((torch.randn(shape, generator=g) * std).to(device))
        if not self.mixed:
            self.flat_work = self.flat_param
        elif peer:
            self.flat_work = self.peer["work"].tensor
            self.flat_work.copy_(self.flat_param)
        else:
            self.flat_work = self.flat_param.to(torch.bfloat16)
        self.flat_grad = self.peer["grad"].tensor if peer else torch.zeros_like(self.flat_work)
        self.p = {}
        for name, shape, _ in table:
            o, n, _ = self.offsets[name]
            view = self.flat_work[o:o + n].view(shape)
            view.requires_grad_(True)
            view.grad = self.flat_grad[o:o + n].view(shape)  # autograd accumulates into the flat buffer in place
            self.p[name] = view
        self.order = [name for name, _, _ in table]
        # parameters whose gradient the backward pass of `_Linear` writes in place
        self.direct_grad = {name for name in self.order
                            if name.startswith("h") and name.split(".")[1] in
                            ("attn_q", "attn_k", "attn_v", "lq_proj", "lk_proj", "lv_proj", "attn_proj", "mlp_fc", "mlp_proj")}
        # bf16 compute on the library's kernels: LayerNorm backward is the library's too, and writes dgamma, dbeta itself
        self.custom_ln = self.mixed and hasattr(kernels, "layernorm_bwd") and cfg.n_embd % 8 == 0
        if self.custom_ln:
            self.direct_grad |= {name for name in self.order if ".ln_" in "." + name}
        self.on_grad_ready = None

    def _linear(self, x, name, bias=True):
        return _Linear.apply(x, self.p[name + ".w"], self.p[name + ".b"] if bias else None, self, name)

    def grad_ready(self, name):
        """Called by backward passes that write a parameter's gradient themselves (`direct_grad`): the autograd
        engine's post-accumulate hooks do not fire for those."""
        if self.on_grad_ready is not None:
            self.on_grad_ready(name)

    def _ln(self, x, name):
        E = self.cfg.n_embd
        g, b = self.p[name + ".g"], self.p[name + ".b"]
        if self.custom_ln:
            return _LayerNorm.apply(x, g, b, self, name)
        if x.dtype == g.dtype:  # one kernel each way; statistics are accumulated in fp32 inside it
            return F.layer_norm(x, (E,), g, b, self.cfg.ln_eps)
        return F.layer_norm(x.float(), (E,), g.float(), b.float(), self.cfg.ln_eps).to(x.dtype)

    def loss(self, idx, targets):
        """Mean next-token cross-entropy of logits = model(idx); idx, targets [B, S] int64."""
        cfg, K = self.cfg, self.kernels
        B, S = idx.shape
        E, H, Dh, dt = cfg.n_embd, cfg.n_head, cfg.head_dim, cfg.compute_dtype
        pos = torch.arange(S, device=idx.device)
        h = (F.embedding(idx, self.p["wte"]) + F.embedding(pos, self.p["wpe"])[None]).reshape(B * S, E).to(dt)
        for i in range(cfg.n_layer):
            p = f"h{i}."
            a = self._ln(h, p + "ln_1")
            q, k, v = (self._linear(a, p + n) for n in ("attn_q", "attn_k", "attn_v"))
            q, k = _rope_pair(q, k, K, B, S, E, Dh, dt)
            ra = _SoftmaxStage.apply(q, k, v, K, B, S, H, Dh)
            lq, lk, lv = (self._linear(ra, p + n, bias=False) for n in ("lq_proj", "lk_proj", "lv_proj"))
            # stage 2, one head of width n_embd: the tensor-core kernels in bf16 when the width is a multiple
            # of 64, the exact fp32 kernels otherwise
            dt2 = dt if (dt == torch.bfloat16 and E % 64 == 0) else torch.float32
            lq, lk = _rope_pair(lq, lk, K, B, S, E, E, dt2)
            ac = _LinearStage.apply(lq, lk, lv.to(dt2), K, B, S, E, E).to(dt)
            h = h + self._linear(ac, p + "attn_proj")
            m = self._linear(F.gelu(self._linear(self._ln(h, p + "ln_2"), p + "mlp_fc")), p + "mlp_proj")
            h = h + m
        h = self._ln(h, "ln_f")
        logits = F.linear(h, self.p["wte"].to(dt))  # weight-tied lm_head
        return F.cross_entropy(logits.float(), targets.reshape(-1))


class DataParallelStep:
    """One optimiser step per call: forward, backward with the bucketed gradient all-reduce started from
    autograd hooks, then the fused mean + AdamW + gradient-norm kernel.  `group` None = the default
    process group when torch.distributed is initialised, else a single rank.

    exchange="nccl": as above.  exchange="peer" (the model built with peer=True; all ranks on one machine):
    no all-reduce of gradients; after the backward pass a one-element all-reduce tells every rank that all
    gradients are final, cxxattn_adamw_step_exchange updates this rank's shard from all ranks' gradients and
    writes it into all ranks' parameter buffers, and the all-reduce of the partial squared norms tells every
    rank that its parameters are complete.  Master parameters and moments exist for the shard only
    (`gather_master()` collects the fp32 master of all shards)."""

    def __init__(self, model, lr=1e-3, beta1=0.9, beta2=0.999, weight_decay=0.01, eps=1e-8, n_buckets=4, group=None,
                 cuda_graph=False, exchange="nccl"):
        assert exchange in ("nccl", "peer")
        self.model, self.group, self.exchange = model, group, exchange
        # cuda_graph: after three eager steps, forward + backward (+ the all-reduces) of a fixed batch
        # shape are captured once and replayed; the step is a few thousand short launches, and issuing
        # them from Python costs more time than the GPU needs to run them
        self.cuda_graph, self.graph, self.eager_steps = cuda_graph, None, 0
        self.hp = (lr, beta1, beta2, weight_decay, eps)
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.norm_sq = torch.zeros(1, dtype=torch.float32, device=model.device)
        self.t = 0
        if exchange == "peer":
            self._setup_peers()
        else:
            self.m = torch.zeros_like(model.flat_param)
            self.v = torch.zeros_like(model.flat_param)
        # Buckets are contiguous ranges of the flat buffer, cut at parameter borders into roughly equal
        # parts.  The backward pass finishes gradients from the end of the buffer towards its start, so
        # the last bucket is ready first.
        names = model.order
        target = model.numel / max(1, n_buckets)
        self.buckets, lo, count = [], 0, 0
        for j, name in enumerate(names):
            o, n, _ = model.offsets[name]
            count += 1
            end = (o + n + 7) // 8 * 8
            if end - lo >= target or j == len(names) - 1:
                self.buckets.append({"lo": lo, "hi": end, "params": count, "ready": 0})
                lo, count = end, 0
        self.bucket_of = {}
        for b in self.buckets:
            for name in names:
                o, _, _ = model.offsets[name]
                if b["lo"] <= o < b["hi"]:
                    self.bucket_of[name] = b
        self.pending = []
        # Eager steps start each bucket's all-reduce from an autograd hook, as soon as the backward pass
        # has finished the bucket.  With CUDA-graph replay the collectives stay outside the graph (a
        # captured NCCL call did not complete on this platform): the buckets are reduced after the
        # replay, last bucket first, and the optimiser kernel follows.
        self.reduce_in_hooks = self.world > 1 and not cuda_graph and exchange == "nccl"
        if self.reduce_in_hooks:
            hooks = {name: self._make_hook(name) for name in names}
            for name in names:
                if name not in model.direct_grad:
                    model.p[name].register_post_accumulate_grad_hook(hooks[name])
            model.on_grad_ready = lambda name: hooks[name](None)

    def _setup_peers(self):
        """Shard bounds, shard-sized moments, and the addresses of every rank's gradient and parameter
        buffers as this rank's GPU sees them (CUDA IPC handles exchanged once through the process group)."""
        model, world, rank = self.model, self.world, self.rank
        if model.peer is None:
            raise ValueError('exchange="peer" needs a model built with peer=True')
        from .sharding import parameter_shard
        self.lo, self.hi, self.shard_len = parameter_shard(model.numel, world, rank)  # numel is a multiple of 8
        n = self.hi - self.lo
        # the fp32 master of the shard: a view of the parameter buffer in fp32 compute (which the exchange
        # kernel then also fills for the other shards), a buffer of its own in mixed precision
        self.master = model.flat_param[self.lo:self.hi] if not model.mixed else model.flat_param[self.lo:self.hi].clone()
        self.m = torch.zeros(n, dtype=torch.float32, device=model.device)
        self.v = torch.zeros(n, dtype=torch.float32, device=model.device)
        self.sync = torch.zeros(1, dtype=torch.float32, device=model.device)
        mine = (model.peer["work"].handle(), model.peer["grad"].handle())
        handles = [mine]
        if world > 1:
            handles = [None] * world
            dist.all_gather_object(handles, mine, group=self.group)
        dtype = model.flat_work.dtype
        self.opened, self.param_ptrs, self.grad_ptrs = [], [], []
        for r in range(world):
            if r == rank:
                self.param_ptrs.append(model.peer["work"].ptr.value)
                self.grad_ptrs.append(model.peer["grad"].ptr.value)
            else:
                w = model.kernels.open_peer(handles[r][0], model.numel, dtype, model.device)
                g = model.kernels.open_peer(handles[r][1], model.numel, dtype, model.device)
                self.opened += [w, g]
                self.param_ptrs.append(w.ptr.value)
                self.grad_ptrs.append(g.ptr.value)

    def close(self):
        """Unmaps the other ranks' buffers (collective in spirit: call it on every rank before the buffers go)."""
        for b in getattr(self, "opened", []):
            b.close()
        self.opened = []

    def gather_master(self):
        """The fp32 master parameters of all shards as one flat tensor (every rank gets all of it)."""
        model = self.model
        if self.exchange != "peer":
            return model.flat_param.clone()
        mine = torch.zeros(self.shard_len, dtype=torch.float32, device=model.device)
        mine[:self.hi - self.lo] = self.master
        if self.world == 1:
            return mine[:model.numel].clone()
        out = torch.empty(self.shard_len * self.world, dtype=torch.float32, device=model.device)
        dist.all_gather_into_tensor(out, mine, group=self.group)
        return out[:model.numel].clone()

    def _make_hook(self, name):
        b = self.bucket_of[name]

        def hook(_param):
            b["ready"] += 1
            if b["ready"] == b["params"]:  # the whole bucket is final: reduce it while backward goes on
                b["ready"] = 0
                self.pending.append(dist.all_reduce(self.model.flat_grad[b["lo"]:b["hi"]], op=dist.ReduceOp.SUM,
                                                    group=self.group, async_op=True))
        return hook

    def _forward_backward(self, idx, targets):
        model = self.model
        model.flat_grad.zero_()
        loss = model.loss(idx, targets)
        loss.backward()
        for w in self.pending:
            w.wait()
        self.pending.clear()
        return loss.detach()

    def _capture(self, idx, targets):
        self.static_idx, self.static_tgt = idx.clone(), targets.clone()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.static_loss = self._forward_backward(self.static_idx, self.static_tgt)
        self.graph = graph

    def step(self, idx, targets):
        """Returns (loss of this rank's batch, squared norm of the mean gradient), both device tensors."""
        model = self.model
        if self.graph is not None:
            self.static_idx.copy_(idx, non_blocking=True)
            self.static_tgt.copy_(targets, non_blocking=True)
            self.graph.replay()
            loss = self.static_loss
        else:
            loss = self._forward_backward(idx, targets)
            self.eager_steps += 1
            if self.cuda_graph and self.eager_steps == 3:
                self._capture(idx, targets)  # the captured pass only records; this step's gradients stand
        self.t += 1
        self.norm_sq.zero_()
        lr, b1, b2, wd, eps = self.hp
        if self.exchange == "peer":
            with torch.no_grad():
                if self.world > 1:
                    dist.all_reduce(self.sync, group=self.group)  # every rank's gradients are final
                model.kernels.adamw_exchange(self.master, self.m, self.v, self.grad_ptrs, self.param_ptrs,
                                             model.flat_work.dtype, self.rank, self.lo, self.t, lr, b1, b2, wd, eps,
                                             1.0 / self.world, self.norm_sq)
                if self.world > 1:  # the shards' shares of the norm; and: every rank's parameters are complete
                    dist.all_reduce(self.norm_sq, group=self.group)
            return loss, self.norm_sq
        if self.world > 1 and not self.reduce_in_hooks:
            works = [dist.all_reduce(model.flat_grad[b["lo"]:b["hi"]], op=dist.ReduceOp.SUM, group=self.group,
                                     async_op=True) for b in reversed(self.buckets)]
            for w in works:
                w.wait()
        with torch.no_grad():
            model.kernels.adamw(model.flat_param, model.flat_grad, self.m, self.v, self.t, lr, b1, b2, wd, eps,
                                1.0 / self.world, self.norm_sq, model.flat_work if model.mixed else None)
        return loss, self.norm_sq
