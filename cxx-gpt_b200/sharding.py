"""Host-side sharding of the attention work over ranks.

Both attention families are independent per (batch, head) unit (softmax: one unit per
(b, h), reference grid index `bh`, two_stage_cuda_kernels.cu:58-59; linear: one unit per folded
batch item, :899), so a job is split by giving each rank a contiguous range of units and nothing
is exchanged between ranks.  A range that cuts through a batch item is expressed as slabs
(b, h0, h1): heads h0..h1-1 of batch item b, which the kernels address in place through the
element strides of the descriptor.
"""


def unit_range(n_units, world, rank):
    """Contiguous, balanced split: the first n_units % world ranks get one unit more."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad world/rank")
    base, extra = divmod(n_units, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def slabs(B, H, world, rank):
    """The (b, h0, h1) slabs that make up this rank's share of the B*H units."""
    lo, hi = unit_range(B * H, world, rank)
    out = []
    u = lo
    while u < hi:
        b, h0 = divmod(u, H)
        h1 = min(H, h0 + (hi - u))
        out.append((b, h0, h1))
        u += h1 - h0
    return out


def calls(B, H, world, rank):
    """This rank's share as kernel calls (b0, nb, h0, nh): batch items b0..b0+nb-1, heads h0..h0+nh-1
    of each.  Consecutive slabs that cover whole batch items merge into one call; a partial slab is a
    call of its own, addressed in place through the descriptor's strides (stride_b = S*H*Dh,
    stride_s = H*Dh, stride_h = Dh of the unsplit tensor, base pointer moved by h0*Dh elements)."""
    out = []
    for b, h0, h1 in slabs(B, H, world, rank):
        whole = h0 == 0 and h1 == H
        if whole and out and out[-1][2] == 0 and out[-1][3] == H and out[-1][0] + out[-1][1] == b:
            out[-1] = (out[-1][0], out[-1][1] + 1, 0, H)
        else:
            out.append((b, 1, h0, h1 - h0))
    return out


def parameter_shard(numel, world, rank, vector=8):
    """The range [lo, hi) of a flat parameter buffer of `numel` elements (a multiple of `vector`) that rank
    `rank` owns in the peer-memory exchange step: equal shards of whole 16-byte vectors, the last ones shorter
    or empty when the ranks do not divide the vectors.  Returns (lo, hi, shard_length)."""
    if world <= 0 or not 0 <= rank < world or numel % vector:
        raise ValueError("bad world/rank/numel")
    per = (numel // vector + world - 1) // world * vector
    lo = min(numel, rank * per)
    return lo, min(numel, lo + per), per


def max_over_ranks(values, group=None):
    """Element-wise maximum of a list of floats over all ranks (the slowest rank counts)."""
    import torch
    import torch.distributed as dist
    t = torch.tensor(list(values), dtype=torch.float64)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        if dist.get_backend(group) == "nccl":
            t = t.cuda()
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return t.cpu().tolist()
