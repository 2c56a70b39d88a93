"""CPU tests of the multi-rank host logic: the unit split is a partition, and two gloo ranks that
each compute only their own slabs (with the CPU oracle standing in for the kernels) reproduce the
single-rank result exactly, with no data-path collective; timings reduce with max."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT, seeded_normal


def load_sharding():
    import __graft_entry__ as g
    g.load_package()
    import importlib
    return importlib.import_module("cxx_gpt_b200.sharding")


@pytest.mark.parametrize("B,H,world", [(16, 12, 8), (4, 12, 8), (1, 12, 8), (3, 5, 4), (2, 3, 7), (64, 12, 2)])
def test_slabs_partition_all_units(B, H, world):
    sh = load_sharding()
    seen = np.zeros((B, H), int)
    sizes = []
    for r in range(world):
        lo, hi = sh.unit_range(B * H, world, r)
        sizes.append(hi - lo)
        n = 0
        for b, h0, h1 in sh.slabs(B, H, world, r):
            assert 0 <= b < B and 0 <= h0 < h1 <= H
            seen[b, h0:h1] += 1
            n += h1 - h0
        assert n == hi - lo
    assert np.all(seen == 1)
    assert max(sizes) - min(sizes) <= 1


@pytest.mark.parametrize("B,H,world", [(16, 12, 8), (4, 12, 8), (1, 12, 8), (3, 5, 4), (2, 3, 7), (64, 12, 1)])
def test_calls_cover_the_slabs_with_merged_whole_batch_items(B, H, world):
    sh = load_sharding()
    seen = np.zeros((B, H), int)
    for r in range(world):
        cs = sh.calls(B, H, world, r)
        for b0, nb, h0, nh in cs:
            assert nb >= 1 and nh >= 1 and (nb == 1 or (h0 == 0 and nh == H))
            seen[b0:b0 + nb, h0:h0 + nh] += 1
        assert len(cs) <= 3 or H > 12   # at most a partial head range either side of whole batch items
    assert np.all(seen == 1)
    sh16 = sh.calls(16, 12, 8, 3)
    assert sh16 == [(6, 2, 0, 12)]                       # 65,536 tokens at S=4096 on 8 ranks: two batch items each
    assert sh.calls(4, 12, 8, 5) == [(2, 1, 6, 6)]        # S=16384: rank g gets batch g/2, heads 6*(g%2)..+5
    assert sh.calls(64, 12, 1, 0) == [(0, 64, 0, 12)]


def _worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    sh = load_sharding()
    orc = oracle.Oracle()
    orc.set_threads(2)
    B, S, H, Dh = 3, 40, 5, 8
    Q, K, V = seeded_normal(77, [(B * S, H * Dh)] * 3)   # same inputs on every rank, own slabs only
    out = np.zeros_like(Q)
    for b, h0, h1 in sh.slabs(B, H, world, rank):
        rows = slice(b * S, (b + 1) * S)
        cols = slice(h0 * Dh, h1 * Dh)
        out[rows, cols] = orc.mha_fwd(Q[rows, cols], K[rows, cols], V[rows, cols], 1, S, h1 - h0, Dh)
    np.save(os.path.join(tmp, f"part{rank}.npy"), out)
    times = sh.max_over_ranks([1.0 + rank, 5.0 - rank])
    assert times == [float(world), 5.0], times
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("numel,world", [(8, 1), (8, 3), (111_401_472, 8), (111_401_472, 7), (4096, 16), (24, 5)])
def test_parameter_shards_tile_the_buffer_in_whole_vectors(numel, world):
    sharding = load_sharding()
    edge = 0
    for rank in range(world):
        lo, hi, per = sharding.parameter_shard(numel, world, rank)
        assert lo == edge and lo <= hi <= numel and lo % 8 == 0 and (hi - lo) % 8 == 0 and hi - lo <= per
        assert per * world >= numel and per % 8 == 0
        edge = hi
    assert edge == numel
    with pytest.raises(ValueError):
        sharding.parameter_shard(12, 2, 0)


def test_two_gloo_ranks_reproduce_single_rank_result(tmp_path):
    world = 2
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    import oracle
    B, S, H, Dh = 3, 40, 5, 8
    Q, K, V = seeded_normal(77, [(B * S, H * Dh)] * 3)
    want = oracle.Oracle().mha_fwd(Q, K, V, B, S, H, Dh)
    got = sum(np.load(os.path.join(tmp_path, f"part{r}.npy")) for r in range(world))
    np.testing.assert_array_equal(got, want)
