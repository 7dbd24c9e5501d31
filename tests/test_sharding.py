"""CPU: the (batch x KV-head) partition used for multi-GPU runs, including a
world_size-2 gloo run of the validation gather (no GPU, no NCCL)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from moda_b200.sharding import (UnitRange, gather_units, partition_units, shard_heads, unit_seed,
                                units_to_slices)


@pytest.mark.parametrize("n,world", [(8, 1), (8, 2), (8, 4), (8, 8), (256, 8), (7, 3), (2, 4), (0, 2)])
def test_partition_covers_every_unit_once(n, world):
    seen = []
    sizes = []
    for r in range(world):
        rng = partition_units(n, world, r)
        seen += list(range(rng.start, rng.stop))
        sizes.append(len(rng))
    assert seen == list(range(n))
    assert max(sizes) - min(sizes) <= 1


def test_units_to_slices_and_views():
    B, T, H, D = 3, 5, 4, 8
    x = torch.arange(B * T * H * D, dtype=torch.float32).reshape(B, T, H, D)
    rng = UnitRange(2, 9)   # units 2..8 = (b0: h2,h3) (b1: h0..h3) (b2: h0)
    sl = units_to_slices(rng, H)
    assert sl == [(0, 2, 4), (1, 0, 4), (2, 0, 1)]
    views = shard_heads(x, sl)
    assert [tuple(v.shape) for v in views] == [(1, T, 2, D), (1, T, 4, D), (1, T, 1, D)]
    assert views[0].data_ptr() == x[0:1, :, 2:4].data_ptr()      # a view, not a copy
    assert sum(v.shape[2] for v in views) == len(rng)


def test_unit_seed_is_independent_of_rank_count():
    a = {unit_seed(3, tid, u) for tid in range(6) for u in range(8)}
    assert len(a) == 48     # distinct streams per (tensor, unit)
    assert unit_seed(3, 1, 5) == unit_seed(3, 1, 5)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_units, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = partition_units(n_units, world, rank)
        # each rank "computes" its units: row u holds (u, 10*u)
        local = torch.tensor([[u, 10.0 * u] for u in range(rng.start, rng.stop)], dtype=torch.float64).reshape(-1, 2)
        full = gather_units(local, n_units, world, rank)
        ret[rank] = full.tolist()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_units", [8, 5])
def test_gather_units_gloo_world2(n_units):
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = _free_port()
    mp.spawn(_worker, args=(world, port, n_units, ret), nprocs=world, join=True)
    want = [[float(u), 10.0 * u] for u in range(n_units)]
    assert ret[0] == want and ret[1] == want
