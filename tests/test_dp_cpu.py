"""Host-side logic of the data-parallel path on CPU: shard bounds, and the bucket reducer
over two gloo ranks (summing buckets asynchronously, finishing before the update)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cnet_b200.dp import GradBucketReducer, shard_bounds


def test_shard_bounds_cover_the_batch():
    for world in (1, 2, 4, 8):
        spans = [shard_bounds(4096, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == 4096
        assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
        assert len({hi - lo for lo, hi in spans}) == 1
    with pytest.raises(ValueError):
        shard_bounds(10, 4, 0)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # a fake gradient arena of 3 buckets; each rank holds the gradient of its batch shard
        g = torch.Generator().manual_seed(7)
        full = torch.randn(world, 1000, generator=g)
        arena = full[rank].clone()
        red = GradBucketReducer()
        assert red.active
        bounds = [(0, 100), (100, 700), (700, 1000)]      # backward order
        for lo, hi in bounds:
            red.on_bucket(arena[lo:hi])
        red.finish()
        ok = torch.allclose(arena, full.sum(0), atol=1e-6) and red.buckets_seen == 3 and not red.works
        # SGD with lr / global batch on the summed gradient gives the same weights on every rank
        w = torch.ones(1000) - (0.01 / 8) * arena
        gathered = [torch.empty_like(w) for _ in range(world)]
        dist.all_gather(gathered, w)
        ok = ok and all(torch.equal(gathered[0], t) for t in gathered)
        out[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_bucket_reducer_two_gloo_ranks():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert dict(out) == {0: True, 1: True}


def test_reducer_is_inert_without_a_process_group():
    red = GradBucketReducer()
    assert not red.active
    t = torch.ones(4)
    red.on_bucket(t)
    red.finish()
    assert torch.equal(t, torch.ones(4))
    assert np.isclose(float(t.sum()), 4.0)
