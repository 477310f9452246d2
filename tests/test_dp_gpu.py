"""Data-parallel training on 2 GPUs (NCCL) against the single-GPU run of the same global batch, at the
benchmark's own width: the token-mixing stack of 8 blocks of 1024, global batch 4096, SGD lr 0.01,
200 steps from seed 0 (4 seeded batches in rotation).  The per-step loss curve (mean over the WHOLE
batch) and the weights after the last update must agree to fp32 reassociation noise.  Needs two CUDA
devices; skipped otherwise.  NVLS is switched off for the child ranks."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

KW = dict(n=1024, blocks=8, m=10)
GLOBAL_BATCH, STEPS, LR, BATCHES = 4096, 200, 0.01, 4


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _train(rank, world, port, out, comm="auto"):
    import torch
    import torch.distributed as dist
    from cnet_b200 import configs
    from cnet_b200.dp import DataParallelTrainer
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    if world > 1:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        tr = DataParallelTrainer(configs.build_mixer, KW, global_batch=GLOBAL_BATCH, lr=LR, device=rank, seed=0, comm=comm)
        losses = []
        data = [configs.make_batch(tr.spec, GLOBAL_BATCH, 0, step=s) for s in range(BATCHES)]
        for s in range(STEPS):
            (xr, xi), labels = data[s % BATCHES]
            if s == 2:
                tr.capture()            # the rest of the run replays the step as a CUDA graph
            l = tr.step((tr.shard(xr), tr.shard(xi)), tr.shard(labels))
            tot = torch.tensor([float(l.sum())], device="cuda")
            if world > 1:
                dist.all_reduce(tot)
            losses.append(float(tot.item()) / GLOBAL_BATCH)
        tr.net.sync()
        w = tr.net.get_values(tr.spec.layers["w7"])
        h = tr.net.get_values(tr.spec.layers["h0"])
        out[(world, rank, comm)] = (np.array(losses), w[0], w[1], h[0], h[1], tr.net.grad_arena()[2])
    finally:
        if world > 1:
            dist.destroy_process_group()


@pytest.mark.parametrize("comm", ["nccl", "symm"])
def test_two_gpu_training_matches_single_gpu(comm):
    """comm = nccl: NCCL all-reduce on the registered symmetric window; symm: the library's own all-reduce kernel
    on torch symmetric memory (multimem where the platform has it)."""
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    mgr = mp.Manager()
    out = mgr.dict()
    if (1, 0, "auto") not in _SINGLE:
        mp.spawn(_train, args=(1, 0, out), nprocs=1, join=True)
        _SINGLE[(1, 0, "auto")] = out[(1, 0, "auto")]
    mp.spawn(_train, args=(2, _free_port(), out, comm), nprocs=2, join=True)
    one, r0, r1 = _SINGLE[(1, 0, "auto")], out[(2, 0, comm)], out[(2, 1, comm)]
    assert one[5] >= 1
    assert np.linalg.norm(r0[0] - one[0]) / np.linalg.norm(one[0]) < 1e-4
    assert np.max(np.abs(r0[0] - one[0]) / one[0]) < 3e-4          # every single step, not only on average
    assert one[0][-1] < 0.9 * one[0][0]                            # and the run did train
    for k in range(1, 5):
        assert np.array_equal(r0[k], r1[k])                     # replicas stay identical
        assert np.linalg.norm(r0[k] - one[k]) / np.linalg.norm(one[k]) < 1e-4


_SINGLE = {}
