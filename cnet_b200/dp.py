"""Data-parallel training of a CNet: the only sharded path.

The batch is split evenly over the ranks (one process per GPU); weights are replicated
(identical seeded init); during the backward pass every finished bucket of the contiguous
weight-gradient arena is summed over the ranks with an asynchronous all-reduce
(torch.distributed: NCCL over NVLink on GPUs, gloo in the CPU tests) that overlaps the rest of
the backward; the fused SGD update runs after the last bucket with lr / global_batch — the
multi-GPU analogue of the reference's gpu_grad_from_clones + gpuUpdateInputs(l_rate / batch)
(gpu/kernels.cpp:566-598, cnet.cpp:147).
"""
import os

import numpy as np

from . import configs


def shard_bounds(global_batch, world, rank):
    """Rows [lo, hi) of the global batch owned by `rank` (even split required)."""
    if global_batch % world != 0:
        raise ValueError("global batch %d is not divisible by %d ranks" % (global_batch, world))
    per = global_batch // world
    return rank * per, (rank + 1) * per


class GradBucketReducer:
    """Sums gradient buckets over the ranks as they complete; `finish()` waits for all of them.

    Works on any torch tensor views (CUDA with NCCL, CPU with gloo).  With world size 1 it
    does nothing.
    """

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist = dist
        self.active = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        self.group = group
        self.works = []
        self.buckets_seen = 0

    def on_bucket(self, view):
        self.buckets_seen += 1
        if self.active:
            self.works.append(self.dist.all_reduce(view, op=self.dist.ReduceOp.SUM, group=self.group, async_op=True))

    def finish(self):
        for w in self.works:
            w.wait()
        self.works = []


class DataParallelTrainer:
    """One rank of a data-parallel training job (or the whole job when there is one rank).

    comm = "nccl": the host facade owns an NCCL communicator and issues the bucket all-reduces
    itself on a communication stream (capturable in a CUDA graph together with the kernels);
    comm = "torch": the buckets are handed to torch.distributed through a Python hook (any backend;
    what the CPU tests exercise with gloo).  "auto" picks "nccl" when the job has several ranks.
    """

    def __init__(self, builder, builder_kwargs, global_batch, lr, device=0, seed=0, fuse=True, comm="auto"):
        import torch
        import torch.distributed as dist
        from .net import Net
        self.torch = torch
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.global_batch = global_batch
        self.lo, self.hi = shard_bounds(global_batch, self.world, self.rank)
        self.local_batch = self.hi - self.lo
        self.lr = lr
        self.graph = False
        torch.cuda.set_device(device)
        self.stream = torch.cuda.Stream(device=device)     # a capturable (non-default) stream
        self.net = Net(device=device)
        self.spec = builder(self.net, **builder_kwargs)
        for uid, (re, im) in configs.init_weights(self.spec, seed).items():
            self.net.set_values(uid, re, im)
        if comm == "auto":
            # several ranks: the library's own all-reduce on symmetric memory where the platform maps it with a
            # multicast address, else NCCL on a registered window (CNB_DP_COMM = symm | nccl forces one)
            # The own kernel has run on 2 and 4 GPUs of this pool; no 8-GPU machine could be had to run it on, so
            # 8 ranks take NCCL (on the same in-switch reduction) unless CNB_DP_COMM=symm asks otherwise.
            default = "symm?" if self.world <= 4 else "nccl"
            comm = os.environ.get("CNB_DP_COMM", default) if self.world > 1 else "none"
        self.comm = comm
        self.symm = None
        if self.world > 1 and self.comm in ("symm", "symm?"):
            made = self._symmetric_arena(device)
            ok = torch.tensor([1 if made and (self.comm == "symm" or made[2].multicast_ptr) else 0], device="cuda")
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)            # every rank takes the same path
            if int(ok.item()) == 0:
                if self.comm == "symm":
                    raise RuntimeError("symmetric memory could not be set up on every rank")
                made = None
                self.comm = "nccl"
            else:
                self.comm = "symm"
        if self.world > 1 and self.comm == "symm":
            # the library's own all-reduce kernel on symmetric memory: torch only maps the arenas of all ranks into
            # every process (peer pointers, a multicast address where the platform has one)
            arena, flags, ah, fh = made
            self.symm = (arena, flags, ah, fh)
            self.net.allocate(self.local_batch, fuse=fuse, stream=self.stream.cuda_stream, arena=arena)
            mc = int(ah.multicast_ptr or 0)                     # 0 where the platform has no NVLink multicast
            if os.environ.get("CNB_DP_MULTICAST", "1") == "0":
                mc = 0
            self.net.dp_set_symmetric(self.rank, self.world, mc, list(ah.buffer_ptrs), list(fh.buffer_ptrs),
                                      int(os.environ.get("CNB_DP_CTAS", "0")))
            self.multicast = bool(mc)
            dist.barrier()
        else:
            # several ranks over NCCL: the arena comes from NCCL's allocator, so the gradients can be a symmetric window
            self.net.allocate(self.local_batch, fuse=fuse, stream=self.stream.cuda_stream,
                              nccl_arena=self.world > 1 and self.comm == "nccl")
        self.reducer = GradBucketReducer() if self.comm == "torch" else None
        if self.world > 1 and self.comm == "nccl":
            box = [self.net.dp_unique_id() if self.rank == 0 else None]
            dist.broadcast_object_list(box, src=0)
            self.net.dp_init(box[0], self.rank, self.world)
        elif self.reducer is not None and self.reducer.active:
            arena = self.net.arena
            base = arena.data_ptr()

            def hook(ptr, count, bucket, n_buckets):
                off = ptr - base
                self.reducer.on_bucket(arena[off:off + 4 * count].view(torch.float32))
                return 0
            self.net.set_bucket_hook(hook)

    def _symmetric_arena(self, device):
        """(arena, flags, arena handle, flags handle) in torch symmetric memory, or None if that fails here."""
        import torch.distributed as dist
        torch = self.torch
        try:
            import torch.distributed._symmetric_memory as symm_mem
            group = dist.group.WORLD
            need = self.net.required_arena(self.local_batch)
            sizes = torch.tensor([need], device="cuda", dtype=torch.int64)
            dist.all_reduce(sizes, op=dist.ReduceOp.MAX)        # the same size (and so the same offsets) on every rank
            arena = symm_mem.empty(int(sizes.item()), dtype=torch.uint8, device="cuda:%d" % device)
            flags = symm_mem.empty(256, dtype=torch.int32, device="cuda:%d" % device)
            flags.zero_()
            ah, fh = symm_mem.rendezvous(arena, group), symm_mem.rendezvous(flags, group)
            torch.cuda.synchronize()
            return arena, flags, ah, fh
        except Exception as e:                                   # no symmetric memory on this platform / build
            import sys
            print("cnet_b200: symmetric memory unavailable (%s: %s)" % (type(e).__name__, e), file=sys.stderr)
            return None

    def upload(self, host_in, host_labels):
        """Copies this rank's shard (pinned host tensors or numpy arrays) to the device."""
        if self.spec.tokens:
            self.net.upload(tokens=host_in[0], labels=host_labels, batch=self.local_batch)
        else:
            self.net.upload(x=host_in, labels=host_labels, batch=self.local_batch)

    def _step_eager(self):
        with self.torch.cuda.stream(self.stream):
            self.net.forward()
            self.net.backward()
            if self.reducer is not None:
                self.reducer.finish()
            self.net.update_inputs(self.lr / self.global_batch)

    def capture(self):
        """Capture forward + backward (+ bucket all-reduces) + update into one CUDA graph.

        The step is a fixed sequence of ~120 launches on static arena addresses; replaying it as a
        graph removes the per-launch host cost, which dominates once the per-GPU batch is small.
        Call after at least one eager step (twiddle tables, kernel attributes and the NCCL
        communicator are set up outside the capture).
        """
        if self.comm == "torch" and self.world > 1:
            raise RuntimeError("graph capture needs comm='nccl' or 'symm' (collectives issued by the host facade)")
        self.torch.cuda.synchronize()
        self.net.capture_begin()
        try:
            self.net.forward()
            self.net.backward()
            self.net.update_inputs(self.lr / self.global_batch)
        finally:
            self.net.capture_end()
        self.torch.cuda.synchronize()
        self.graph = True

    def step_resident(self):
        """forward + backward (+ overlapped gradient all-reduce) + update on the resident batch."""
        if self.graph:
            self.net.graph_launch()
        else:
            self._step_eager()

    def kernels_per_step(self):
        return self.net.graph_kernel_count() if self.graph else None

    def prefetch(self, host_in, host_labels):
        """Start the H2D copy of this rank's shard of the NEXT batch (overlaps the running step)."""
        if self.spec.tokens:
            self.net.prefetch(tokens=host_in[0], labels=host_labels, batch=self.local_batch)
        else:
            self.net.prefetch(x=host_in, labels=host_labels, batch=self.local_batch)

    def step_pipelined(self, next_in, next_labels, loss_out):
        """One step on the batch staged by the previous call, while `next_*` is copied in for the next one;
        the step's per-sample losses land in `loss_out` (pinned) asynchronously: call net.wait_losses()."""
        self.net.commit()
        if next_in is not None:
            self.prefetch(next_in, next_labels)
        self.step_resident()
        self.net.wait_losses()          # the previous step's losses: the host stays one step ahead at most
        self.net.read_losses_async(loss_out, self.local_batch)

    def step(self, host_in, host_labels):
        self.upload(host_in, host_labels)
        self.step_resident()
        return self.net.losses(self.local_batch)

    def shard(self, arr):
        return np.ascontiguousarray(arr[self.lo:self.hi])
