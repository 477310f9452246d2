"""Python face of the host facade: build a CNet, put it on a B200, run training steps.

Mirrors the reference's API names (add / init_inputs / allocateOnGpu / gpuForward /
gpuBackward / gpuUpdateInputs / getLoss, gpu/gpu_func.h:1013-1101) over the flat binding
in include/cnet_b200_host.h.  All compute is in libcnet_b200.so; torch is used only to own
device memory (the arena) and streams.
"""
import ctypes as C

import numpy as np

from . import lib as _lib
from .configs import (CROSSENT, EMBEDDING, FOURIER, GELU, HADAMARD, INPUT, LINEAR, RESIDUAL,  # noqa: F401
                      SOFTMAX)


def _addr(a):
    """Address of a host buffer: numpy array or CPU torch tensor (contiguous)."""
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        assert a.flags["C_CONTIGUOUS"]
        return a.ctypes.data
    return a.data_ptr()


class Net:
    def __init__(self, device=0, arena_bytes=0, use_torch_arena=True):
        self.lib = _lib.load()
        self.device = device
        self.arena_bytes = arena_bytes
        self.use_torch_arena = use_torch_arena
        self.arena = None
        self.h = None
        self.h = C.c_void_p(self.lib.cnh_create(device, 0, None))
        self._specs = {}
        self.batch = 0
        self.main_is_tokens = False
        self._hook_ref = None
        self.allocated = False

    def __del__(self):
        try:
            if self.h:
                self.lib.cnh_destroy(self.h)
                self.h = None
        except Exception:
            pass

    # ------------------------------------------------------------------ graph
    def _check(self, rc, what):
        if rc < 0:
            msg = self.lib.cnh_error(self.h).decode()
            self.lib.cnh_clear_error(self.h)
            raise _lib.CnetError("%s: %s" % (what, msg))
        return rc

    def add(self, type_, a=0, b=0, c=0, prev=()):
        p = np.asarray(list(prev), np.int32)
        uid = self._check(self.lib.cnh_add(self.h, type_, a, b, c, p.ctypes.data_as(C.POINTER(C.c_int32)), len(p)),
                          "add")
        in_len = a * c if type_ == EMBEDDING else self.lib.cnh_out_size(self.h, uid)
        self._specs[uid] = (type_, in_len)
        if len(self._specs) == 1:
            self.main_is_tokens = type_ == EMBEDDING
        return uid

    def out_size(self, uid):
        return self.lib.cnh_out_size(self.h, uid)

    def init_inputs(self, seed=0):
        self._check(self.lib.cnh_init_inputs(self.h, seed), "init_inputs")

    def set_values(self, uid, re, im):
        re = np.ascontiguousarray(re, np.float32).reshape(-1)
        im = np.ascontiguousarray(im, np.float32).reshape(-1)
        self._check(self.lib.cnh_set_values(self.h, uid, re.ctypes.data, im.ctypes.data, re.size), "set_values")

    def _pair(self, fn, uid, what):
        n = self._specs[uid][1]
        re, im = np.empty(n, np.float32), np.empty(n, np.float32)
        self._check(fn(self.h, uid, re.ctypes.data, im.ctypes.data, n), what)
        return re, im

    def get_values(self, uid):
        return self._pair(self.lib.cnh_get_values, uid, "get_values")

    def get_wgrad(self, uid):
        return self._pair(self.lib.cnh_get_wgrad, uid, "get_wgrad")

    # ------------------------------------------------------------ checkpoints
    def save(self, path):
        """CNet::save: the reference's ModelSaver byte format (weights are read back from the device first)."""
        self._check(self.lib.cnh_save(self.h, str(path).encode()), "save")

    @classmethod
    def restore(cls, path, device=0):
        """CNet::restore into a fresh net; returns it (not yet allocated on the GPU)."""
        net = cls(device=device)
        net._check(net.lib.cnh_restore(net.h, str(path).encode()), "restore")
        for i in range(net.lib.cnh_num_funcs(net.h)):
            uid = net.lib.cnh_uid_at(net.h, i)
            t = net.lib.cnh_type_of(net.h, uid)
            in_len = net.lib.cnh_in_size(net.h, uid) if t == EMBEDDING else net.lib.cnh_out_size(net.h, uid)
            net._specs[uid] = (t, in_len)
            if i == 0:
                net.main_is_tokens = t == EMBEDDING
        return net

    def uids(self):
        return [self.lib.cnh_uid_at(self.h, i) for i in range(self.lib.cnh_num_funcs(self.h))]

    def type_of(self, uid):
        return self.lib.cnh_type_of(self.h, uid)

    # ----------------------------------------------------------------- device
    def required_arena(self, batch):
        return self.arena_bytes or self.lib.cnh_required_arena(self.h, batch)

    def allocate(self, batch, fuse=True, stream=None, nccl_arena=False, arena=None):
        """allocateOnGpu(batch): plan the batched tensors in one arena and upload the weights.
        nccl_arena: the host facade takes the arena from NCCL's allocator (for a symmetric window in dp_init).
        arena: a uint8 CUDA tensor of at least required_arena(batch) bytes to use (e.g. symmetric memory)."""
        import torch
        if not torch.cuda.is_available():
            raise _lib.CnetError("no CUDA device: the path has no CPU fallback")
        need = self.required_arena(batch)
        if arena is not None:
            assert arena.numel() >= need and arena.dtype == torch.uint8
            self.arena = arena
            need = arena.numel()
            ext = arena.data_ptr()
        elif nccl_arena:
            torch.cuda.set_device(self.device)
            self.lib.cnh_dp_use_nccl_arena(self.h, 1)
            ext = None
        elif self.use_torch_arena:
            torch.cuda.set_device(self.device)
            self.arena = torch.empty(need, dtype=torch.uint8, device="cuda:%d" % self.device)
            ext = self.arena.data_ptr()
        else:
            ext = None
        self.lib.cnh_set_fusion(self.h, 1 if fuse else 0)
        self._set_arena(need, ext)
        if stream is None:
            stream = torch.cuda.current_stream().cuda_stream
        self.lib.cnh_set_stream(self.h, C.c_void_p(stream))
        self.stream = stream
        self._check(self.lib.cnh_allocate(self.h, batch), "allocateOnGpu")
        self.batch = batch
        self.allocated = True

    def _set_arena(self, nbytes, ext):
        self.lib.cnh_set_device(self.h, self.device, nbytes, ext)

    def set_stream(self, stream):
        """Stream (raw cudaStream_t value) every following call launches on."""
        self.lib.cnh_set_stream(self.h, C.c_void_p(stream))
        self.stream = stream

    def upload(self, x=None, tokens=None, labels=None, batch=None):
        """batchToGpu: host planes [B, n] (numpy or pinned CPU torch tensors) or tokens [B, T]; labels [B]."""
        if tokens is not None:
            B = batch or tokens.shape[0]
            rc = self.lib.cnh_upload(self.h, None, None, _addr(tokens), _addr(labels), B)
        else:
            B = batch or x[0].shape[0]
            rc = self.lib.cnh_upload(self.h, _addr(x[0]), _addr(x[1]), None, _addr(labels), B)
        self._check(rc, "batchToGpu")
        self.cur_batch = B

    def prefetch(self, x=None, tokens=None, labels=None, batch=None):
        """Start copying the NEXT batch (pinned host buffers) to a device staging area on the copy stream."""
        if tokens is not None:
            B = batch or tokens.shape[0]
            rc = self.lib.cnh_prefetch(self.h, None, None, _addr(tokens), _addr(labels), B)
        else:
            B = batch or x[0].shape[0]
            rc = self.lib.cnh_prefetch(self.h, _addr(x[0]), _addr(x[1]), None, _addr(labels), B)
        self._check(rc, "prefetchBatch")
        self._staged = B

    def commit(self):
        """Make the staged batch the current one (compute stream waits for its copy)."""
        self._check(self.lib.cnh_commit(self.h), "commitBatch")
        self.cur_batch = self._staged

    def read_losses_async(self, pinned_out, n):
        self._check(self.lib.cnh_read_losses_async(self.h, _addr(pinned_out), n), "readLossesAsync")

    def wait_losses(self):
        self._check(self.lib.cnh_wait_losses(self.h), "waitLosses")

    def forward(self):
        self._check(self.lib.cnh_forward(self.h), "forward")

    def backward(self):
        self._check(self.lib.cnh_backward(self.h), "backward")

    def update_inputs(self, lr):
        """gpuUpdateInputs(l_rate): w -= l_rate * dz*_w, gradients zeroed."""
        self._check(self.lib.cnh_update(self.h, lr), "updateInputs")

    def adam_update(self, lr, beta, t):
        """CNet::adamUpdate: momentum-only Adam of the reference; pass lr / batch."""
        self._check(self.lib.cnh_adam_update(self.h, lr, beta, t), "adamUpdate")

    def infer(self):
        self._check(self.lib.cnh_infer(self.h), "infer")

    def losses(self, n=None):
        n = n or self.cur_batch
        out = np.empty(n, np.float32)
        self._check(self.lib.cnh_get_losses(self.h, out.ctypes.data, n), "getLoss")
        return out

    def losses_into(self, host_tensor, n):
        self._check(self.lib.cnh_get_losses(self.h, _addr(host_tensor), n), "getLoss")

    def sync(self):
        self._check(self.lib.cnh_sync(self.h), "sync")

    # ------------------------------------------------- data parallel, graphs
    def dp_init(self, unique_id, rank, nranks):
        """setDataParallel: join the NCCL communicator made from `unique_id` (128 bytes)."""
        self._check(self.lib.cnh_dp_init(self.h, unique_id, rank, nranks), "setDataParallel")

    @staticmethod
    def dp_unique_id():
        buf = C.create_string_buffer(128)
        if _lib.load().cnh_dp_unique_id(buf) != 0:
            raise _lib.CnetError("ncclGetUniqueId failed (is libnccl.so.2 loadable?)")
        return buf.raw

    def dp_set_symmetric(self, rank, world, multicast_ptr, arena_ptrs, flag_ptrs, ctas=0):
        """setSymmetricPeers: every rank's arena and flag block as mapped in this process (symmetric memory)."""
        a = (C.c_void_p * world)(*[C.c_void_p(int(x)) for x in arena_ptrs])
        f = (C.c_void_p * world)(*[C.c_void_p(int(x)) for x in flag_ptrs])
        self._check(self.lib.cnh_dp_set_symmetric(self.h, rank, world, C.c_void_p(int(multicast_ptr) or None), a, f, ctas),
                    "setSymmetricPeers")

    def dp_allreduce_grads(self):
        """Sum the whole weight-gradient arena over the ranks now."""
        self._check(self.lib.cnh_dp_allreduce_grads(self.h), "allReduceGradients")

    def capture_begin(self):
        self._check(self.lib.cnh_capture_begin(self.h), "beginCapture")

    def capture_end(self):
        self._check(self.lib.cnh_capture_end(self.h), "endCapture")

    def graph_launch(self):
        self._check(self.lib.cnh_graph_launch(self.h), "launchGraph")

    def graph_kernel_count(self):
        return self.lib.cnh_graph_kernel_count(self.h)

    def context(self):
        return C.c_void_p(self.lib.cnh_context(self.h))

    def grad_arena(self):
        """(device pointer, float count, bucket count) of the contiguous weight-gradient arena."""
        p, n, nb = C.c_void_p(), C.c_size_t(), C.c_int()
        self.lib.cnh_grad_arena(self.h, C.byref(p), C.byref(n), C.byref(nb))
        return p.value, n.value, nb.value

    def grad_tensor(self):
        """The weight-gradient arena as a torch float32 view (for collectives)."""
        import torch
        p, n, _ = self.grad_arena()
        off = p - self.arena.data_ptr()
        return self.arena[off:off + 4 * n].view(torch.float32)

    def set_bucket_hook(self, fn):
        """fn(device_ptr, count, bucket, n_buckets) -> int, called as gradient buckets complete."""
        if fn is None:
            self._hook_ref = None
            self.lib.cnh_set_bucket_hook(self.h, C.cast(None, _lib.BUCKET_HOOK), None)
            return
        self._hook_ref = _lib.BUCKET_HOOK(lambda user, ptr, count, b, nb: int(fn(ptr, count, b, nb) or 0))
        self.lib.cnh_set_bucket_hook(self.h, self._hook_ref, None)

    # ------------------------------------------------ checker-compatible face
    def run_batch(self, main_uid, x=None, tokens=None, labels=None, record=True):
        """One forward + backward over a batch; same signature as the CPU checkers in tests."""
        labels = np.ascontiguousarray(labels, np.int32)
        if tokens is not None:
            self.upload(tokens=np.ascontiguousarray(tokens, np.int32), labels=labels)
        else:
            self.upload(x=(np.ascontiguousarray(x[0], np.float32), np.ascontiguousarray(x[1], np.float32)),
                        labels=labels)
        self.forward()
        self.backward()
        self.sync()
        return self.losses().astype(np.float64)

    def get_record(self, uid, what):
        n = self.out_size(uid)
        re, im = np.empty((self.cur_batch, n), np.float32), np.empty((self.cur_batch, n), np.float32)
        self._check(self.lib.cnh_read_output(self.h, uid, what, re.ctypes.data, im.ctypes.data), "readOutput")
        return re, im

    def update(self, lr, batch_size):
        """ComplexNet::update(lr, batch): w -= (lr / batch) * dz*_w."""
        self.update_inputs(lr / batch_size)
        self.sync()

    def adam(self, lr, batch_size, beta, t):
        """ComplexNet::adamUpdate(lr, batch, beta, t)."""
        self.adam_update(lr / batch_size, beta, t)
        self.sync()
