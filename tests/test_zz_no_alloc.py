"""The allocation-free Hadamard backward (cnb_hadamard_bwd_static) against the arena-backed
entry point, through the C ABI.  Collected last on purpose: with `-x` every other test has
already run if this one fails.  Some callers of the library may not allocate device memory at
call time (their own pool owns the device, or they cannot take cudaMalloc's device-wide
stall); for them the reduction partials live in an array inside the loaded library, shared by
every call — so the test makes two calls in a row, with different shapes, and checks that the
second is not polluted by what the first left behind."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _p(t):
    return C.c_void_p(t.data_ptr())


def test_static_scratch_entry_matches_arena_entry_on_two_calls():
    import torch
    from cnet_b200 import lib as cl
    from cnet_b200.ops import Context

    lib = cl.load()
    ctx = Context(arena_bytes=64 << 20)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    gen = torch.Generator(device="cuda").manual_seed(11)
    try:
        for B, N in ((300, 1024), (37, 130)):          # second call: smaller and ragged
            t = [torch.randn(B, N, device="cuda", generator=gen) for _ in range(4)]
            g, u = (t[0], t[1]), (t[2], t[3])
            v = tuple(torch.randn(N, device="cuda", generator=gen) for _ in range(2))
            du_ref, dv_ref = ctx.hadamard_bwd(g, u, v)
            du = (torch.full((B, N), 7.0, device="cuda"), torch.full((B, N), 7.0, device="cuda"))
            dv = (torch.full((N,), 7.0, device="cuda"), torch.full((N,), 7.0, device="cuda"))
            rc = lib.cnb_hadamard_bwd_static(_p(g[0]), _p(g[1]), _p(u[0]), _p(u[1]), _p(v[0]), _p(v[1]),
                                             _p(du[0]), _p(du[1]), 0, _p(dv[0]), _p(dv[1]), 0, B, N, stream)
            assert rc == 0, lib.cnb_last_error()
            torch.cuda.synchronize()
            for got, want in zip(du + dv, du_ref + dv_ref):
                err = float((got - want).norm() / want.norm())
                assert err < 1e-6, (B, N, err)
            # and directly against the definition in float64 (impl/hadamard.h:46-68): du* = g* o conj(v),
            # dv* = sum over the batch of g* o conj(u)
            g64, u64 = g[0].double() + 1j * g[1].double(), u[0].double() + 1j * u[1].double()
            v64 = v[0].double() + 1j * v[1].double()
            for got, want in (((du[0].double() + 1j * du[1].double()), g64 * v64.conj()),
                              ((dv[0].double() + 1j * dv[1].double()), (g64 * u64.conj()).sum(0))):
                assert float((got - want).abs().pow(2).sum().sqrt() / want.abs().pow(2).sum().sqrt()) < 1e-5
            # accumulate form: adds onto what is there
            rc = lib.cnb_hadamard_bwd_static(_p(g[0]), _p(g[1]), _p(u[0]), _p(u[1]), _p(v[0]), _p(v[1]),
                                             None, None, 0, _p(dv[0]), _p(dv[1]), 1, B, N, stream)
            assert rc == 0
            torch.cuda.synchronize()
            assert float((dv[0] - 2 * dv_ref[0]).norm() / dv_ref[0].norm()) < 1e-6
        # beyond the built-in scratch: refused with a message, nothing launched
        n_big = 4096 + 4
        z = torch.zeros(2, n_big, device="cuda")
        zv = torch.zeros(n_big, device="cuda")
        before = lib.cnb_launch_count()
        rc = lib.cnb_hadamard_bwd_static(_p(z), _p(z), _p(z), _p(z), _p(zv), _p(zv), None, None, 0, _p(zv), _p(zv), 0,
                                         2, n_big, stream)
        assert rc == -1 and b"exceeds" in lib.cnb_last_error()
        assert lib.cnb_launch_count() == before
    finally:
        ctx.close()
    assert np.isfinite(float(dv[0].sum()))
