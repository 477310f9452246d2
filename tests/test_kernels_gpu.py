"""GPU parity of single operators through the C ABI (cnet_b200.ops -> libcnet_b200.so)
against the float64 math of the reference layers, including ragged and edge shapes."""
import numpy as np
import pytest

import util
from oracle import cnet_oracle as co

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    from cnet_b200.ops import Context
    c = Context(arena_bytes=512 << 20)
    yield c
    c.close()


def _rand(rng, *shape, scale=1.0):
    return ((rng.standard_normal(shape) * scale).astype(np.float32),
            (rng.standard_normal(shape) * scale).astype(np.float32))


def _dev(pair):
    import torch
    return tuple(torch.from_numpy(np.ascontiguousarray(p)).cuda() for p in pair)


def _host(pair):
    return tuple(p.cpu().numpy() for p in pair)


def _c(pair):
    return pair[0].astype(np.float64) + 1j * pair[1].astype(np.float64)


def _pair(z):
    return (z.real, z.imag)


# the last rows exercise the tensor-core GEMM's schedules: k-split tiles summed with atomics,
# runs that cover whole tiles plus a split remainder, one-tile-per-CTA grids, ragged M/N/K edges
@pytest.mark.parametrize("B,n_in,n_out", [(1, 1, 1), (7, 48, 40), (64, 784, 10), (4095, 1024, 10), (3, 33, 16), (33, 100, 130), (256, 512, 384),
                                          (128, 1024, 1024), (4096, 256, 1024), (3072, 64, 3200), (200, 100, 72),
                                          (1000, 36, 1000),
                                          # ragged tiles under every GEMM schedule: whole tiles first + shared remainder
                                          # (180 tiles), stream-K, clusters of 2 and 4 with an uneven K split
                                          (2500, 520, 1064), (300, 1024, 1024)])
def test_linear_three_products(ctx, B, n_in, n_out):
    rng = np.random.default_rng(B * 1000 + n_in)
    x, w, g = _rand(rng, B, n_in), _rand(rng, n_out, n_in, scale=n_in ** -0.5), _rand(rng, B, n_out)
    r = _rand(rng, B, n_out)
    X, W, G = _c(x), _c(w), _c(g)
    y = _host(ctx.linear_fwd(_dev(x), _dev(w)))
    assert util.relerr(y, _pair(X @ W.T)) < 1e-5
    # square shapes run on the tcgen05 tiles, skinny / tiny ones on the fp32 SIMT tiles
    want_engine = 4 if (n_out <= 16 and n_in >= 32) else 1 if (B >= 64 and n_out >= 64 and n_in >= 32 and n_in % 8 == 0) else 2
    assert ctx.last_gemm_engine() == want_engine
    yr = _host(ctx.linear_fwd(_dev(x), _dev(w), res=_dev(r)))
    assert util.relerr(yr, _pair(X @ W.T + _c(r))) < 1e-5
    dx = _host(ctx.linear_bwd_x(_dev(g), _dev(w)))
    assert util.relerr(dx, _pair(G @ np.conj(W))) < 1e-5
    dw = _host(ctx.linear_bwd_w(_dev(g), _dev(x)))
    assert util.relerr(dw, _pair(G.T @ np.conj(X))) < 1e-5
    # accumulate form
    acc = _dev(dw)
    dw2 = _host(ctx.linear_bwd_w(_dev(g), _dev(x), out=acc))
    assert util.relerr(dw2, _pair(2 * (G.T @ np.conj(X)))) < 1e-5


@pytest.mark.parametrize("B,N", [(3, 8), (5, 100), (64, 784), (32, 1024), (37, 1024), (5, 256), (3, 4096),
                                 (600, 1024)])
def test_fourier_forward_backward(ctx, B, N):
    rng = np.random.default_rng(N)
    x, g = _rand(rng, B, N), _rand(rng, B, N)
    want_f = _pair(np.fft.fft(_c(x), axis=1) / np.sqrt(N))
    want_b = _pair(np.fft.ifft(_c(g), axis=1) * np.sqrt(N))
    y = _host(ctx.dft_fwd(_dev(x)))
    assert util.relerr(y, want_f) < 1e-5
    # N = 256, 1024, 4096 use the shared-memory FFT kernel, everything else the DFT GEMM
    assert (ctx.last_gemm_engine() == 3) == (N in (256, 1024, 4096))
    dx = _host(ctx.dft_bwd(_dev(g)))
    assert util.relerr(dx, want_b) < 1e-5
    acc = _dev((want_b[0].astype(np.float32), want_b[1].astype(np.float32)))
    dx2 = _host(ctx.dft_bwd(_dev(g), out=acc))
    assert util.relerr(dx2, (2 * want_b[0], 2 * want_b[1])) < 1e-5
    if N in (256, 1024, 4096):       # the GEMM form of the same transform agrees
        ctx.lib.cnb_set_dft_engine(ctx.h, 1)
        try:
            assert util.relerr(_host(ctx.dft_fwd(_dev(x))), want_f) < 1e-5
            assert ctx.last_gemm_engine() != 3
            assert util.relerr(_host(ctx.dft_bwd(_dev(g))), want_b) < 1e-5
        finally:
            ctx.lib.cnb_set_dft_engine(ctx.h, 0)


@pytest.mark.parametrize("B,N", [(1, 1), (5, 7), (64, 784), (300, 1024), (9, 130)])
def test_hadamard_gelu_residual(ctx, B, N):
    rng = np.random.default_rng(B + N)
    u, h, v, g = _rand(rng, B, N), _rand(rng, N), _rand(rng, B, N), _rand(rng, B, N)
    U, H, V, G = _c(u), _c(h), _c(v), _c(g)
    assert util.relerr(_host(ctx.hadamard_fwd(_dev(u), _dev(h))), _pair(U * H)) < 1e-6
    assert util.relerr(_host(ctx.hadamard_fwd(_dev(u), _dev(v))), _pair(U * V)) < 1e-6
    du, dh = ctx.hadamard_bwd(_dev(g), _dev(u), _dev(h))
    assert util.relerr(_host(du), _pair(G * np.conj(H))) < 1e-6
    assert util.relerr(_host(dh), _pair((G * np.conj(U)).sum(0))) < 1e-5
    du, dv = ctx.hadamard_bwd(_dev(g), _dev(u), _dev(v))
    assert util.relerr(_host(dv), _pair(G * np.conj(U))) < 1e-6
    # CGelu
    want = co._gelu(U.real) + 1j * co._gelu(U.imag)
    assert util.relerr(_host(ctx.gelu_fwd(_dev(u))), _pair(want)) < 1e-6
    dx, dy = 0.5 * co._dgelu(U.real), 0.5 * co._dgelu(U.imag)
    wantb = np.conj(G) * (dx - dy) + G * (dx + dy)
    assert util.relerr(_host(ctx.gelu_bwd(_dev(g), _dev(u))), _pair(wantb)) < 1e-5
    # fused pair
    a, y = ctx.hadamard_gelu_fwd(_dev(u), _dev(h))
    A = U * H
    assert util.relerr(_host(a), _pair(A)) < 1e-6
    assert util.relerr(_host(y), _pair(co._gelu(A.real) + 1j * co._gelu(A.imag))) < 1e-6
    dx, dy = 0.5 * co._dgelu(A.real), 0.5 * co._dgelu(A.imag)
    T = np.conj(G) * (dx - dy) + G * (dx + dy)
    du, dh = ctx.hadamard_gelu_bwd(_dev(g), a, _dev(u), _dev(h))
    assert util.relerr(_host(du), _pair(T * np.conj(H))) < 1e-5
    assert util.relerr(_host(dh), _pair((T * np.conj(U)).sum(0))) < 1e-5
    # residual and pass-through
    assert util.relerr(_host(ctx.residual_fwd(_dev(u), _dev(v))), _pair(U + V)) < 1e-7
    dst = _dev(v)
    assert util.relerr(_host(ctx.axpy(_dev(g), dst, True)), _pair(V + G)) < 1e-7
    assert util.relerr(_host(ctx.axpy(_dev(g), dst, False)), _pair(G)) == 0.0


@pytest.mark.parametrize("B,M", [(1, 2), (64, 10), (17, 130), (8, 8192)])
def test_crossent_and_softmax(ctx, B, M):
    import torch
    rng = np.random.default_rng(M)
    z, g = _rand(rng, B, M), _rand(rng, B, M)
    labels = rng.integers(0, M, B).astype(np.int32)
    Z, G = _c(z), _c(g)
    S = np.maximum((np.abs(Z) ** 2).sum(1), 1e-15)
    zl = Z[np.arange(B), labels]
    loss, d = ctx.crossent(_dev(z), torch.from_numpy(labels).cuda())
    assert util.relerr(loss.cpu().numpy(), -np.log(np.maximum(np.abs(zl) ** 2 / S, 1e-15))) < 1e-5
    want = Z / S[:, None]
    m = np.maximum(np.abs(zl) ** 2, 1e-15)
    want[np.arange(B), labels] = -zl * (S - m) / (m * S)
    assert util.relerr(_host(d), _pair(want)) < 1e-5
    y, inv = ctx.softmax_fwd(_dev(z))
    n = np.sqrt((np.abs(Z) ** 2).sum(1, keepdims=True))
    assert util.relerr(_host(y), _pair(Z / n)) < 1e-6
    s = (G * np.conj(Z)).sum(1, keepdims=True).real
    assert util.relerr(_host(ctx.softmax_bwd(_dev(g), _dev(z), inv)), _pair(G / n - Z * s / n ** 3)) < 1e-5


def test_crossent_clamps_on_zero_row(ctx):
    """All-zero logits hit the 1e-15 clamps of the reference (impl/crossent.h:63-70, 88-90)."""
    import torch
    z = (np.zeros((2, 10), np.float32), np.zeros((2, 10), np.float32))
    loss, d = ctx.crossent(_dev(z), torch.zeros(2, dtype=torch.int32).cuda())
    assert np.allclose(loss.cpu().numpy(), -np.log(1e-15), rtol=1e-5)
    assert np.all(np.isfinite(d[0].cpu().numpy()))


def test_embedding_gather_scatter(ctx):
    import torch
    rng = np.random.default_rng(3)
    V, D, B, T = 50, 12, 9, 5
    table = _rand(rng, V, D)
    tok = rng.integers(0, V, (B, T)).astype(np.int32)
    tok[0, 3:] = -1
    tok[2, :] = 7                      # heavy duplicates
    out = _host(ctx.embed_fwd(_dev(table), torch.from_numpy(tok).cuda()))
    want = _c(table)[np.where(tok < 0, 0, tok)]
    want[tok < 0] = 0
    assert util.relerr(out, _pair(want.reshape(B, T * D))) == 0.0
    g = _rand(rng, B, T * D)
    dt = (torch.zeros(V, D).cuda(), torch.zeros(V, D).cuda())
    ctx.embed_bwd(_dev(g), torch.from_numpy(tok).cuda(), dt)
    acc = np.zeros((V, D), np.complex128)
    np.add.at(acc, tok[tok >= 0], _c(g).reshape(B, T, D)[tok >= 0])
    assert util.relerr(_host(dt), _pair(acc)) < 1e-6


def test_sgd_update(ctx):
    import torch
    rng = np.random.default_rng(5)
    for n in (1, 1023, 1 << 20):
        w = rng.standard_normal(n).astype(np.float32)
        g = rng.standard_normal(n).astype(np.float32)
        W, G = torch.from_numpy(w).cuda(), torch.from_numpy(g).cuda()
        ctx.sgd_update(W, G, 0.125)
        assert np.array_equal(W.cpu().numpy(), w - np.float32(0.125) * g)
        assert float(G.abs().max()) == 0.0


def test_sgd_update_with_weight_split(ctx):
    """The fused update leaves the operand split of the new weight, only inside the spans: hi = the weight cut to
    TF32, h16 = bf16(hi), l16 = bf16(weight - hi) (round to nearest even)."""
    import torch
    rng = np.random.default_rng(6)
    n = 1 << 16
    w = rng.standard_normal(n).astype(np.float32)
    g = rng.standard_normal(n).astype(np.float32)
    W, G = torch.from_numpy(w).cuda(), torch.from_numpy(g).cuda()
    spans = [(256, 4096), (8192, 1 << 15)]
    outs = [(torch.full((c,), 7.0, device="cuda"), torch.full((c,), 7.0, device="cuda", dtype=torch.bfloat16),
             torch.full((c,), 7.0, device="cuda", dtype=torch.bfloat16)) for _, c in spans]
    ctx.sgd_update_split(W, G, 0.25, [(b, c) + o for (b, c), o in zip(spans, outs)])
    want = w - np.float32(0.25) * g
    assert np.array_equal(W.cpu().numpy(), want)
    assert float(G.abs().max()) == 0.0
    for (b, c), (hi, h16, l16) in zip(spans, outs):
        x = torch.from_numpy(want[b:b + c])
        h = (x.view(torch.int32) & ~0x1FFF).view(torch.float32)
        assert torch.equal(hi.cpu(), h)
        assert torch.equal(h16.cpu(), h.to(torch.bfloat16))
        assert torch.equal(l16.cpu(), (x - h).to(torch.bfloat16))
        # together they give the weight back to 2^-18
        back = hi.cpu() + l16.cpu().float()
        assert float((back - x).abs().max() / x.abs().max()) < 2.0 ** -18


def test_bad_arguments_are_rejected_not_fatal(ctx):
    import ctypes as C
    from cnet_b200 import lib
    l = lib.load()
    assert l.cnb_gelu_fwd(ctx.h, None, None, None, None, 4, None) == -1
    assert b"gelu" in l.cnb_last_error()
    assert l.cnb_linear_fwd(ctx.h, C.c_void_p(256), C.c_void_p(256), C.c_void_p(256), C.c_void_p(256), None, None,
                            C.c_void_p(256), C.c_void_p(256), 0, 4, 4, None) == -1
    p = C.c_void_p()
    assert l.cnb_alloc(ctx.h, 1 << 40, C.byref(p)) == -2     # arena exhausted, reported not fatal
