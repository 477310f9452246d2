"""Full benchmark sizes on the GPU, checked through size-independent properties (the CPU checkers
would need hours there): adjoint identities of the three Linear products, unitarity and inversion of
FourierTrans, additivity of the weight gradients over the batch (what data parallelism relies on)."""
import numpy as np
import pytest

from cnet_b200 import configs
from cnet_b200.net import Net

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    from cnet_b200.ops import Context
    c = Context(arena_bytes=3 << 30)
    yield c
    c.close()


def _rand(gen, *shape, scale=1.0):
    import torch
    return tuple(torch.randn(*shape, device="cuda", generator=gen) * scale for _ in range(2))


def _dot(a, b):
    """sum a * conj(b) in float64 (complex as a (re, im) pair)."""
    ar, ai, br, bi = a[0].double(), a[1].double(), b[0].double(), b[1].double()
    return complex(float((ar * br + ai * bi).sum()), float((ai * br - ar * bi).sum()))


@pytest.mark.parametrize("B,n_in,n_out", [(4096, 4096, 4096), (4096, 1024, 1024), (1024, 16384, 2048)])
def test_linear_adjoint_identities(ctx, B, n_in, n_out):
    """<dX*, X> = <dW*, W> = <G*, Y> for Y = X W^T, dX* = G* conj(W), dW* = G*^T conj(X)."""
    import torch
    gen = torch.Generator(device="cuda").manual_seed(B + n_in)
    x, w, g = _rand(gen, B, n_in, scale=n_in ** -0.5), _rand(gen, n_out, n_in, scale=n_in ** -0.5), _rand(gen, B, n_out)
    y = ctx.linear_fwd(x, w)
    assert ctx.last_gemm_engine() == 1
    ref = _dot(g, y)
    dx = ctx.linear_bwd_x(g, w)
    dw = ctx.linear_bwd_w(g, x)
    for got in (_dot(dx, x), _dot(dw, w)):
        assert abs(got - ref) / abs(ref) < 1e-4
    # linearity in X on a slice of rows: L(2x) - 2 L(x) = 0
    y2 = ctx.linear_fwd((2 * x[0], 2 * x[1]), w)
    err = float((y2[0] - 2 * y[0]).norm() / y2[0].norm())
    assert err < 1e-5
    # a sample of outputs against float64
    rows = slice(0, 4)
    want = (x[0][rows].double() + 1j * x[1][rows].double()) @ (w[0].double() + 1j * w[1].double()).T
    got = y[0][rows].double() + 1j * y[1][rows].double()
    assert float((got - want).norm() / want.norm()) < 1e-4


@pytest.mark.parametrize("B,N", [(4096, 1024), (64, 784), (512, 4096)])
def test_fourier_is_unitary_and_backward_inverts_it(ctx, B, N):
    import torch
    gen = torch.Generator(device="cuda").manual_seed(N)
    x = _rand(gen, B, N)
    y = ctx.dft_fwd(x)
    n_x = float((x[0].double() ** 2 + x[1].double() ** 2).sum())
    n_y = float((y[0].double() ** 2 + y[1].double() ** 2).sum())
    assert abs(n_y - n_x) / n_x < 1e-5                       # Parseval with the N^-1/2 scaling
    back = ctx.dft_bwd(y)                                    # conjugate transform = inverse
    err = float(((back[0] - x[0]).norm() ** 2 + (back[1] - x[1]).norm() ** 2) ** 0.5 / n_x ** 0.5)
    assert err < 1e-5


def test_weight_gradients_add_over_the_batch_at_full_size():
    """Token-mixing stack at the benchmark size: gradients of a 1024-sample batch equal the sum of
    the gradients of its two halves (same weights, no update in between)."""
    kw = dict(n=1024, blocks=8, m=10)
    B = 1024
    net = Net()
    spec = configs.build_mixer(net, **kw)
    for uid, (re, im) in configs.init_weights(spec, 0).items():
        net.set_values(uid, re, im)
    net.allocate(B)
    (xr, xi), labels = configs.make_batch(spec, B, 0)
    loss_full = net.run_batch(spec.main, x=(xr, xi), labels=labels)
    names = ("w0", "h3", "w7", "wh")
    full = {k: net.get_wgrad(spec.layers[k]) for k in names}
    net.update(0.0, 1)                                       # lr 0: only clears the gradients
    h = B // 2
    l0 = net.run_batch(spec.main, x=(xr[:h].copy(), xi[:h].copy()), labels=labels[:h].copy())
    l1 = net.run_batch(spec.main, x=(xr[h:].copy(), xi[h:].copy()), labels=labels[h:].copy())
    assert np.allclose(np.concatenate([l0, l1]), loss_full, rtol=1e-5)
    assert np.all(np.isfinite(loss_full)) and 0.5 < loss_full.mean() < 10
    for k in names:
        got = net.get_wgrad(spec.layers[k])                  # accumulated over the two halves
        num = np.sqrt(((got[0] - full[k][0]) ** 2).sum() + ((got[1] - full[k][1]) ** 2).sum())
        den = np.sqrt((full[k][0] ** 2).sum() + (full[k][1] ** 2).sum())
        assert num / den < 1e-4, k


@pytest.mark.parametrize("B", [512, 1024])
def test_small_batch_step_runs_at_the_expected_order_of_speed(B):
    """Schedules of the tensor-core products are chosen per launch from the shape and the SMs a launch may fill; a
    wrong count there (one CTA pair for a whole product) passes every numerical test and costs a factor of nine.
    A step of the 8-block stack takes 0.8 ms at 512 rows and 1.2 ms at 1024: a loose bound catches the factor."""
    import time
    import torch
    kw = dict(n=1024, blocks=8, m=10)
    net = Net()
    spec = configs.build_mixer(net, **kw)
    for uid, (re, im) in configs.init_weights(spec, 0).items():
        net.set_values(uid, re, im)
    net.allocate(B)
    (xr, xi), labels = configs.make_batch(spec, B, 0)
    for _ in range(3):
        net.run_batch(spec.main, x=(xr, xi), labels=labels)
        net.update(0.01, B)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    steps = 10
    for _ in range(steps):
        net.run_batch(spec.main, x=(xr, xi), labels=labels)
        net.update(0.01, B)
    torch.cuda.synchronize()
    ms = 1e3 * (time.perf_counter() - t0) / steps
    # run_batch also uploads the batch and reads the losses back (a few hundred microseconds)
    assert ms < 5.0, "a %d-row step took %.2f ms" % (B, ms)
