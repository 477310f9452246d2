"""GPU parity of whole training steps: the device net (through the host facade and the
C ABI) against the float64 restatement and against the fixtures produced by the
unmodified reference CPU path.  Tolerances (norm-relative per tensor): 1e-4 on
activations, losses and post-update weights, 1e-3 on gradients."""
import numpy as np
import pytest

import util
from cnet_b200 import configs
from cnet_b200.net import Net
from oracle import cnet_oracle

pytestmark = pytest.mark.gpu

TOL_ACT, TOL_GRAD = 1e-4, 1e-3
# The reference's own fp32 Bluestein FFT is ~1e-4 off an exact DFT at these lengths, so
# against its fixtures the activation bound is its error plus ours.
GOLDEN_ACT = {"classifier_784": 3e-4, "classifier_100_train": 3e-4}


def _device_case(name, fuse):
    return util.run_case(Net(), name, post_alloc=lambda n, B: n.allocate(B, fuse=fuse))


@pytest.mark.parametrize("fuse", [False, True])
@pytest.mark.parametrize("name", sorted(util.CASES))
def test_step_matches_restatement_and_reference(name, fuse):
    got = _device_case(name, fuse)
    want = util.run_case(cnet_oracle.OracleNet(), name)
    util.compare(got, want, TOL_ACT, TOL_GRAD, label=name + " vs float64 restatement")
    golden = util.load_golden(name)
    util.compare(got, golden, GOLDEN_ACT.get(name, TOL_ACT), TOL_GRAD, label=name + " vs reference fixture")


def test_fused_and_unfused_agree():
    a = _device_case("mixer_64x2", False)
    b = _device_case("mixer_64x2", True)
    util.compare(b, a, 1e-5, 1e-5, label="fused vs unfused")


def test_gradients_accumulate_until_update():
    """Two backward passes without an update sum the weight gradients (impl/cinput.h:54-65)."""
    net = Net()
    spec = configs.build_classifier(net, n=64, m=10)
    for uid, (re, im) in configs.init_weights(spec, 0).items():
        net.set_values(uid, re, im)
    net.allocate(8)
    x, labels = configs.make_batch(spec, 8, 0)
    net.run_batch(spec.main, x=x, labels=labels)
    g1 = net.get_wgrad(spec.layers["w"])
    net.run_batch(spec.main, x=x, labels=labels)
    g2 = net.get_wgrad(spec.layers["w"])
    assert util.relerr(g2, (2 * g1[0], 2 * g1[1])) < 1e-6
    net.update(0.01, 8)
    g3 = net.get_wgrad(spec.layers["w"])
    assert np.all(g3[0] == 0) and np.all(g3[1] == 0)


def test_partial_batch_and_batch_of_one():
    net = Net()
    spec = configs.build_mixer(net, n=32, blocks=1, m=10)
    w = configs.init_weights(spec, 0)
    for uid, (re, im) in w.items():
        net.set_values(uid, re, im)
    net.allocate(6)
    x, labels = configs.make_batch(spec, 6, 0)
    ora = cnet_oracle.OracleNet()
    ospec = configs.build_mixer(ora, n=32, blocks=1, m=10)
    for uid, (re, im) in w.items():
        ora.set_values(uid, re, im)
    for B in (1, 5):
        xs = (x[0][:B].copy(), x[1][:B].copy())
        got = net.run_batch(spec.main, x=xs, labels=labels[:B].copy())
        want = ora.run_batch(ospec.main, x=xs, labels=labels[:B])
        assert got.shape == (B,)
        assert util.relerr(got, want) < TOL_ACT
        net.update(0.0, 1)


def test_oversized_batch_is_rejected():
    from cnet_b200.lib import CnetError
    net = Net()
    spec = configs.build_classifier(net, n=16, m=4)
    net.init_inputs(1)
    net.allocate(2)
    x, labels = configs.make_batch(spec, 3, 0)
    with pytest.raises(CnetError, match="exceeds"):
        net.upload(x=x, labels=labels)


def test_loss_curve_follows_reference_training():
    """100-step SGD on the classifier shape (reduced width so the CPU checker is quick):
    the device loss curve tracks the float64 restatement."""
    n, m, B, steps = 196, 10, 16, 30
    dev, ora = Net(), cnet_oracle.OracleNet()
    sd, so = configs.build_classifier(dev, n=n, m=m), configs.build_classifier(ora, n=n, m=m)
    w = configs.init_weights(sd, 0)
    for uid, (re, im) in w.items():
        dev.set_values(uid, re, im)
        ora.set_values(uid, re, im)
    dev.allocate(B)
    ld, lo = [], []
    for s in range(steps):
        x, labels = configs.make_batch(sd, B, 0, step=s)
        ld.append(dev.run_batch(sd.main, x=x, labels=labels).mean())
        lo.append(ora.run_batch(so.main, x=x, labels=labels).mean())
        dev.update(0.5, B)
        ora.update(0.5, B)
    assert util.relerr(np.array(ld), np.array(lo)) < 1e-4
    assert ld[-1] < ld[0]


def test_graph_replay_matches_eager_steps():
    """The captured CUDA graph of a step gives the same losses and weights as eager launches."""
    import torch
    from cnet_b200.dp import DataParallelTrainer
    kw = dict(n=256, blocks=2, m=10)
    runs = []
    for use_graph in (False, True):
        tr = DataParallelTrainer(configs.build_mixer, kw, global_batch=32, lr=0.5, device=0, seed=0)
        losses = []
        for s in range(5):
            (xr, xi), labels = configs.make_batch(tr.spec, 32, 0, step=s)
            if use_graph and s == 1:
                tr.capture()
            losses.append(tr.step((xr, xi), labels).mean())
        torch.cuda.synchronize()
        runs.append((np.array(losses), tr.net.get_values(tr.spec.layers["w0"])))
    assert util.relerr(runs[1][0], runs[0][0]) < 1e-5
    assert util.relerr(runs[1][1], runs[0][1]) < 1e-5


def test_input_pipeline_matches_plain_uploads():
    """prefetch / commit / async loss read-back give the same training run as synchronous uploads."""
    import torch
    from cnet_b200.dp import DataParallelTrainer
    kw = dict(n=128, blocks=1, m=10)
    B, steps = 64, 5
    batches = []
    runs = []
    for pipelined in (False, True):
        tr = DataParallelTrainer(configs.build_mixer, kw, global_batch=B, lr=0.5, device=0, seed=0)
        if not batches:
            for s in range(steps):
                (xr, xi), labels = configs.make_batch(tr.spec, B, 0, step=s)
                batches.append(((torch.from_numpy(xr).pin_memory(), torch.from_numpy(xi).pin_memory()),
                                torch.from_numpy(labels).pin_memory()))
        losses = []
        if pipelined:
            outs = [torch.empty(B).pin_memory() for _ in range(steps)]
            tr.prefetch(*batches[0])
            for s in range(steps):
                nxt = batches[s + 1] if s + 1 < steps else (None, None)
                tr.step_pipelined(nxt[0], nxt[1], outs[s])
            tr.net.wait_losses()
            losses = [float(o.mean()) for o in outs]
        else:
            for s in range(steps):
                losses.append(float(tr.step(*batches[s]).mean()))
        torch.cuda.synchronize()
        runs.append((np.array(losses), tr.net.get_values(tr.spec.layers["w0"])))
    assert util.relerr(runs[1][0], runs[0][0]) < 1e-6
    assert util.relerr(runs[1][1], runs[0][1]) < 1e-6


def test_restored_checkpoint_trains_on_the_device(tmp_path):
    """A checkpoint written by the reference loads, runs on the GPU like the restatement, and the weights
    saved after an update are the device's."""
    import os
    path = os.path.join(util.GOLDEN_DIR, "embed_lm_small.cnet")
    dev = Net.restore(path)
    ora = cnet_oracle.OracleNet()
    spec = configs.build_embed_lm(ora, tokens=4, vocab=32, dim=8, hidden=16)
    for uid, (re, im) in configs.init_weights(spec, 0).items():
        ora.set_values(uid, re, im)
    dev.allocate(6)
    tok, labels = configs.make_batch(spec, 6, 0)
    ld = dev.run_batch(spec.main, tokens=tok, labels=labels)
    lo = ora.run_batch(spec.main, tokens=tok, labels=labels)
    assert util.relerr(ld, lo) < 1e-4
    dev.update(0.01, 6)
    ora.update(0.01, 6)
    out = tmp_path / "trained.cnet"
    dev.save(out)
    again = Net.restore(out)
    for name in ("emb", "w1", "w2"):
        assert util.relerr(again.get_values(spec.layers[name]), ora.get_values(spec.layers[name])) < 1e-4


def test_infer_gives_the_losses_without_touching_gradients():
    net = Net()
    spec = configs.build_classifier(net, n=64, m=10)
    for uid, (re, im) in configs.init_weights(spec, 0).items():
        net.set_values(uid, re, im)
    net.allocate(8)
    x, labels = configs.make_batch(spec, 8, 0)
    want = net.run_batch(spec.main, x=x, labels=labels)
    g1 = net.get_wgrad(spec.layers["w"])
    gs1 = net.get_record(spec.layers["lin"], 1)
    net.upload(x=(x[0] * 0 + 1, x[1]), labels=labels)      # a different batch ...
    net.infer()                                            # ... forward only
    net.sync()
    assert not np.allclose(net.losses(), want)
    assert np.array_equal(net.get_record(spec.layers["lin"], 1)[0], gs1[0])   # seed of the last backward untouched
    assert np.array_equal(net.get_wgrad(spec.layers["w"])[0], g1[0])


def test_stale_graph_replay_is_refused():
    """What a captured step froze (row count, 'weights already split', Adam's step count) is checked at
    replay: a different batch, weights set from the host, or a captured adamUpdate fail with a message."""
    import torch
    from cnet_b200.dp import DataParallelTrainer
    from cnet_b200.lib import CnetError
    tr = DataParallelTrainer(configs.build_mixer, dict(n=128, blocks=1, m=10), global_batch=32, lr=0.5, device=0, seed=0)
    (xr, xi), labels = configs.make_batch(tr.spec, 32, 0)
    tr.step((xr, xi), labels)
    tr.capture()
    tr.step((xr, xi), labels)                              # replay at the captured batch: fine
    tr.net.upload(x=(xr[:16].copy(), xi[:16].copy()), labels=labels[:16].copy())
    with pytest.raises(CnetError, match="sized for 32"):
        tr.net.graph_launch()
    tr.net.upload(x=(xr, xi), labels=labels)
    tr.net.graph_launch()
    w = tr.net.get_values(tr.spec.layers["w0"])
    tr.net.set_values(tr.spec.layers["w0"], w[0], w[1])
    with pytest.raises(CnetError, match="set from the host"):
        tr.net.graph_launch()
    tr.capture()                                           # a fresh capture clears it
    tr.net.graph_launch()
    tr.net.capture_begin()
    with pytest.raises(CnetError, match="adamUpdate"):
        tr.net.adam_update(0.1, 0.9, 0)
    tr.net.capture_end()
    torch.cuda.synchronize()


def test_second_backward_before_update_is_refused_when_gradients_are_reduced_in_place():
    from cnet_b200.lib import CnetError
    net = Net()
    spec = configs.build_classifier(net, n=64, m=10)
    for uid, (re, im) in configs.init_weights(spec, 0).items():
        net.set_values(uid, re, im)
    net.allocate(8)
    seen = []
    net.set_bucket_hook(lambda ptr, count, b, nb: seen.append((b, nb)) or 0)
    x, labels = configs.make_batch(spec, 8, 0)
    net.run_batch(spec.main, x=x, labels=labels)
    assert seen and seen[-1][0] == seen[-1][1] - 1
    with pytest.raises(CnetError, match="second backward"):
        net.run_batch(spec.main, x=x, labels=labels)
    net.update(0.01, 8)
    net.run_batch(spec.main, x=x, labels=labels)           # after the update the next step is fine
