"""Shared helpers of the parity tests: named cases, running a case on any net
implementation (device net, numpy checker, compiled reference), error metrics."""
import os

import numpy as np

from cnet_b200 import configs

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# name -> (builder, builder kwargs, batch, input kind, sgd steps)
CASES = {
    "classifier_784": (configs.build_classifier, dict(n=784, m=10), 4, "image", 1),
    "classifier_100_train": (configs.build_classifier, dict(n=100, m=10), 3, "image", 3),
    "mixer_64x2": (configs.build_mixer, dict(n=64, blocks=2, m=10), 5, "normal", 1),
    "embed_lm_small": (configs.build_embed_lm, dict(tokens=4, vocab=32, dim=8, hidden=16), 6, None, 2),
    "linear_48x40": (configs.build_linear, dict(n_in=48, n_out=40), 7, "fanin", 1),
    # large enough for the tensor-core GEMM with cached operand splits (all dims >= 64), two updates
    "mixer_64x1_b64": (configs.build_mixer, dict(n=64, blocks=1, m=10), 64, "normal", 2),
    # the layers outside the benchmark configs (TriangFourier, CRelu, L2Out), trained with the reference's Adam
    "relu_tri_adam": (configs.build_relu_tri, dict(n=24, m=6), 5, "normal", 3),
}
ADAM_CASES = {"relu_tri_adam"}
ADAM_BETA = 0.9
LR = 0.01


def relerr(a, b):
    """Norm-relative error ||a-b|| / ||b|| over both planes of a (re, im) pair or one array."""
    if isinstance(a, tuple):
        a = np.concatenate([np.asarray(x, np.float64).ravel() for x in a])
        b = np.concatenate([np.asarray(x, np.float64).ravel() for x in b])
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def case_inputs(name):
    builder, kw, B, kind, steps = CASES[name]

    class _Shape:   # builds the spec without a backend
        def __init__(self):
            self.n = 0

        def add(self, *a, **k):
            self.n += 1
            return self.n
    spec = builder(_Shape(), **kw)
    weights = configs.init_weights(spec, seed=0)
    batches = []
    for s in range(steps):
        data, labels = configs.make_batch(spec, B, seed=0, step=s, kind=kind)
        if spec.tokens and s == 0:
            data = data.copy()
            data[0, -1] = -1          # one padded position (NO_TOKEN)
            data[1, 1] = data[1, 0]   # a duplicate token within a sample
        batches.append((data, labels))
    return spec, weights, batches


def run_case(net, name, post_alloc=None):
    """Runs the case on `net` (flat interface) and returns {key: array}."""
    builder, kw, B, kind, steps = CASES[name]
    spec = builder(net, **kw)
    _, weights, batches = case_inputs(name)
    for uid, (re, im) in weights.items():
        net.set_values(uid, re, im)
    if post_alloc:
        post_alloc(net, B)
        for uid, (re, im) in weights.items():
            net.set_values(uid, re, im)
    out = {}
    weight_uids = {u for u, _, _ in spec.weights}
    for s, (data, labels) in enumerate(batches):
        if spec.tokens:
            losses = net.run_batch(spec.main, tokens=data, labels=labels)
        else:
            losses = net.run_batch(spec.main, x=data, labels=labels)
        out["loss%d" % s] = np.asarray(losses, np.float64)
        if s == 0:
            for lname, uid in spec.layers.items():
                if lname == "ce":
                    continue
                if uid in weight_uids:
                    g = net.get_wgrad(uid)
                    out["wgrad_%s_re" % lname], out["wgrad_%s_im" % lname] = g
                if uid not in weight_uids or uid == spec.main:
                    try:
                        a = net.get_record(uid, 0)
                        g = net.get_record(uid, 1)
                    except Exception:      # tensor fused away on the device
                        continue
                    out["act_%s_re" % lname], out["act_%s_im" % lname] = a
                    out["gstar_%s_re" % lname], out["gstar_%s_im" % lname] = g
        if name in ADAM_CASES:
            net.adam(LR, B, ADAM_BETA, s)
        else:
            net.update(LR, B)
    for lname, uid in spec.layers.items():
        if uid in weight_uids:
            v = net.get_values(uid)
            out["final_%s_re" % lname], out["final_%s_im" % lname] = v
    return out


def load_golden(name):
    with np.load(os.path.join(GOLDEN_DIR, name + ".npz")) as z:
        return {k: z[k] for k in z.files}


def compare(got, want, tol_act, tol_grad, skip_missing=True, label=""):
    """Pairs (re, im) keys and checks the norm-relative error per tensor."""
    bad = []
    keys = sorted(k[:-3] for k in want if k.endswith("_re"))
    for k in keys:
        if k + "_re" not in got:
            assert skip_missing, "missing " + k
            continue
        e = relerr((got[k + "_re"], got[k + "_im"]), (want[k + "_re"], want[k + "_im"]))
        tol = tol_act if k.startswith("act_") else tol_grad
        if k.startswith("final_"):
            tol = tol_act
        if not e <= tol:
            bad.append((k, e, tol))
    for k in want:
        if k.startswith("loss") and k in got:
            e = relerr(got[k], want[k])
            if not e <= tol_act:
                bad.append((k, e, tol_act))
    assert not bad, "%s: tensors beyond tolerance: %s" % (label, bad)


# ----------------------------------------------------------------- benchmark widths
# The benchmark configurations at their full widths.  The reference CPU path does the first
# WIDTH_ROWS samples of the seeded batch (samples are independent, impl/cnet.h:366-411) and the
# fixtures keep WIDTH_SAMPLES seeded entries of every tensor; the device runs the whole batch
# (activations, per-sample dL/dz*) and a batch of those rows alone (accumulated weight gradients,
# post-update weights).
# name -> (builder, kwargs, benchmark batch, input kind)
WIDTH_CASES = {
    "width_classifier_784": (configs.build_classifier, dict(n=784, m=10), 64, "image"),
    "width_linear_4096": (configs.build_linear, dict(n_in=4096, n_out=4096), 4096, "fanin"),
    "width_mixer_1024x8": (configs.build_mixer, dict(n=1024, blocks=8, m=10), 512, "normal"),
    "width_embed_lm": (configs.build_embed_lm, dict(tokens=64, vocab=8192, dim=256, hidden=2048), 1024, None),
}
WIDTH_ROWS = 64
WIDTH_SAMPLES = 1024
# one update with a step large enough that the weight change is well above the fp32 rounding of the
# reference's own weights (at lr 0.01 the change is ~1e-6 of a weight of ~0.03)
WIDTH_LR = 1.0


def sample_index(key, size):
    """The seeded flat indices of tensor `key` kept by the width fixtures."""
    import zlib
    if size <= WIDTH_SAMPLES:
        return np.arange(size)
    r = np.random.Generator(np.random.Philox(key=[zlib.crc32(key.encode()), 4242]))
    return np.sort(r.integers(0, size, WIDTH_SAMPLES))


def _sampled(out, key, pair, rows=None):
    re, im = (np.asarray(p) for p in pair)
    if rows is not None:
        re, im = re[:rows], im[:rows]
    idx = sample_index(key, re.size)
    out[key + "_re"] = re.reshape(-1)[idx].astype(np.float32)
    out[key + "_im"] = im.reshape(-1)[idx].astype(np.float32)


def width_batch(name, rows=None):
    builder, kw, B, kind = WIDTH_CASES[name]

    class _Shape:
        def __init__(self):
            self.n = 0

        def add(self, *a, **k):
            self.n += 1
            return self.n
    spec = builder(_Shape(), **kw)
    data, labels = configs.make_batch(spec, B, seed=0, step=0, kind=kind)
    if rows is not None:
        data = data[:rows].copy() if spec.tokens else (data[0][:rows].copy(), data[1][:rows].copy())
        labels = labels[:rows].copy()
    return spec, data, labels


def run_width_case(net, name, batch, weights=None, alloc=None, record=True, train=True):
    """One step of a width case on `net` at `batch` rows (the first rows of the seeded benchmark
    batch); returns the sampled tensors of its first WIDTH_ROWS rows.  train: also the sampled
    weight gradients and the sampled weight change of one update (lr / batch)."""
    builder, kw, _, _ = WIDTH_CASES[name]
    spec = builder(net, **kw)
    if weights is None:
        weights = configs.init_weights(spec, seed=0)
    for uid, (re, im) in weights.items():
        net.set_values(uid, re, im)
    if alloc:
        alloc(net, batch)
    _, data, labels = width_batch(name, batch)
    rows = min(batch, WIDTH_ROWS)
    if spec.tokens:
        losses = net.run_batch(spec.main, tokens=data, labels=labels, record=record)
    else:
        losses = net.run_batch(spec.main, x=data, labels=labels, record=record)
    out = {"loss": np.asarray(losses, np.float64)[:rows]}
    weight_uids = {u for u, _, _ in spec.weights}
    for lname, uid in spec.layers.items():
        if lname == "ce" or (uid in weight_uids and uid != spec.main):
            continue
        for what, prefix in ((0, "act_"), (1, "gstar_")):
            try:
                t = net.get_record(uid, what)
            except Exception:      # tensor fused away on the device / not recorded
                continue
            _sampled(out, prefix + lname, t, rows)
    if train:
        for lname, uid in spec.layers.items():
            if uid in weight_uids:
                _sampled(out, "wgrad_" + lname, net.get_wgrad(uid))
        net.update(WIDTH_LR, batch)
        for lname, uid in spec.layers.items():
            if uid in weight_uids:
                v = net.get_values(uid)
                w0 = weights[uid]
                _sampled(out, "delta_" + lname, (v[0].astype(np.float64) - w0[0], v[1].astype(np.float64) - w0[1]))
    return out
