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
