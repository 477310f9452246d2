"""GPU parity at the benchmark widths against the reference itself.

The fixtures tests/golden/width_*.npz hold what the unmodified reference CPU path computed for
the first 64 samples of each benchmark configuration's seeded batch (seeded entries of every
tensor, made by tests/golden/make_width_golden.py).  The device net runs
  * the whole benchmark batch (config 2: 4096, config 3/5: 512, config 4: 1024, config 1: 64) and
    its first 64 rows are compared: per-sample losses, layer outputs, per-sample dL/dz*;
  * a batch of those 64 rows alone (still on the tensor-core path): accumulated weight dL/dz* and
    the weight change of one update.
Tolerances (norm-relative over the kept entries): 1e-4 losses and activations, 1e-3 gradients and
weight changes; 3e-4 on activations of the 784-point net, where the reference's own fp32 Bluestein
FFT is ~1e-4 away from an exact DFT.
"""
import numpy as np
import pytest

import util
from cnet_b200.net import Net

pytestmark = pytest.mark.gpu

ACT_TOL = {"width_classifier_784": 3e-4}


def _compare(got, want, act_tol, label, need=()):
    bad, seen = [], set()
    for k in sorted(k[:-3] for k in want if k.endswith("_re")):
        if k + "_re" not in got:
            continue
        seen.add(k)
        e = util.relerr((got[k + "_re"], got[k + "_im"]), (want[k + "_re"], want[k + "_im"]))
        tol = act_tol if k.startswith("act_") else 1e-3
        if not e <= tol:
            bad.append((k, e, tol))
    e = util.relerr(got["loss"], want["loss"])
    if not e <= act_tol:
        bad.append(("loss", e, act_tol))
    assert not bad, "%s: beyond tolerance: %s" % (label, bad)
    missing = [k for k in need if k not in seen]
    assert not missing, "%s: tensors not compared: %s" % (label, missing)
    return seen


# tensors every run must have compared (the rest depends on what the fused kernels materialise)
NEED_FULL = {
    "width_classifier_784": ["act_ft", "act_lin", "gstar_lin", "gstar_ft"],
    "width_linear_4096": ["act_lin", "gstar_x", "gstar_lin"],
    "width_mixer_1024x8": ["act_ft0", "act_gelu7", "act_res7", "act_head", "gstar_x", "gstar_ft0", "gstar_ft7"],
    "width_embed_lm": ["act_emb", "act_l1", "act_l2", "act_sm", "gstar_emb", "gstar_l1", "gstar_sm"],
}
NEED_TRAIN = {
    "width_classifier_784": ["wgrad_h", "wgrad_w", "delta_h", "delta_w"],
    "width_linear_4096": ["wgrad_w", "delta_w"],
    "width_mixer_1024x8": ["wgrad_h0", "wgrad_w0", "wgrad_w7", "wgrad_wh", "delta_w3", "delta_h7"],
    "width_embed_lm": ["wgrad_emb", "wgrad_w1", "wgrad_w2", "delta_emb", "delta_w1", "delta_w2"],
}


@pytest.mark.parametrize("fuse", [True, False])
@pytest.mark.parametrize("name", sorted(util.WIDTH_CASES))
def test_benchmark_batch_matches_reference_rows(name, fuse):
    if not fuse and name in ("width_linear_4096", "width_embed_lm"):
        pytest.skip("no fusible layers in this net")
    want = util.load_golden(name)
    batch = util.WIDTH_CASES[name][2]
    got = util.run_width_case(Net(), name, batch, alloc=lambda n, B: n.allocate(B, fuse=fuse), train=False)
    _compare(got, want, ACT_TOL.get(name, 1e-4), "%s at batch %d" % (name, batch), NEED_FULL[name])


@pytest.mark.parametrize("name", sorted(util.WIDTH_CASES))
def test_weight_gradients_and_update_match_reference(name):
    want = util.load_golden(name)
    got = util.run_width_case(Net(), name, util.WIDTH_ROWS, alloc=lambda n, B: n.allocate(B))
    _compare(got, want, ACT_TOL.get(name, 1e-4), name + " at batch 64", NEED_TRAIN[name])
