"""Generates the golden fixtures in this directory from the UNMODIFIED reference CPU path.

Run in the build container (needs the reference tree for `make -C oracle ref`):
    python tests/golden/make_golden.py
Every case in tests/util.py:CASES is run on oracle/_ref (ComplexNet::forward /
backward(label) / update per sample, exactly as the reference trainer loops) and its
losses, per-layer activations and dL/dz*, accumulated weight gradients and post-update
weights are stored as float32 .npz files.  Inputs are seeded (cnet_b200/configs.py).
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle import ref  # noqa: E402
import util  # noqa: E402

if __name__ == "__main__":
    assert ref.available(), "build oracle/_ref first: make -C oracle ref"
    for name in util.CASES:
        out = util.run_case(ref.RefNet(), name)
        path = os.path.join(util.GOLDEN_DIR, name + ".npz")
        np.savez_compressed(path, **{k: np.asarray(v, np.float32) if not k.startswith("loss") else v
                                     for k, v in out.items()})
        print(name, len(out), "arrays", os.path.getsize(path) // 1024, "KiB")
    # a checkpoint written by the reference's own ModelSaver (impl/model_saver.h:799-821)
    from cnet_b200 import configs
    net = ref.RefNet()
    spec = configs.build_embed_lm(net, tokens=4, vocab=32, dim=8, hidden=16)
    for uid, (re, im) in configs.init_weights(spec, 0).items():
        net.set_values(uid, re, im)
    net.save(os.path.join(util.GOLDEN_DIR, "embed_lm_small.cnet"))
