"""Generates the full-width fixtures (width_*.npz) from the UNMODIFIED reference CPU path.

Run in the build container (needs the reference tree for `make -C oracle ref`):
    python tests/golden/make_width_golden.py [case ...]
Each case of tests/util.py:WIDTH_CASES is a benchmark configuration at its full layer widths.
The reference (oracle/_ref: ComplexNet::forward / backward(label) per sample, then update) runs the
first WIDTH_ROWS samples of the seeded benchmark batch; a full-width tensor has up to 33 M
elements, so the fixture keeps WIDTH_SAMPLES seeded entries of each (tests/util.py:sample_index):
per-sample losses, layer outputs and their dL/dz*, the weight gradients accumulated over those
samples and the weight change of one update.  A few minutes of CPU for the embedding net.
"""
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle import ref  # noqa: E402
import util  # noqa: E402

if __name__ == "__main__":
    assert ref.available(), "build oracle/_ref first: make -C oracle ref"
    ref.set_threads(os.cpu_count())
    for name in (sys.argv[1:] or util.WIDTH_CASES):
        t0 = time.time()
        rows = min(util.WIDTH_ROWS, util.WIDTH_CASES[name][2])
        out = util.run_width_case(ref.RefNet(), name, rows, record=2)
        path = os.path.join(util.GOLDEN_DIR, name + ".npz")
        np.savez_compressed(path, **out)
        print(name, len(out), "arrays", os.path.getsize(path) // 1024, "KiB, %.0f s" % (time.time() - t0))
