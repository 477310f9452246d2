"""MnistDataReader against idx files written by the test (the MNIST files themselves are not available offline):
format and quirks of the reference's reader (data/data.h:82-165): headers skipped, a pixel byte taken as a signed
char, real = imaginary = pixel, batches wrap around."""
import struct

import numpy as np
import pytest

from cnet_b200.data import MnistDataReader
from cnet_b200.lib import CnetError


def _write_idx(tmp_path, n, seed=0):
    r = np.random.default_rng(seed)
    pixels = r.integers(0, 256, (n, 28, 28), dtype=np.uint8)
    labels = r.integers(0, 10, n, dtype=np.uint8)
    img, lab = tmp_path / "images.idx3-ubyte", tmp_path / "labels.idx1-ubyte"
    img.write_bytes(struct.pack(">iiii", 2051, n, 28, 28) + pixels.tobytes())
    lab.write_bytes(struct.pack(">ii", 2049, n) + labels.tobytes())
    return img, lab, pixels, labels


def test_reads_idx_files_like_the_reference(built_lib, tmp_path):
    img, lab, pixels, labels = _write_idx(tmp_path, 37)
    rd = MnistDataReader(img, lab, 37)
    assert rd.size() == 37 and rd.has_next_batch(37) and not rd.has_next_batch(38)
    (re, im), got = rd.next_batch(16)
    want = pixels[:16].reshape(16, 784).astype(np.int8).astype(np.float32)     # signed char, as in the reference
    assert np.array_equal(re, want) and np.array_equal(im, want)
    assert np.array_equal(got, labels[:16].astype(np.int32))
    assert want.min() < 0                                                       # bytes above 127 come out negative
    rd.next_batch(16)
    (re, _), got = rd.next_batch(16)                                            # rows 32..36, then 0..10: wraps around
    idx = np.arange(32, 48) % 37
    assert np.array_equal(re, pixels[idx].reshape(16, 784).astype(np.int8).astype(np.float32))
    assert np.array_equal(got, labels[idx].astype(np.int32))


def test_short_or_missing_files_are_refused(built_lib, tmp_path):
    img, lab, _, _ = _write_idx(tmp_path, 5)
    with pytest.raises(CnetError):
        MnistDataReader(img, lab, 6)                                            # fewer images than asked for
    with pytest.raises(CnetError):
        MnistDataReader(tmp_path / "none", lab, 5)


def test_shuffle_keeps_samples_and_labels_together(built_lib, tmp_path):
    img, lab, pixels, labels = _write_idx(tmp_path, 20, seed=3)
    rd = MnistDataReader(img, lab, 20)
    rd.shuffle(7)
    (re, _), got = rd.next_batch(20)
    flat = pixels.reshape(20, 784).astype(np.int8).astype(np.float32)
    order = [int(np.where((flat == row).all(1))[0][0]) for row in re]
    assert sorted(order) == list(range(20)) and order != list(range(20))
    assert np.array_equal(got, labels[order].astype(np.int32))
