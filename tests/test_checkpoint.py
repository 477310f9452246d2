"""Checkpoint interop with the reference's ModelSaver byte format (impl/model_saver.h): files written
by the reference load here and files written here load in the reference.  CPU only (no GPU needed:
weights not yet on a device are saved from the host copies)."""
import os

import numpy as np
import pytest

import util
from cnet_b200 import configs
from cnet_b200.net import Net
from oracle import ref

FIXTURE = os.path.join(util.GOLDEN_DIR, "embed_lm_small.cnet")     # written by the reference (make_golden.py)


def _small_nets():
    return [(configs.build_classifier, dict(n=16, m=4)),
            (configs.build_mixer, dict(n=8, blocks=2, m=3)),
            (configs.build_embed_lm, dict(tokens=4, vocab=32, dim=8, hidden=16)),
            (configs.build_relu_tri, dict(n=12, m=3))]


def test_restore_reference_written_fixture(built_lib, tmp_path):
    net = Net.restore(FIXTURE)
    shape = Net()
    spec = configs.build_embed_lm(shape, tokens=4, vocab=32, dim=8, hidden=16)
    assert net.uids() == shape.uids()
    assert [net.type_of(u) for u in net.uids()] == [shape.type_of(u) for u in shape.uids()]
    assert [net.out_size(u) for u in net.uids()] == [shape.out_size(u) for u in shape.uids()]
    w = configs.init_weights(spec, 0)
    for uid, (re, im) in w.items():
        got = net.get_values(uid)
        assert np.array_equal(got[0], re) and np.array_equal(got[1], im)
    # writing it back reproduces the reference's bytes exactly
    out = tmp_path / "again.cnet"
    net.save(out)
    assert open(out, "rb").read() == open(FIXTURE, "rb").read()


@pytest.mark.skipif(not ref.available(), reason="oracle/_ref not built")
@pytest.mark.parametrize("k", range(4))
def test_round_trip_with_live_reference(built_lib, tmp_path, k):
    builder, kw = _small_nets()[k]
    ours, theirs = Net(), ref.RefNet()
    spec = builder(ours, **kw)
    builder(theirs, **kw)
    for uid, (re, im) in configs.init_weights(spec, 3).items():
        ours.set_values(uid, re, im)
        theirs.set_values(uid, re, im)
    a, b = tmp_path / "ours.cnet", tmp_path / "ref.cnet"
    ours.save(a)
    theirs.save(b)
    assert open(a, "rb").read() == open(b, "rb").read()            # same bytes
    back = ref.RefNet.restore(a)                                    # the reference loads our file ...
    assert back.uids() == theirs.uids()
    for uid, (re, im) in configs.init_weights(spec, 3).items():
        got = back.get_values(uid)
        assert np.array_equal(got[0], re) and np.array_equal(got[1], im)
    # ... and trains on it exactly like the net it was built from
    data, labels = configs.make_batch(spec, 3, 0)
    kwargs = dict(tokens=data) if spec.tokens else dict(x=data)
    l1 = theirs.run_batch(spec.main, labels=labels, **kwargs)
    l2 = back.run_batch(spec.main, labels=labels, **kwargs)
    assert np.array_equal(l1, l2)


def test_restore_rejects_garbage(built_lib, tmp_path):
    from cnet_b200.lib import CnetError
    p = tmp_path / "bad.cnet"
    p.write_bytes(b"\x00\x01\x02\x03 not a checkpoint")
    with pytest.raises(CnetError, match="magic"):
        Net.restore(p)
    good = open(FIXTURE, "rb").read()
    p.write_bytes(good[:len(good) // 2])                            # truncated file
    with pytest.raises(CnetError, match="truncated"):
        Net.restore(p)
    with pytest.raises(CnetError):
        Net.restore(tmp_path / "missing.cnet")


def test_restore_rejects_corrupt_lengths(built_lib, tmp_path):
    """Lengths come from the file: negative or absurd ones must be refused with a message, not sized."""
    import struct
    from cnet_b200.lib import CnetError
    good = bytearray(open(FIXTURE, "rb").read())
    # first record: magic | type | uid | input length | out size | #producers | dim | tokens | vocab
    for field, value in ((3, -5), (3, 0x7FFFFFF0), (4, -1), (2, -7), (6, -8), (8, 0x7FFFFFF0)):
        bad = bytearray(good)
        bad[4 * field:4 * field + 4] = struct.pack(">i", value)
        p = tmp_path / ("bad_%d_%d.cnet" % (field, value & 0xFFFF))
        p.write_bytes(bytes(bad))
        with pytest.raises(CnetError, match="corrupt|truncated"):
            Net.restore(p)
