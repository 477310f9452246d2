"""The schedule of the tensor-core products (cnb_gemm_schedule: host arithmetic, no GPU): at the shapes of the
benchmark configurations, on a whole device, beside a collective and on half a device, a product must spread over
most of the SMs it may fill.  A mis-counted schedule (one CTA pair for a whole product) passes every numerical
test and costs a factor of nine."""
import ctypes as C

import pytest

from cnet_b200 import lib as L

SMS = 148
# (M, N, K, accumulate): forward / dX* / dW* of the 1024-wide mixer at the per-GPU batches of 1, 2, 4, 8 GPUs,
# config 2 (4096^3), both layers of config 4
SHAPES = [(B, 1024, 1024, 0) for B in (4096, 2048, 1024, 512)] + [(1024, 1024, B, 1) for B in (4096, 2048, 1024, 512)] + \
         [(4096, 4096, 4096, 0), (1024, 2048, 16384, 0), (1024, 8192, 2048, 0), (2048, 16384, 1024, 1), (1024, 16384, 2048, 0)]
# sm_limit: the whole device, 6 / 8 SMs set aside for a collective, half a device, half of what a collective leaves
LIMITS = [0, 142, 140, 74, 71, 70]


def _schedule(lib, M, N, K, acc, limit):
    out = (C.c_int * 8)()
    assert lib.cnb_gemm_schedule(M, N, K, acc, SMS, limit, out) == 0
    keys = ("pair", "ctas", "cluster_ctas", "run", "whole_per_cta", "segments", "atomics", "clear_from_row")
    return dict(zip(keys, out))


@pytest.fixture(scope="module")
def lib():
    return L.load()


@pytest.mark.parametrize("limit", LIMITS)
@pytest.mark.parametrize("M,N,K,acc", SHAPES)
def test_products_fill_the_sms_they_may_use(lib, M, N, K, acc, limit):
    s = _schedule(lib, M, N, K, acc, limit)
    may_use = limit if limit > 0 else SMS
    tiles = -(-M // 128) * -(-N // 128)
    k_blocks = -(-K // 16)
    # never more CTAs in flight per wave than allowed, unless the schedule is whole tiles in several waves
    if s["whole_per_cta"] == 0 and s["segments"] == 0 and s["ctas"] > may_use:
        assert s["ctas"] in (tiles, 2 * -(-M // 256) * -(-N // 128)), s
    # enough parallelism: at least 40 % of the SMs it may use, or one CTA per tile-and-k-slice when the product is small
    assert s["ctas"] >= min(0.4 * may_use, tiles * max(1, k_blocks // 8) * 0.4), (s, may_use)
    assert s["cluster_ctas"] in (1, 2, 4, 8)
    if s["pair"]:
        assert s["ctas"] % 2 == 0 and s["cluster_ctas"] in (2, 4) and M >= 256
    if s["cluster_ctas"] > (2 if s["pair"] else 1):
        assert not s["atomics"]                          # K-split clusters sum through shared memory
    if s["segments"]:
        assert k_blocks > 256 and s["run"] <= 64         # capped accumulation chains


def test_bench_shapes_take_cta_pairs_on_a_whole_device(lib):
    for M, N, K, acc in [(4096, 1024, 1024, 0), (1024, 1024, 4096, 1), (4096, 4096, 4096, 0)]:
        s = _schedule(lib, M, N, K, acc, 0)
        assert s["pair"] and s["ctas"] >= 128 and s["cluster_ctas"] == 2, s
    s = _schedule(lib, 512, 1024, 1024, 0, 0)              # 512 rows: one CTA per tile, clusters of 4 along K
    assert not s["pair"] and s["ctas"] == 128 and s["cluster_ctas"] == 4, s
    s = _schedule(lib, 1024, 1024, 1024, 0, 142)           # 1024 rows beside a collective: two pairs per tile
    assert s["pair"] and s["ctas"] == 128 and s["cluster_ctas"] == 4, s
    s = _schedule(lib, 1024, 1024, 1024, 1, 71)            # half a device beside a collective: no pairs
    assert not s["pair"], s


def test_small_and_ragged_products(lib):
    s = _schedule(lib, 64, 784, 784, 0, 0)                 # the classifier's DFT as a product: 7 tiles, clusters of 8 along K
    assert not s["pair"] and s["cluster_ctas"] == 8 and s["ctas"] == 56, s
    s = _schedule(lib, 2500, 1064, 520, 0, 0)              # ragged M / N / K: pairs cover the last 256-row tile partly
    assert s["pair"] and s["ctas"] % 2 == 0 and s["ctas"] <= 148, s
    s = _schedule(lib, 300, 1024, 1024, 0, 0)              # 16 pair tiles cannot fill the device with two pairs each
    assert not s["pair"] and s["ctas"] >= 96, s
    s = _schedule(lib, 1024, 2048, 16384, 0, 0)            # K > 4096: chains capped at 64 k-blocks, segment-major
    assert s["segments"] == 16 and s["run"] == 64 and s["atomics"], s
    for bad in ((0, 8, 8), (8, 0, 8), (8, 8, 0)):
        out = (C.c_int * 8)()
        assert lib.cnb_gemm_schedule(bad[0], bad[1], bad[2], 0, SMS, 0, out) != 0
