"""The arithmetic of the split product, restated in numpy (no GPU): x = hi + lo with hi = x cut to TF32 and
lo = x - hi; a product is hi.hi (exact in fp32) plus the cross terms from the bf16 roundings of hi and lo.
Checks the error budget the kernel's header states: per product about 2^-17 of |x y| in the worst case (2^-19.5
rms), and the
norm-relative error of a K = 1024 dot product around 1e-6 (fp64 accumulation here: what the operand rounding
alone costs, without the tensor core's accumulator truncation)."""
import numpy as np


def _tf32_hi(x):
    return (x.view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)


def _bf16(x):
    """round to nearest even to bfloat16, returned as float32"""
    b = x.astype(np.float32).view(np.uint32).astype(np.uint64)
    r = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32)


def _split(x):
    hi = _tf32_hi(x)
    lo = (x - hi).astype(np.float32)
    assert np.array_equal((hi.astype(np.float64) + lo.astype(np.float64)).astype(np.float32), x)     # the split is exact
    return hi, _bf16(hi), _bf16(lo)


def test_per_product_error_bound():
    rng = np.random.default_rng(0)
    x = (rng.standard_normal(1 << 16) * np.exp(rng.uniform(-20, 20, 1 << 16))).astype(np.float32)
    y = (rng.standard_normal(1 << 16) * np.exp(rng.uniform(-20, 20, 1 << 16))).astype(np.float32)
    xh, xh16, xl16 = _split(x)
    yh, yh16, yl16 = _split(y)
    got = xh.astype(np.float64) * yh + xh16.astype(np.float64) * yl16 + xl16.astype(np.float64) * yh16
    want = x.astype(np.float64) * y
    rel = np.abs(got - want) / np.abs(want)
    assert rel.max() < 2.0 ** -17 + 2.0 ** -19       # two cross terms at 2^-18 each, plus the dropped lo.lo
    assert np.sqrt((rel ** 2).mean()) < 2.0 ** -19


def test_dot_products_of_length_1024_keep_fp32_accuracy():
    rng = np.random.default_rng(1)
    A = rng.standard_normal((64, 1024)).astype(np.float32)
    B = rng.standard_normal((48, 1024)).astype(np.float32)
    ah, ah16, al16 = _split(A)
    bh, bh16, bl16 = _split(B)
    f = np.float64
    got = ah.astype(f) @ bh.astype(f).T + ah16.astype(f) @ bl16.astype(f).T + al16.astype(f) @ bh16.astype(f).T
    want = A.astype(f) @ B.astype(f).T
    err = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert err < 2e-6, err
    # the all-TF32 form (lo kept in fp32, rounded to TF32 by the tensor core) for comparison: a few 1e-7
    al = _tf32_hi((A - ah).astype(np.float32))
    bl = _tf32_hi((B - bh).astype(np.float32))
    ref = ah.astype(f) @ bh.astype(f).T + ah.astype(f) @ bl.astype(f).T + al.astype(f) @ bh.astype(f).T
    assert np.linalg.norm(ref - want) / np.linalg.norm(want) < err
