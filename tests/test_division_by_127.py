"""The encoders derive scale = max / 127 with q0 = m*r, e = fma(-127, q0, m),
q = fma(e, r, q0), r = fl(1/127), instead of an IEEE division.  This checks,
for every binary32 significand, that the sequence returns the correctly
rounded quotient; a power-of-two scaling carries it to every exponent inside
the range the kernels accept."""
import numpy as np


def test_fma_sequence_equals_ieee_division_for_every_significand():
    bits = np.arange(0x3F800000, 0x40000000, dtype=np.uint32)      # all m in [1, 2)
    m = bits.view(np.float32)
    r = np.float32(1.0) / np.float32(127.0)
    exact = m / np.float32(127.0)
    m64, r64 = m.astype(np.float64), np.float64(r)
    q0 = (m64 * r64).astype(np.float32)                  # 48-bit product: one rounding
    e64 = m64 - 127.0 * q0.astype(np.float64)            # exact in binary64
    e = e64.astype(np.float32)
    assert np.array_equal(e.astype(np.float64), e64)     # the fma result is exact
    s = q0.astype(np.float64) + e.astype(np.float64) * r64
    q = s.astype(np.float32)
    # the binary64 sum is itself rounded: make sure no value sits within
    # 1e-6 ulp of a binary32 rounding boundary, where that could matter
    ulp = np.float64(2.0) ** -30                          # q in [2^-7, 2^-6)
    assert np.all(np.abs(((s / ulp) % 1.0) - 0.5) > 1e-6)
    assert np.array_equal(q.view(np.uint32), exact.view(np.uint32))
