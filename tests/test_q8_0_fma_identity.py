"""Host check of the arithmetic the tcgen05 producer uses to turn a Q8_0 int8 into q * d without an integer convert.

The kernel places u = q + 128 in byte 1 of a float whose other bytes are those of 2^23 (f = 2^23 + 256 u) and evaluates
fma(f, d / 256, -(2^23 + 2^15) * d / 256).  The claim tested here: every term of that expression is exact in fp32 for
every int8 q and every finite fp16 scale d, so the fma returns q * d exactly and the only rounding is the final one to
the 16-bit operand type.
"""
import numpy as np


def _all_finite_f16():
    bits = np.arange(0x10000, dtype=np.uint32).astype(np.uint16)
    d = bits.view(np.float16)
    return d[np.isfinite(d)].astype(np.float64)


def test_q8_0_magic_terms_are_exact_in_fp32():
    d = _all_finite_f16()
    q = np.arange(-128, 128, dtype=np.int64)
    u = (q + 128).astype(np.uint32)
    f_bits = np.uint32(0x4B000000) | (u << np.uint32(8))
    f = f_bits.view(np.float32).astype(np.float64)
    assert np.array_equal(f, 2.0 ** 23 + 256.0 * u)                      # the byte-permuted pattern is that float
    d256 = d / 256.0
    assert np.array_equal(d256.astype(np.float32).astype(np.float64), d256)   # d / 256 is an fp32 number
    c = -(2.0 ** 23 + 2.0 ** 15) * d256
    assert np.array_equal(c.astype(np.float32).astype(np.float64), c)         # 9 x 11 significant bits: exact
    # float64 holds f * d256 (24 + 11 bits) and the sum exactly, so this is the infinitely precise fma result
    w = f[:, None] * d256[None, :] + c[None, :]
    assert np.array_equal(w, q[:, None].astype(np.float64) * d[None, :])
    assert np.array_equal(w.astype(np.float32).astype(np.float64), w)         # and it is an fp32 number: no rounding
