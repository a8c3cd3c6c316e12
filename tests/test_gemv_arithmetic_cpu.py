"""The integer identities the decode GEMV kernel relies on, checked in numpy (no GPU).

The kernel feeds `word & (0x01010101 << j)` (an int8x4 with values {0, 2^j}, {0, -128} for j = 7) to an s8 MMA as
the A operand and the activations, quantised to a fixed-point X with |X| <= 64000, as B operands X * 2^(7-j)
(-X for j = 7) split into three signed bytes.  Every product is then 128 * X on the columns whose bit is set, the
three byte terms recombine exactly, and sum(+-X) = sum(X) - 2 * sum_{bit=1}(X) = sum(X) - terms / 64.
"""
import numpy as np

Q_MAX = 64000


def byte_terms(y):
    """Split Y (int64 array, |Y| < 2^23) into signed bytes b0, b1, b2 with Y = 65536*b2 + 256*b1 + b0, the way
    the kernel does it on 32-bit registers: b0 = byte 0 of Y, b1 = byte 1 of Y + 0x80, b2 = byte 2 of Y + 0x8080."""
    u = y.astype(np.int64) & 0xFFFFFFFF
    as_s8 = lambda v: ((v & 0xFF) ^ 0x80) - 0x80
    b0 = as_s8(u)
    b1 = as_s8((u + 0x80) >> 8)
    b2 = as_s8((u + 0x8080) >> 16)
    return b0, b1, b2


def test_three_signed_bytes_recombine_exactly():
    g = np.random.default_rng(0)
    x = np.concatenate([g.integers(-Q_MAX, Q_MAX + 1, size=200000), [Q_MAX, -Q_MAX, 0, 1, -1, 127, 128, -128, -129, 32767, -32768]])
    for j in range(8):
        y = -x if j == 7 else x << (7 - j)           # class-shifted operand, |Y| <= 64000 * 128 < 2^23
        b0, b1, b2 = byte_terms(y)
        assert np.all(np.abs(b0) <= 128) and np.all(np.abs(b1) <= 128) and np.all(np.abs(b2) <= 128)
        assert np.array_equal(65536 * b2 + 256 * b1 + b0, y)


def test_masked_bits_times_shifted_operand_is_128_x():
    # A value of class j: 2^j as a signed byte (-128 for j = 7); operand: X * 2^(7-j) (-X for j = 7)
    x = np.arange(-Q_MAX, Q_MAX + 1, 997, dtype=np.int64)
    for j in range(8):
        a = -128 if j == 7 else 1 << j
        y = -x if j == 7 else x << (7 - j)
        assert np.array_equal(a * y, 128 * x)


def test_sign_sum_from_the_three_accumulators():
    g = np.random.default_rng(1)
    K = 4096
    x = g.integers(-Q_MAX, Q_MAX + 1, size=K).astype(np.int64)
    bits = g.integers(0, 2, size=(32, K)).astype(np.int64)          # 1 = weight -1
    j = (np.arange(K) % 256) // 32                                   # class of a column inside its 256-column chunk
    a = np.where(j == 7, -128, 1 << j) * bits                        # what the masked registers hold
    y = np.where(j == 7, -x, x << (7 - j))
    b0, b1, b2 = byte_terms(y)
    c0, c1, c2 = a @ b0, a @ b1, a @ b2                              # the three int32 accumulators per row
    assert np.all(np.abs(c0) < 2**31) and np.all(np.abs(c1) < 2**31) and np.all(np.abs(c2) < 2**31)
    terms = 65536 * c2 + 256 * c1 + c0
    assert np.all(terms % 128 == 0)
    got = x.sum() - (terms >> 6)
    want = ((1 - 2 * bits) * x).sum(axis=1)
    assert np.array_equal(got, want)


def test_accumulators_stay_inside_int32_at_the_largest_k():
    # worst case per accumulator: every bit set, every byte term at its extreme, K = 32768 columns
    K = 32768
    assert K * 128 * 128 < 2**31
    assert K * Q_MAX < 2**31       # sum(X)
