"""Exact-rational f32 fused multiply-add in pure Python (small cases only).

TEST INFRASTRUCTURE ONLY.  An independent second statement of
``f32::mul_add`` (one correctly rounded operation, round-to-nearest-even),
used to pin that the C oracle's ``fmaf`` chain is what
compiler/src/interp.rs:9270-9287 specifies, without trusting the C compiler's
flags.  Python 3.12 has no ``math.fma``, hence the Fractions.
"""
from __future__ import annotations

import struct
from fractions import Fraction


def f32_bits(x: float) -> int:
    return struct.unpack("<I", struct.pack("<f", x))[0]


def bits_f32(u: int) -> float:
    return struct.unpack("<f", struct.pack("<I", u & 0xFFFFFFFF))[0]


def round_fraction_to_f32(v: Fraction) -> float:
    """Nearest-even rounding of an exact rational to binary32 (finite range)."""
    if v == 0:
        return 0.0
    sign = -1 if v < 0 else 1
    v = abs(v)
    # e = floor(log2(v))
    e = v.numerator.bit_length() - v.denominator.bit_length()
    if Fraction(2) ** e > v:
        e -= 1
    if Fraction(2) ** (e + 1) <= v:
        e += 1
    e = max(e, -126)                      # subnormals share the 2^-149 grid
    ulp = Fraction(2) ** (e - 23)
    q = v / ulp
    n = q.numerator // q.denominator
    rem = q - n
    if rem > Fraction(1, 2) or (rem == Fraction(1, 2) and (n & 1)):
        n += 1
    out = float(n) * float(ulp)           # both exact in binary64
    if out >= 2.0 ** 128:
        out = float("inf")
    return sign * out


def fma_f32(a: float, b: float, c: float) -> float:
    """round_f32(a*b + c) with a single rounding."""
    return round_fraction_to_f32(Fraction(a) * Fraction(b) + Fraction(c))


def gemm_f32_fma(a, b):
    """compiler/src/interp.rs:9270-9287 on nested lists of f32-exact floats."""
    m, k, n = len(a), len(b), len(b[0])
    out = [[0.0] * n for _ in range(m)]
    for i in range(m):
        for j in range(n):
            acc = 0.0
            for kk in range(k):
                acc = fma_f32(a[i][kk], b[kk][j], acc)
            out[i][j] = acc
    return out
