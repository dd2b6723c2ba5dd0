"""Generates tests/golden/kat_rounding.npz and kat_matmul_int.npz.

The reference has no golden vectors for this path (its .mlir tests carry no
data), so these known-answer tests are derived independently of the C checker:
exact rational arithmetic (fractions.Fraction) with a pure-Python
round-to-nearest-even, and exact integer matrix products.  They pin the checker;
the checker then pins the CUDA path.

    python tests/golden/make_golden.py
"""
import os
import random
from fractions import Fraction

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

FMT = {"f16": (11, -14, 15, 5), "bf16": (8, -126, 127, 8)}


def decode(bits: int, fmt: str) -> Fraction:
    p, emin, emax, ebits = FMT[fmt]
    mbits = p - 1
    sign = -1 if bits >> 15 else 1
    e = (bits >> mbits) & ((1 << ebits) - 1)
    m = bits & ((1 << mbits) - 1)
    if e == 0:
        return sign * Fraction(m, 1 << mbits) * Fraction(2) ** emin
    return sign * (1 + Fraction(m, 1 << mbits)) * Fraction(2) ** (e - (emax))


def round_rn(x: Fraction, fmt: str, rz=False) -> int:
    """Exact value -> bit pattern, round to nearest even (or toward zero)."""
    p, emin, emax, ebits = FMT[fmt]
    mbits = p - 1
    if x == 0:
        return 0
    sign = 0x8000 if x < 0 else 0
    a = abs(x)
    # exponent of the leading bit
    e = 0
    while Fraction(2) ** (e + 1) <= a:
        e += 1
    while Fraction(2) ** e > a:
        e -= 1
    e = max(e, emin)
    ulp = Fraction(2) ** (e - mbits)
    q = a / ulp
    n = q.numerator // q.denominator
    rem = q - n
    if not rz:
        if rem > Fraction(1, 2) or (rem == Fraction(1, 2) and n % 2 == 1):
            n += 1
    if n >= (1 << p):  # carried into the next binade
        n >>= 1
        e += 1
    if e > emax:
        return sign | ((((1 << ebits) - 1) << mbits) if not rz else
                       ((((1 << ebits) - 2) << mbits) | ((1 << mbits) - 1)))
    if n < (1 << mbits):  # subnormal
        return sign | n
    return sign | ((e + emax) << mbits) | (n - (1 << mbits))


def rounding_kat(seed=20251125, n=4000):
    rnd = random.Random(seed)
    rows = []
    for fmt_id, fmt in ((0, "f16"), (1, "bf16")):
        p, emin, emax, ebits = FMT[fmt]
        mbits = p - 1
        maxe = (1 << ebits) - 2

        def rand_bits(span):
            e = rnd.randint(max(1, emax - span), min(maxe, emax + span))
            return (rnd.getrandbits(1) << 15) | (e << mbits) | rnd.getrandbits(mbits)

        for i in range(n):
            kind = i % 4
            a, b = rand_bits(4), rand_bits(4)
            if kind == 0:
                c = rand_bits(6)
            elif kind == 1:   # addend far below the product: sticky-bit cases
                c = (rnd.getrandbits(1) << 15) | (max(1, emax - 30) << mbits) | rnd.getrandbits(mbits)
            elif kind == 2:   # exact ties: product with low half exactly 1000...
                a = (a & ~((1 << (mbits // 2)) - 1)) | (1 << (mbits // 2 - 1))
                b = (1 << 15 & b) | (emax << mbits) | (1 << (mbits - 1))  # +-1.5
                c = 0
            else:             # cancellation
                c = round_rn(-decode(a, fmt) * decode(b, fmt), fmt) ^ rnd.getrandbits(2)
            exact = decode(a, fmt) * decode(b, fmt) + decode(c, fmt)
            rows.append((fmt_id, a, b, c, round_rn(exact, fmt)))
    return np.array(rows, dtype=np.int64)


def cvt_kat(seed=7, n=3000):
    """f32 -> f16/bf16 with RN and RZ from exact rationals."""
    rnd = random.Random(seed)
    rows = []
    for _ in range(n):
        # a float32 value: 24-bit significand, modest exponent, some near-tie tails
        sig = rnd.getrandbits(24) | (1 << 23)
        if rnd.random() < 0.3:
            sig = (sig & ~0xFFFF) | rnd.choice([0x8000, 0x7FFF, 0x8001, 0x0000])
        if rnd.random() < 0.3:
            sig = (sig & ~0x1FFF) | rnd.choice([0x1000, 0x0FFF, 0x1001, 0x0000])
        e = rnd.randint(-30, 20)
        sgn = -1 if rnd.getrandbits(1) else 1
        x = sgn * Fraction(sig, 1 << 23) * Fraction(2) ** e
        f32 = np.float32(float(x))
        assert Fraction(float(f32)) == x
        rows.append((int(f32.view(np.uint32)),
                     round_rn(x, "f16"), round_rn(x, "f16", rz=True),
                     round_rn(x, "bf16"), round_rn(x, "bf16", rz=True)))
    return np.array(rows, dtype=np.int64)


def matmul_int_kat(seed=11):
    """Small-integer matrices: every product and every partial sum is exact in
    f16/bf16 x f32, so the expected output is the exact integer product."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, (M, N, K) in {"a": (96, 80, 72), "b": (128, 256, 192), "c": (33, 17, 41)}.items():
        A = rng.integers(-4, 5, size=(M, K)).astype(np.int64)
        B = rng.integers(-4, 5, size=(K, N)).astype(np.int64)
        bias = rng.integers(-8, 9, size=(N,)).astype(np.int64)
        out[f"A_{name}"] = A.astype(np.int8)
        out[f"B_{name}"] = B.astype(np.int8)
        out[f"bias_{name}"] = bias.astype(np.int8)
        out[f"C_{name}"] = (A @ B + bias[None, :]).astype(np.int32)
    return out


if __name__ == "__main__":
    np.savez_compressed(os.path.join(HERE, "kat_rounding.npz"), fma=rounding_kat(), cvt=cvt_kat())
    np.savez_compressed(os.path.join(HERE, "kat_matmul_int.npz"), **matmul_int_kat())
    print("wrote", os.listdir(HERE))
