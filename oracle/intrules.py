"""Integer rounding rules shared by both modes (numpy int64; oracle, test infrastructure only).

Follows `src/bitexact/intops.py` of the reference: round-half-up everywhere, floor division,
exact integer square root, first-index argmax, signed base-256 limbs.
"""

import numpy as np

I64 = np.int64
LIM = {1: 127, 2: 32639, 3: 8355711}      # intops.py:11 -- reach of n signed base-256 digits


def i64(x):
    return np.asarray(x, dtype=I64)


def bitlen(x):
    """Bits needed for x >= 0 (0 -> 0).  intops.py:14-21 gets this from frexp plus a fix-up;
    here a six-step binary search on shifts gives the same exact value."""
    x = i64(x)
    n = np.zeros_like(x)
    v = x.copy()
    for s in (32, 16, 8, 4, 2, 1):
        big = (v >> s) != 0
        n = n + np.where(big, s, 0)
        v = np.where(big, v >> s, v)
    return n + (v != 0)


def rsh(x, s):
    """round(x / 2^s) ties up for s > 0, x * 2^-s for s <= 0 (intops.py:24-34)."""
    x = i64(x)
    if isinstance(s, (int, np.integer)):
        s = int(s)
        return ((x + (1 << (s - 1))) >> s) if s > 0 else (x << (-s))
    s = i64(s)
    pos = np.maximum(s, 0)
    neg = np.maximum(-s, 0)
    half = np.where(pos > 0, I64(1) << np.maximum(pos - 1, 0), 0)
    return ((x + half) >> pos) << neg


def fdiv(a, b):
    """floor(a / b), b > 0 (intops.py:37-39)."""
    return np.floor_divide(i64(a), i64(b))


def rdiv(a, b):
    """round(a / b) ties up, b > 0 (intops.py:42-44)."""
    a, b = i64(a), i64(b)
    return np.floor_divide(2 * a + b, 2 * b)


def isqrt(x):
    """floor(sqrt(x)), x >= 0: float64 estimate then two integer corrections (intops.py:46-52)."""
    x = i64(x)
    s = np.floor(np.sqrt(x.astype(np.float64))).astype(I64)
    for _ in range(2):
        s = np.where(s * s > x, s - 1, s)
        s = np.where((s + 1) * (s + 1) <= x, s + 1, s)
    return s


def first_argmax(v):
    """Index of the first maximum along the last axis (intops.py:55-59)."""
    v = i64(v)
    m = v.max(-1, keepdims=True)
    col = np.broadcast_to(np.arange(v.shape[-1], dtype=I64), v.shape)
    return np.where(v == m, col, v.shape[-1]).min(-1)


def split_limbs(x, n):
    """Signed base-256 digits, least significant first, and the remainder (intops.py:62-70)."""
    r = i64(x).copy()
    out = []
    for _ in range(n):
        lo = ((r + 128) & 255) - 128
        out.append(lo)
        r = (r - lo) >> 8
    return out, r
