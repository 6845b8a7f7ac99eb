"""int8-mode integer rules in numpy int64.  Oracle: test infrastructure only.

Restates `src/bitexact/int8/ops.py`, `int8/segs.py` and the weight quantisation of `int8/consts.py` of the
reference.  Fixed points: residual stream / logits FR = 16, gamma FG = 12.
"""

import math

import numpy as np

from .intrules import I64, bitlen, i64, isqrt, rdiv, rsh, split_limbs

FR, FG, FA, FE, FT = 16, 12, 12, 30, 16
EPS40 = 10995116
QMAX_BITS = 23


def qmax(nl):
    return 127 << (8 * (nl - 1))                              # int8/ops.py:20-21


def quant_rows(z, nl):
    """Per-row quantisation to |q| <= qmax(nl): (q, as_, sh) (int8/ops.py:24-35; rdiv32 gives the same
    integers as rdiv, int8/ops.py:48-55)."""
    z = i64(z)
    amax = np.maximum(np.abs(z).max(-1), 1)
    sh = bitlen(amax) - 30
    as_ = rsh(amax, sh)
    zs = rsh(z, sh[:, None])
    return rdiv(zs * qmax(nl), as_[:, None]), as_, sh


def norm24(mant, e):
    """(mant, e) -> same value with mant in [2^23, 2^24] (int8/ops.py:70-73)."""
    b = bitlen(mant) - 24
    return rsh(mant, b), e + b


def pre_plain(x, nl):
    """quant_rows + row scale at FR (int8/segs.py:55-58)."""
    q, as_, sh = quant_rows(x, nl)
    mant, e = norm24(as_, sh - FR)
    return q, mant, e


def stack_limbs(q, nl):
    """int8 [nl M padded, K]: limbs stacked along rows, padded to >= 24 rows, a multiple of 8 (intops.py:73-79)."""
    a = np.concatenate([l.astype(np.int8) for l in split_limbs(q, nl)[0]])
    rows = a.shape[0]
    pad = max(24, (rows + 7) // 8 * 8) - rows
    return np.concatenate([a, np.zeros((pad, a.shape[1]), np.int8)]) if pad else a


def imm(q, w):
    """Exact q @ W^T as the reference's CPU path does it: float64 GEMM, every partial sum < 2^53
    (int8/ops.py:87-90). w int8 [N, K]."""
    return (i64(q).astype(np.float64) @ w.astype(np.float64).T).astype(I64)


def post(acc, m, fmsh, mant, e, check=True):
    """y = rsh(rsh(acc * m_c, fmsh) * mant_r, 24 - FR - e_r) and the |t| >= 2^38 flag (int8/segs.py:62-67)."""
    t = rsh(i64(acc) * i64(m)[None, :], int(fmsh))
    flag = bool(np.abs(t).max(initial=0) >= 1 << 38) if check else None
    with np.errstate(over="ignore"):
        return rsh(t * i64(mant)[:, None], (24 - FR - i64(e))[:, None]), flag


def q_linear(w):
    """float64 [N, K] -> (int8 [N, K], int64 multipliers [N], fm) (int8/consts.py:38-47)."""
    w = np.asarray(w, dtype=np.float64)
    amax = np.maximum(np.abs(w).max(1), 1e-30)
    s = amax / 127.0
    q = np.clip(np.round(w / s[:, None]), -127, 127)
    l1 = np.abs(q).sum(1)
    worst = float((l1 * s / 127.0).max()) * 2.0 ** QMAX_BITS * 127.0
    fm = min(60, int(math.floor(62 - math.log2(worst))) - 1)
    m = np.round(s / 127.0 * 2.0 ** fm).astype(I64)
    return q.astype(np.int8), m, fm
