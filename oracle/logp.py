"""Integer log p of given tokens from int64 logits rows.  Oracle (test only).

Restates `int_logp` and `lse_table` of the reference (src/bitexact/vllm_plugin/rl.py:32-65): the row maximum, a sum of
e^(l - max) terms from a table of e^x at 44 bits with step 2^-12 (linear interpolation, rounded), the logarithm of the
sum from the sampler's ln table (`ln_q`, src/bitexact/sampling.py:40-47), and the target token's term. Everything is
int64; the reference returns the integer at 2^-40 converted to float64.
"""

import numpy as np

from .intrules import i64, rsh
from .sampler import FL, LN2Q, ln_q

LSE_FE, LSE_MIN, LSE_STEP = 44, -40, 12


def lse_table():
    """e^x at LSE_FE bits for x in [LSE_MIN, 0] at step 2^-12, float64 rounded once (rl.py:32-40)."""
    xs = np.arange(LSE_MIN << LSE_STEP, 1, dtype=np.float64) / (1 << LSE_STEP)
    return np.round(np.exp(xs) * 2.0 ** LSE_FE).astype(np.int64)


def shard_sum(lg, mx, tab, fr=16):
    """Sum over the given columns of e^(l - mx) at LSE_FE bits, mx [n, 1] the maximum of the full row (rl.py:50-60)."""
    zc = np.maximum(i64(lg) - mx, -((-LSE_MIN) << fr))
    zi = zc >> (fr - LSE_STEP)
    r = zc - (zi << (fr - LSE_STEP))
    i0 = zi - (LSE_MIN << LSE_STEP)
    a = tab[i0]
    b = tab[np.minimum(i0 + 1, tab.shape[0] - 1)]
    return (a + rsh((b - a) * r, fr - LSE_STEP)).sum(-1)


def finish(S, zt, lnt, fr=16):
    """log p at 2^-FL from the row sum S and the target term zt = l_tok - max (rl.py:61-65)."""
    lse = ln_q(S, lnt) - LSE_FE * LN2Q
    return (np.maximum(i64(zt), -(1 << 36)) << (FL - fr)) - lse


def int_logp_q(lg, tok, lnt, tab=None, fr=16):
    """The integer numerator of log p (at 2^-FL) of tok [n] under logits rows lg [n, V] at fr bits (rl.py:43-65)."""
    tab = lse_table() if tab is None else tab
    lg = i64(lg)
    mx = lg.max(-1, keepdims=True)
    zt = np.take_along_axis(lg, i64(tok)[:, None], 1)[:, 0] - mx[:, 0]
    return finish(shard_sum(lg, mx, tab, fr), zt, lnt, fr)


def int_logp(lg, tok, lnt, tab=None, fr=16):
    """log p as float64: the integer at 2^-40, converted (rl.py:65)."""
    return int_logp_q(lg, tok, lnt, tab, fr).astype(np.float64) / 2.0 ** FL
