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


# ---- stages between the linears (int8/ops.py, int8/segs.py, int8/consts.py) ----
FQ, FV, FP8 = 14, 14, 20
EXP_MIN, SILU_LIM = -32, 32
LIM3 = 8355711
NEG = -(1 << 62)


def rms(x):
    """(r, shx): rms value = r * 2^(shx - FR) (int8/ops.py:76-84)."""
    x = i64(x)
    d = x.shape[-1]
    amax = np.maximum(np.abs(x).max(-1), 1)
    shx = bitlen(amax) - 24
    xs = rsh(x, shx[:, None])
    ms = (xs * xs).sum(-1) // d
    eps = rsh(np.full_like(shx, EPS40), 40 - 2 * (FR - shx))
    return isqrt(ms + eps), shx


def pre_norm(x, gamma, nl=2):
    """RMSNorm + per-row quantisation -> q, mant, e (int8/segs.py:48-53)."""
    r, shx = rms(x)
    q, as_, sh = quant_rows(i64(x) * i64(gamma), nl)
    mant, e = norm24(rdiv(as_ << 30, r), sh - FG - shx - 30)
    return q, mant, e


def exp_table():
    xs = np.arange(EXP_MIN << FA, 1, dtype=np.float64) / (1 << FA)
    return np.round(np.exp(xs) * (1 << FE)).astype(I64)              # int8/consts.py:50-53


def silu_table():
    xs = np.arange(-SILU_LIM << FA, (SILU_LIM << FA) + 1, dtype=np.float64) / (1 << FA)
    return np.round(xs / (1.0 + np.exp(-xs)) * (1 << FR)).astype(I64)   # int8/consts.py:79-80


def weight_table(lut):
    """rsh(exp table, FE - FP) (vllm_plugin/tri_paged.py:351-356)."""
    return (lut + (1 << (FE - FP8 - 1))) >> (FE - FP8)


def silu(g, lut):
    """SiLU at FR from the table at step 2^-FA with interpolation (int8/ops.py:100-108)."""
    g = i64(g)
    lo, hi = -SILU_LIM << FA, SILU_LIM << FA
    gi = g >> (FR - FA)
    r = g - (gi << (FR - FA))
    i = np.clip(gi, lo, hi - 1) - lo
    a = lut[i]
    v = a + rsh((lut[i + 1] - a) * r, FR - FA)
    return np.where(gi >= hi, g, np.where(gi < lo, 0, v))


def rope_qkv(y, pos, cos, sin, H, HKV, HD):
    """y [N, (H + 2 HKV) HD] at FR -> q [N, H, HD], k, v [N, HKV, HD], flag (int8/segs.py:69-88)."""
    y = i64(y)
    N = y.shape[0]
    c, s = i64(cos)[pos][:, None, :], i64(sin)[pos][:, None, :]
    shr = FT + FR - FQ

    def rot(x):
        x1, x2 = x[..., :HD // 2], x[..., HD // 2:]
        return np.concatenate([rsh(x1 * c - x2 * s, shr), rsh(x2 * c + x1 * s, shr)], -1)

    q = rot(y[:, :H * HD].reshape(N, H, HD))
    k = rot(y[:, H * HD:(H + HKV) * HD].reshape(N, HKV, HD))
    v = rsh(y[:, (H + HKV) * HD:].reshape(N, HKV, HD), FR - FV)
    flag = any(int(np.abs(t).max(initial=0)) > LIM3 for t in (q, k, v))
    return q, k, v, flag


def softmax(raw, ok, expt, zsh=2 * FQ + 3 - FA):
    """Attention weights at FP from exact scores; masked keys give 0 (int8/segs.py:91-99, head_dim 64)."""
    raw = np.where(ok, i64(raw), NEG)
    d = raw - raw.max(-1, keepdims=True)
    z = np.maximum(rsh(d, zsh), -(1 << 40))
    idx = z - (EXP_MIN << FA)
    val = np.where(idx < 0, 0, expt[np.maximum(idx, 0)])
    p = np.where(ok, rsh(val, FE - FP8), 0)
    return p, p.sum(-1, keepdims=True)


def attn_out(num, den, nl=2):
    """o = rdiv(num << (FR - FV), den) per head, then pre_plain of the token rows (int8/segs.py:101-109).
    num [N, H, HD], den [N, H, 1]."""
    o = rdiv(i64(num) << (FR - FV), i64(den))
    return pre_plain(o.reshape(o.shape[0], -1), nl)


def silu_mul(gu, lut, nl=2):
    """gate/up output [N, 2 FF] -> (q, mant, e, flag) (int8/segs.py:111-118). The flag is over the whole batch."""
    ff = gu.shape[1] // 2
    g, u = i64(gu[:, :ff]), i64(gu[:, ff:])
    sg = silu(g, lut)
    flag = int(np.abs(sg).max(initial=0)) * int(np.abs(u).max(initial=0)) >= 1 << 62
    q, mant, e = pre_plain(rsh(sg * u, FR), nl)
    return q, mant, e, flag


def paged_attention(q, qpos, cache, bt, rmap, expt):
    """int8-mode counterpart of oracle.exact.paged_attention (vllm_plugin/tri_paged.py:363-430): q int64
    [R, HKV, M, HD] within 3 limbs, no row exponent."""
    from .exact import cache_gather
    R, HKV, M, HD = q.shape
    num = np.zeros((R, HKV, M, HD), dtype=I64)
    den = np.zeros((R, HKV, M, 1), dtype=I64)
    for r in range(R):
        S = int(qpos[r].max()) + 1
        if S <= 0:
            continue
        K, V = cache_gather(cache, bt[int(rmap[r])], S, HD)
        raw = np.einsum("hmd,hsd->hms", i64(q[r]), K)
        ok = np.arange(S)[None, None, :] <= i64(qpos[r])[None, :, None]
        p, dn = softmax(raw, np.broadcast_to(ok, raw.shape), expt)
        num[r] = np.einsum("hms,hsd->hmd", p, V)
        den[r] = dn
    return num, den
