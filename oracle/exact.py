"""Exact-mode (original bf16 weights) integer rules in numpy int64.  Oracle: test infrastructure only.

Restates `src/bitexact/exact/ops.py`, `exact/wmm.py`, `exact/consts.py` and `exact/segs.py` of the
reference.  All arrays are int64 unless said otherwise; every rule is row-local.
"""

import numpy as np

from .intrules import I64, LIM, bitlen, fdiv, first_argmax, i64, isqrt, rdiv, rsh, split_limbs

# fixed points and constants (exact/consts.py:23-30, exact/ops.py:13-22, exact/segs.py:21)
FR, FT, FL = 24, 30, 40
EXP2_BITS, EXP2_ONE = 14, 60
QB, FN, FT2, FZ = 22, 40, 26, 26
FK, FV, FP = 17, 19, 22
L2E28, L2E30 = 387270501, 1549082005
L2E28_HD = {64: L2E28, 128: 273841598}
EPS60 = 11529215046068
NEG_BIG = -(1 << 20)
LIM3 = LIM[3]


def rshc(x, s):
    """round(x / 2^s) with the shift clamped to [-62, 62] (exact/ops.py:25-34)."""
    x = i64(x)
    if isinstance(s, (int, np.integer)):
        s = max(-62, min(62, int(s)))
        return ((x + (I64(1) << (s - 1))) >> s) if s > 0 else (x << (-s))
    s = np.clip(i64(s), -62, 62)
    pos = np.maximum(s, 0)
    half = np.where(pos > 0, I64(1) << np.maximum(pos - 1, 0), 0)
    return ((x + half) >> pos) << np.maximum(-s, 0)


def div_round(a, p, r, chunk=28):
    """round(a * 2^p / r) by long division in 28-bit chunks (exact/ops.py:37-57)."""
    a, r = i64(a), i64(r)
    p = np.broadcast_to(i64(p), np.broadcast(a, r, i64(p)).shape).copy()
    Q = fdiv(a, r)
    R = a - Q * r
    left = np.maximum(p, 0)
    for _ in range(3):
        c = np.minimum(left, chunk)
        X = R << c
        q1 = fdiv(X, r)
        Q = (Q << c) + q1
        R = X - q1 * r
        left = left - c
    up = Q + (2 * R >= r)
    k = np.clip(-p, 1, 62)
    down = (Q + (I64(1) << (k - 1))) >> k
    return np.where(p >= 0, up, down)


def combine(T, d, B):
    """(H, L): H * 2^32 + L = T * 2^d + B, 0 <= L < 2^32 (exact/ops.py:60-66)."""
    T, d, B = i64(T), i64(d), i64(B)
    s = 32 - d
    H = T >> s
    L = ((T & ((I64(1) << s) - 1)) << d) + B
    return H + (L >> 32), L & 0xFFFFFFFF


def shift_round_hl(H, L, p):
    """round((H * 2^32 + L) * 2^p) in three shift regimes (exact/ops.py:69-79)."""
    p = i64(p)
    k = np.maximum(-p, 0)
    pp = np.clip(p, 0, 30)
    up = (H << (32 + pp)) + (L << pp)
    k1 = np.clip(k, 1, 31)
    small = (H << (32 - k1)) + ((L + (I64(1) << (k1 - 1))) >> k1)
    k2 = np.clip(k, 32, 94)
    carry = np.where(k2 == 32, (L + (I64(1) << 31)) >> 32, I64(1) << np.maximum(k2 - 33, 0))
    big = (H + carry) >> np.minimum(k2 - 32, 62)
    return np.where(p >= 0, up, np.where(k < 32, small, big))


def epilogue(T, B, d, g, sh, checked=False):
    """y = round((T 2^d + B) 2^p), p = sh[m] + g[n] - d[n] + FR, and the lost-bit / range flag
    (exact/wmm.py:132-150)."""
    H, L = combine(T, i64(d)[None, :], B)
    p = i64(sh)[:, None] + (i64(g) - i64(d))[None, :] + FR
    with np.errstate(over="ignore"):
        y = shift_round_hl(H, L, p)
    if not checked:
        return y
    up_limit = I64(1) << (31 - np.clip(p, 0, 30))
    small_limit = I64(1) << (31 + np.clip(-p, 1, 31))
    up_lost = (H >= up_limit) | (H < -up_limit) | ((p > 30) & ((H != 0) | (L != 0)))
    small_lost = (H >= small_limit) | (H < -small_limit)
    lost = np.where(p >= 0, up_lost, (p > -32) & small_lost)
    flag = bool((lost | (y <= -(1 << 62)) | (y >= (1 << 62))).any())
    return y, flag


def quant(P, eps):
    """Per-row power-of-two quantisation: q (|q| <= 2^22), sh (exact/ops.py:82-89)."""
    P = i64(P)
    e = np.where(P != 0, bitlen(np.abs(P)) + i64(eps), NEG_BIG)
    sh = np.maximum(e.max(-1) - QB, NEG_BIG)
    return rshc(P, sh[..., None] - i64(eps)), sh


def rms(x):
    """(r, er): sqrt(mean(x^2) + 1e-5) = r * 2^er with 2^30 <= r < 2^31 (exact/ops.py:92-105)."""
    x = i64(x)
    D = x.shape[-1]
    lg = D.bit_length() - 1
    assert D == 1 << lg and lg <= 12
    amax = np.maximum(np.abs(x).max(-1), 1)
    shx = np.maximum(bitlen(amax) - 25, -6)
    xs = rshc(x, shx[:, None])
    S = (xs * xs).sum(-1)
    T = S + rshc(np.full_like(S, EPS60 * D), 60 - 2 * (FR - shx))
    m = (62 + lg - bitlen(T)) // 2
    s = 2 * m - lg
    V = np.where(s >= 0, T << np.maximum(s, 0), T >> np.maximum(-s, 0))
    return isqrt(V), shx - FR - m


def exp2_table():
    """2^-f at 2^60 for f = i / 2^14, i = 0..2^14 (exact/consts.py:112-113)."""
    f = np.arange((1 << EXP2_BITS) + 1, dtype=np.float64) / (1 << EXP2_BITS)
    return np.round(np.power(2.0, -f) * 2.0 ** EXP2_ONE).astype(I64)


def ln_table(bits=FL):
    """ln(1 + i / 2^16) at `bits` fractional bits (llama.py:72-75)."""
    i = np.arange((1 << 16) + 1, dtype=np.float64)
    return np.round(np.log1p(i / (1 << 16)) * 2.0 ** bits).astype(I64)


def exp2neg_lut(t, lut, out_bits):
    """2^-t at out_bits for t >= 0 at FT2 bits: table + linear interpolation (exact/ops.py:108-116)."""
    t = i64(t)
    n = t >> FT2
    f = t & ((1 << FT2) - 1)
    idx = f >> (FT2 - EXP2_BITS)
    rr = f & ((1 << (FT2 - EXP2_BITS)) - 1)
    a = lut[idx]
    v = a + rshc((lut[idx + 1] - a) * rr, FT2 - EXP2_BITS)
    return rshc(v, EXP2_ONE - out_bits + n)


def silu_mul(g, u, lut):
    """P = silu(g) * u for g, u at FR, with the bound check (exact/ops.py:119-130)."""
    g, u = i64(g), i64(u)
    a = np.minimum(np.abs(g), 64 << FR)
    t = rshc(a * L2E30, FR + 30 - FT2)
    E = exp2neg_lut(t, lut, 30)
    den = (1 << 30) + E
    sig = np.where(g >= 0, rdiv(np.full_like(E, 1 << 60), den), rdiv(E << 30, den))
    gc = np.clip(g, -(1 << 32), 1 << 32)
    s = rshc(gc * sig, 30)
    ok = bool(((bitlen(np.abs(s)) + bitlen(np.abs(u))) <= 62).all()) and bool(np.abs(g).max(initial=0) <= 1 << 32)
    with np.errstate(over="ignore"):
        return s * u, ok


def softmax_w(raw, ok, sh, lut, l2e=L2E28, kbits=FK, fp=FP):
    """Attention weights at fp bits from exact scores; masked keys give 0 (exact/ops.py:133-143).
    raw [.., S], ok bool [.., S], sh [.., 1]."""
    raw = np.where(ok, i64(raw), -(1 << 62))
    z = raw.max(-1, keepdims=True) - raw
    zf = np.minimum(rshc(z, kbits + 3 - i64(sh) - FZ), 48 << FZ)
    t = rshc(zf * l2e, FZ + 28 - FT2)
    p = np.where(ok, exp2neg_lut(t, lut, fp), 0)
    return p, p.sum(-1, keepdims=True)


# ---- weights (exact/consts.py) ----

def bf16_parts(bits):
    """uint16 bf16 bit patterns -> (signed significand, exponent): w = sm * 2^ex (exact/consts.py:33-42)."""
    b = i64(bits) & 0xFFFF
    e = (b >> 7) & 0xFF
    assert not (e == 255).any(), "inf/nan weight"
    m = b & 0x7F
    mag = np.where(e > 0, m | 0x80, m)
    ex = np.where(e > 0, e, 1) - 134
    return np.where((b >> 15) == 1, -mag, mag), ex


def decompose(bits):
    """bf16 bit patterns [N, K] -> limbs int8 [3, N, K], g, d [N], COO residual (rr, rc, rv)
    (exact/consts.py:67-107).  Row grid g: smallest exponent with max |W| <= LIM3; the bits below
    the grid go to the sparse residual on the finer grid gf = g - d."""
    sm, ex = bf16_parts(bits)
    mag = np.abs(sm)
    nz = mag > 0
    top = np.where(nz, ex + bitlen(mag), -10 ** 6).max(1)
    g = top - 23
    while True:
        sh = np.minimum(ex - g[:, None], 40)
        big = nz & (sh >= 0) & ((mag << np.maximum(sh, 0)) > LIM3)
        bad = big.any(1)
        if not bad.any():
            break
        g = np.where(bad, g + 1, g)
    g = np.where(top < -10 ** 5, 0, g)
    sh = ex - g[:, None]
    up = sh >= 0
    shl = np.clip(sh, 0, 40)
    shr = np.clip(-sh, 0, 40)
    dmag = np.where(up, mag << shl, mag >> shr)
    rmag = np.where(up, 0, mag - (dmag << shr))
    W = np.where(sm < 0, -dmag, dmag)
    has = rmag > 0
    lowbit = bitlen(rmag & -rmag) - 1                       # index of the lowest set bit
    low = np.where(has, ex + lowbit, 10 ** 6)
    gf = np.minimum(low.min(1), g)
    d = g - gf
    assert int(d.max(initial=0)) <= 30
    rr, rc = np.nonzero(has)
    s_ = ex[rr, rc] - gf[rr]
    rm_ = rmag[rr, rc]
    rv = np.where(s_ >= 0, rm_ << np.maximum(s_, 0), rm_ >> np.maximum(-s_, 0))
    rv = np.where(sm[rr, rc] < 0, -rv, rv)
    lim, rem = split_limbs(W, 3)
    assert not rem.any()
    return {"limbs": np.stack([l.astype(np.int8) for l in lim]), "g": g, "d": d,
            "rr": i64(rr), "rc": i64(rc), "rv": rv}


def dense_product(q, limbs, cache=None):
    """T = q @ W^T exactly, as the reference's CPU path does it: the three activation limbs against
    the float64 weight, every partial sum < 2^53 (exact/wmm.py:117-121, exact/model.py:56-58).
    cache: optional dict that keeps the float64 weight copy between calls (the reference's Lin.w64)."""
    if cache is not None and "w64" in cache:
        w64 = cache["w64"]
    else:
        w64 = limbs[0].astype(np.float64)
        w64 += 256.0 * limbs[1]
        w64 += 65536.0 * limbs[2]
        w64 = np.ascontiguousarray(w64.T)
        if cache is not None and cache.get("keep_w64"):
            cache["w64"] = w64
    M = q.shape[0]
    A = np.concatenate(split_limbs(q, 3)[0]).astype(np.float64)
    C = (A @ w64).astype(I64)
    return C[:M] + (C[M:2 * M] << 8) + (C[2 * M:] << 16)


def residual(q, rr, rc, rv, N):
    """B[m, n] = sum over residual entries of row n of q[m, col] * val (exact/wmm.py:124-129)."""
    B = np.zeros((q.shape[0], N), dtype=I64)
    if len(rr):
        np.add.at(B, (slice(None), rr), i64(q)[:, rc] * rv)
    return B


def linear(q, sh, w, checked=True):
    """The exact linear y = round((q @ W_bf16) 2^(sh + FR)): dense limbs + residual + one rounding
    (exact/model.py:61-70 + exact/segs.py:25-32).  w = decompose(...) dict."""
    N = w["limbs"].shape[1]
    T = dense_product(i64(q), w["limbs"], w if isinstance(w, dict) else None)
    B = residual(q, w["rr"], w["rc"], w["rv"], N)
    return epilogue(T, B, w["d"], w["g"], sh, checked)


# ---- stages between the linears (exact/segs.py) ----

def norm_quant(x, gm, ge):
    """rms + ndiv + quant(., -FN) -> q (int64 values, |q| <= 2^22), sh, flag (exact/segs.py:49-68)."""
    x = i64(x)
    r, er = rms(x)
    P = div_round(x * i64(gm), i64(ge) - FR - er[:, None] + FN, r[:, None])
    q, sh = quant(P, -FN)
    return q, sh, bool(np.abs(x).max(initial=0) >= 1 << 40)


def rope_qkv(y, pos, cos, sin, H, HKV, HD):
    """qkv output rows y [N, (H + 2 HKV) HD] at FR -> q [N, H, HD] (quantised per token and head),
    shq [N, H], k [N, HKV, HD] at FK, v at FV, flag (exact/segs.py:71-99)."""
    y = i64(y)
    N = y.shape[0]
    c, s = i64(cos)[pos][:, None, :], i64(sin)[pos][:, None, :]

    def rot(x):
        x1, x2 = x[..., :HD // 2], x[..., HD // 2:]
        return np.concatenate([x1 * c - x2 * s, x2 * c + x1 * s], -1)

    Pq = rot(y[:, :H * HD].reshape(N, H, HD))
    k = rshc(rot(y[:, H * HD:(H + HKV) * HD].reshape(N, HKV, HD)), FR + FT - FK)
    v = rshc(y[:, (H + HKV) * HD:].reshape(N, HKV, HD), FR - FV)
    q, shq = quant(Pq, -(FR + FT))
    flag = bool(np.abs(y).max(initial=0) >= 1 << 31) or bool(np.abs(k).max(initial=0) > LIM3) \
        or bool(np.abs(v).max(initial=0) > LIM3) or bool(shq.max(initial=NEG_BIG) > FK + 3 - FZ)
    return q, shq, k, v, flag


def attn_out(num, den):
    """o = div_round(num, FR - FV, den), then quant(o, -FR) per token row (exact/segs.py:108-113,187-188).
    num [N, H, HD], den [N, H, 1] -> q [N, H HD], sh [N]."""
    o = div_round(num, FR - FV, den)
    return quant(o.reshape(o.shape[0], -1), -FR)


def silu_quant(y, lut):
    """gate/up output [N, 2 FF] -> quant(silu(g) u, -2 FR), flag (exact/segs.py:120-128)."""
    ff = y.shape[1] // 2
    P, ok = silu_mul(y[:, :ff], y[:, ff:], lut)
    q, sh = quant(P, -2 * FR)
    return q, sh, not ok


# ---- paged limb-plane KV cache and attention (vllm_plugin/tri_paged.py, tri_exact_attn.py) ----

def cache_store(cache, slot, k, v):
    """Write K / V [N, HKV, HD] at flat slots into cache int8 [nb, HKV, bs, 8 HD]: K limbs at bytes
    [0, 3 HD), V limbs at [3 HD, 6 HD); slot < 0 skipped (tri_paged.py:22-25, 311-335)."""
    bs, HD = cache.shape[2], k.shape[2]
    kl, _ = split_limbs(k, 3)
    vl, _ = split_limbs(v, 3)
    for n in range(len(slot)):
        s = int(slot[n])
        if s < 0:
            continue
        for i in range(3):
            cache[s // bs, :, s % bs, i * HD:(i + 1) * HD] = kl[i][n].astype(np.int8)
            cache[s // bs, :, s % bs, (3 + i) * HD:(4 + i) * HD] = vl[i][n].astype(np.int8)


def cache_gather(cache, bt_row, S, HD):
    """Keys / values 0..S-1 of one request as int64 [HKV, S, HD] each, joined from the limb planes."""
    bs = cache.shape[2]
    s = np.arange(S)
    rows = cache[i64(bt_row)[s // bs], :, s % bs].astype(I64)          # [S, HKV, 8 HD]
    join = lambda o: rows[..., o * HD:(o + 1) * HD] + (rows[..., (o + 1) * HD:(o + 2) * HD] << 8) \
        + (rows[..., (o + 2) * HD:(o + 3) * HD] << 16)
    return join(0).transpose(1, 0, 2), join(3).transpose(1, 0, 2)


def paged_attention(q, sh, qpos, cache, bt, rmap, lut, l2e=L2E28):
    """num int64 [R, HKV, M, HD], den [R, HKV, M, 1] as tri_exact_attn.attend returns them
    (tri_exact_attn.py:1-16, 138-165; unfused form exact/model.py:114-119)."""
    R, HKV, M, HD = q.shape
    num = np.zeros((R, HKV, M, HD), dtype=I64)
    den = np.zeros((R, HKV, M, 1), dtype=I64)
    for r in range(R):
        S = int(qpos[r].max()) + 1
        if S <= 0:
            continue
        K, V = cache_gather(cache, bt[int(rmap[r])], S, HD)             # [HKV, S, HD]
        raw = np.einsum("hmd,hsd->hms", i64(q[r]), K)
        ok = np.arange(S)[None, None, :] <= i64(qpos[r])[None, :, None]
        p, dn = softmax_w(raw, np.broadcast_to(ok, raw.shape), i64(sh[r])[..., None], lut, l2e)
        num[r] = np.einsum("hms,hsd->hmd", p, V)
        den[r] = dn
    return num, den
