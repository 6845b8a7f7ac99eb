"""Integer Gumbel-max sampler: PCG64 words, integer -ln(-ln u), first argmax.  Oracle (test only).

Restates `src/bitexact/sampling.py` of the reference.  The raw words there come from numpy
(`np.random.default_rng([SEED_BASE, seed, t]).bit_generator.random_raw(V)`, sampling.py:27-28), a
third-party dependency the reference pins only as "numpy"; here SeedSequence and PCG64 (XSL-RR 128/64)
are restated from their published algorithms with Python integers, and the tests compare them with the
installed numpy word for word.
"""

import numpy as np

from .intrules import I64, bitlen, first_argmax, i64, rdiv, rsh

SEED_BASE = 20261022          # sampling.py:19
FL = 40
LN2Q = 762123384786           # round(ln 2 * 2^40)
UMIN = 9008

M32 = 0xFFFFFFFF
M128 = (1 << 128) - 1
PCG_MULT = (2549297995355413924 << 64) + 4865540595714422341


def seed_words(entropy, n_words=8, pool_size=4):
    """numpy SeedSequence(entropy).generate_state(n_words // 2, uint64) as uint32 words."""
    INIT_A, MULT_A, INIT_B, MULT_B = 0x43B0D7E5, 0x931E8875, 0x8B51F9DD, 0x58F38DED
    MIX_L, MIX_R, XS = 0xCA01F9DD, 0x4973F715, 16
    ent = []
    for e in entropy:                                   # every integer as little-endian uint32 words
        e = int(e)
        ent.append(e & M32)
        e >>= 32
        while e:
            ent.append(e & M32)
            e >>= 32
    hc = [INIT_A]

    def hashmix(v):
        v = (v ^ hc[0]) & M32
        hc[0] = (hc[0] * MULT_A) & M32
        v = (v * hc[0]) & M32
        return v ^ (v >> XS)

    def mix(x, y):
        r = (MIX_L * x - MIX_R * y) & M32
        return r ^ (r >> XS)

    pool = [hashmix(ent[i] if i < len(ent) else 0) for i in range(pool_size)]
    for i_src in range(pool_size):
        for i_dst in range(pool_size):
            if i_src != i_dst:
                pool[i_dst] = mix(pool[i_dst], hashmix(pool[i_src]))
    for i_src in range(pool_size, len(ent)):
        for i_dst in range(pool_size):
            pool[i_dst] = mix(pool[i_dst], hashmix(ent[i_src]))
    hb = INIT_B
    out = []
    for i in range(n_words):
        v = pool[i % pool_size] ^ hb
        hb = (hb * MULT_B) & M32
        v = (v * hb) & M32
        out.append(v ^ (v >> XS))
    return out


def pcg_state(seed, t):
    """(state, inc) of PCG64 after numpy seeds it from SeedSequence([SEED_BASE, seed, t])."""
    w = seed_words([SEED_BASE, seed, t])
    u64 = [w[2 * i] | (w[2 * i + 1] << 32) for i in range(4)]
    initstate = (u64[0] << 64) | u64[1]
    initseq = (u64[2] << 64) | u64[3]
    inc = ((initseq << 1) | 1) & M128
    state = inc                                            # (0 * mult + inc)
    state = (state + initstate) & M128
    state = (state * PCG_MULT + inc) & M128
    return state, inc


def raw_words(seed, t, n):
    """First n raw 64-bit outputs as int64 (two's complement of the uint64 words)."""
    state, inc = pcg_state(seed, t)
    out = np.empty(n, dtype=np.uint64)
    for i in range(n):
        state = (state * PCG_MULT + inc) & M128
        hi, lo = state >> 64, state & ((1 << 64) - 1)
        x = hi ^ lo
        rot = state >> 122
        out[i] = ((x >> rot) | (x << ((64 - rot) & 63))) & ((1 << 64) - 1)
    return out.view(I64)


def raw_rows(keys, n):
    return np.stack([raw_words(s, t, n) for s, t in keys]) if len(keys) else np.zeros((0, n), I64)


def ln_q(n, lnt):
    """ln(n) at FL bits for n >= 1 (sampling.py:40-47)."""
    n = i64(n)
    k = bitlen(n) - 1
    m = np.where(k <= 52, n << np.maximum(52 - k, 0), n >> np.maximum(k - 52, 0))
    idx = (m >> 36) - (1 << 16)
    r = (m >> 16) & ((1 << 20) - 1)
    a = lnt[idx]
    return k * LN2Q + a + (((lnt[idx + 1] - a) * r) >> 20)


def gumbel(raw, lnt, bits):
    """-ln(-ln u) at `bits` fractional bits from raw words (sampling.py:50-59)."""
    U = np.clip((i64(raw) >> 11) & ((1 << 53) - 1), UMIN, (1 << 53) - UMIN)
    Dd = (1 << 53) - U
    A = 53 * LN2Q - ln_q(U, lnt)
    main = ln_q(np.maximum(A, 1), lnt) - FL * LN2Q
    dq = Dd >> 13
    ser = ln_q(Dd, lnt) - 53 * LN2Q + (dq >> 1) + (5 * (dq >> 8) ** 2) // (24 << 24)
    return rsh(-np.where(Dd < (1 << 45), ser, main), FL - bits)


def sample(logits, tn, td, g=None):
    """Greedy (tn == 0) or Gumbel-max at T = tn / td (sampling.py:62-67)."""
    if tn == 0:
        return first_argmax(logits)
    return first_argmax(rdiv(i64(logits) * td, I64(tn)) + g)
