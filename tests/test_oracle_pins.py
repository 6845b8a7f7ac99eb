"""Pins of the CPU oracle: the reference's known-answer transcript, Fraction restatements of its unit
tests, and golden vectors produced by the reference itself (tests/golden/make_golden.py)."""

import hashlib
import json
import math
import os
import random
from fractions import Fraction

import numpy as np

from oracle import exact as ox
from oracle import intrules as ir
from oracle import sampler as osamp

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def rnd(fr):
    return math.floor(fr + Fraction(1, 2))


def bf16_bits_of(vals):
    """float values exactly representable in bf16 -> uint16 bit patterns."""
    f = np.asarray(vals, dtype=np.float32)
    return (f.view(np.uint32) >> 16).astype(np.uint16)


def test_known_answer_transcript_hash():
    """The eight fixtures of the reference's self-check (src/bitexact/repro.py:144-187), recomputed with the
    oracle, hash to the value its test pins (tests/test_repro.py:126)."""
    vectors = {}
    values = [-(1 << 50) + 3, -17, -1, 0, 1, 17, (1 << 50) - 3]
    for shift in [-3, 0, 1, 7, 31]:
        got = ir.rsh(np.array(values), shift).tolist()
        assert got == [rnd(Fraction(v) / Fraction(2) ** shift) for v in values]
        vectors[f"round_shift_{shift}"] = got
    denom = [3, 7, 11, 13, 17, 19, 23]
    vectors["floor_division"] = ir.fdiv(np.array(values), np.array(denom)).tolist()
    squares = [0, 1, 2, 3, 4, 17, (1 << 60) - 1]
    vectors["integer_sqrt"] = ir.isqrt(np.array(squares)).tolist()
    assert vectors["integer_sqrt"] == [math.isqrt(x) for x in squares]
    w = [[1.0, -0.5, 2 ** -30, -2 ** -28, 0.125, 0.0, 0.75, -0.25],
         [-0.25, 0.5, -0.125, 1.0, -2 ** -29, 2 ** -31, -0.75, 0.0]]
    dec = ox.decompose(bf16_bits_of(w))
    q = np.array([[13, -7, 3, 11, 0, -5, 17, -19], [-2, 5, 7, -11, 3, 0, 1, 4]])
    shifts = [-10, -6]
    y, bad = ox.linear(q, np.array(shifts), dec, checked=True)
    assert not bad
    want = [[rnd(sum(Fraction(wv) * int(x) for wv, x in zip(row, qs)) * Fraction(2) ** (s + ox.FR)) for row in w]
            for qs, s in zip(q, shifts)]
    assert y.tolist() == want
    vectors["bf16_linear_with_sparse_residual"] = y.tolist()
    enc = json.dumps(vectors, sort_keys=True, separators=(",", ":")).encode()
    assert hashlib.sha256(enc).hexdigest() == "5053b757aad61165cb7d22d271f6b87acbc0edbd29ec06f352f1f4e022b1b214"


def test_rounding_rules_vs_python_integers():
    rng = random.Random(1)
    xs = [rng.randrange(-(1 << 61), 1 << 61) for _ in range(2000)]
    ss = [rng.randrange(-3, 63) for _ in range(2000)]
    got = ox.rshc(np.array(xs), np.array(ss))
    for x, s, gv in zip(xs, ss, got.tolist()):
        if s <= 0 and abs(x) >= 1 << (62 + s):
            continue
        assert gv == rnd(Fraction(x) * Fraction(2) ** (-s))
    assert ir.bitlen(np.array([0, 1, 2, 3, 4, (1 << 53) - 1, 1 << 53, (1 << 62) + 1])).tolist() \
        == [0, 1, 2, 2, 3, 53, 54, 63]
    xs = [rng.randrange(0, 1 << 62) for _ in range(2000)] + [k * k - 1 for k in range(2, 200)] + [(1 << 62) - 1]
    assert ir.isqrt(np.array(xs)).tolist() == [math.isqrt(x) for x in xs]


def test_div_round_vs_fractions():
    """exact/ops.py:37-57 as tested by the reference (tests/test_exact_ops.py:30-42)."""
    rng = random.Random(2)
    a, p, r = [], [], []
    for _ in range(4000):
        a.append(rng.randrange(-(1 << 61), 1 << 61))
        p.append(rng.randrange(-70, 85))
        r.append(rng.randrange(1 << 11, 1 << 34))
        if p[-1] > 0:                                   # keep the result below 2^62
            a[-1] >>= min(61, p[-1] + 2)
    got = ox.div_round(np.array(a), np.array(p), np.array(r)).tolist()
    for av, pv, rv, gv in zip(a, p, r, got):
        if pv >= 0:
            assert gv == rnd(Fraction(av) * Fraction(2) ** pv / rv)
        else:                                            # floor quotient first, then one rounding of the shift
            assert gv == rnd(Fraction(av // rv) / Fraction(2) ** min(-pv, 62))


def test_epilogue_vs_fractions():
    rng = random.Random(3)
    T = np.array([[rng.randrange(-(1 << 58), 1 << 58) for _ in range(8)] for _ in range(50)])
    B = np.array([[rng.randrange(-(1 << 40), 1 << 40) for _ in range(8)] for _ in range(50)])
    d = np.array([0, 1, 5, 12, 30, 7, 0, 29])
    g = np.array([-30, -25, -31, -20, -3, -28, -33, -2])
    sh = np.array([rng.randrange(-60, -5) for _ in range(50)])
    y = ox.epilogue(T, B, d, g, sh)
    for m in range(50):
        for j in range(8):
            p = int(sh[m] + g[j] - d[j] + ox.FR)
            want = rnd((Fraction(int(T[m, j])) * 2 ** int(d[j]) + int(B[m, j])) * Fraction(2) ** p)
            if p <= 30 and abs(want) < 1 << 61:
                assert int(y[m, j]) == want


def test_golden_exact_linear_and_decompose():
    z = np.load(os.path.join(GOLD, "exact_ops.npz"))
    dec = ox.decompose(z["lin_w"])
    for k in ("limbs", "g", "d", "rr", "rc", "rv"):
        assert np.array_equal(dec[k], z["lin_" + k]), k
    assert len(dec["rr"]) > 0
    y, flag = ox.linear(z["lin_q"], z["lin_sh"], dec, checked=True)
    assert np.array_equal(y, z["lin_y"]) and flag == bool(z["lin_flag"])
    rows = [ox.linear(z["lin_q"][m:m + 1], z["lin_sh"][m:m + 1], dec, checked=True)[1] for m in range(len(y))]
    assert rows == z["lin_rowflag"].tolist()
    assert any(rows) and not all(rows)


def test_golden_exact_stages():
    z = np.load(os.path.join(GOLD, "exact_ops.npz"))
    r, er = ox.rms(z["norm_x"])
    assert np.array_equal(r, z["norm_r"]) and np.array_equal(er, z["norm_er"])
    q, sh, _ = ox.norm_quant(z["norm_x"], z["norm_gm"], z["norm_ge"])
    assert np.array_equal(q, z["norm_q"]) and np.array_equal(sh, z["norm_sh"])
    q, shq, k, v, _ = ox.rope_qkv(z["rope_y"], z["rope_pos"], z["rope_cos"], z["rope_sin"], 4, 2, 64)
    for a, b in ((q, "rope_q"), (shq, "rope_sh"), (k, "rope_k"), (v, "rope_v")):
        assert np.array_equal(a, z[b]), b
    q, sh, err = ox.silu_quant(z["silu_y"], ox.exp2_table())
    assert np.array_equal(q, z["silu_q"]) and np.array_equal(sh, z["silu_sh"]) and err == bool(z["silu_err"])


def test_golden_paged_attention():
    z = np.load(os.path.join(GOLD, "exact_ops.npz"))
    R = z["attn_q"].shape[0]
    num, den = ox.paged_attention(z["attn_q"], z["attn_sh"], z["attn_qpos"], z["attn_cache"], z["attn_bt"],
                                  np.arange(R), ox.exp2_table())
    assert np.array_equal(num, z["attn_num"]) and np.array_equal(den, z["attn_den"])
    HKV, G, HD = num.shape[1:]
    qo, sho = ox.attn_out(num.reshape(R, HKV * G, HD), den.reshape(R, HKV * G, 1))
    assert np.array_equal(qo, z["attn_qo"]) and np.array_equal(sho, z["attn_sho"])


def test_cache_store_roundtrip():
    rng = np.random.RandomState(0)
    cache = np.zeros((6, 2, 16, 512), dtype=np.int8)
    k = rng.randint(-8355711, 8355712, (5, 2, 64))
    v = rng.randint(-8355711, 8355712, (5, 2, 64))
    slot = np.array([16, 17, -1, 40, 95])
    ox.cache_store(cache, slot, k, v)
    bt = np.array([1, 2, 5])
    K, V = ox.cache_gather(cache, bt, 48, 64)
    assert np.array_equal(K[:, 0], k[0]) and np.array_equal(V[:, 1], v[1]) and np.array_equal(K[:, 24], k[3])
    assert not cache[5, :, 14].any() and np.array_equal(cache[5, :, 15, :64].astype(np.int64),
                                                         ir.split_limbs(k[4], 3)[0][0])


def test_golden_sampler_and_numpy_words():
    z = np.load(os.path.join(GOLD, "sampler.npz"))
    keys = [tuple(int(v) for v in k) for k in z["keys"]]
    raw = osamp.raw_rows(keys, 2048)
    ref = z["raw"].copy()
    assert np.array_equal(raw[1:], ref[1:]) and np.array_equal(raw[0, 6:], ref[0, 6:])
    for s, t in keys:                                    # and against the installed numpy, word for word
        want = np.random.default_rng([osamp.SEED_BASE, s, t]).bit_generator.random_raw(64)
        assert np.array_equal(osamp.raw_words(s, t, 64).view(np.uint64), want)
    lnt = ox.ln_table()
    g = osamp.gumbel(ref, lnt, 24)
    assert np.array_equal(g, z["gumbel"])
    assert np.array_equal(osamp.sample(z["logits"], 0, 1), z["tok_greedy"])
    assert np.array_equal(osamp.sample(z["logits"], 7, 10, g), z["tok_t07"])
    assert int(z["tok_greedy"][2]) == 100                # first of two equal maxima


def test_golden_int8_linear():
    from oracle import int8 as o8
    z = np.load(os.path.join(GOLD, "int8_ops.npz"))
    wq, m, fm = o8.q_linear(z["w"])
    assert np.array_equal(wq, z["wq"]) and np.array_equal(m, z["m"]) and fm == int(z["fm"])
    q, mant, e = o8.pre_plain(z["x"], 2)
    assert np.array_equal(q, z["q"]) and np.array_equal(mant, z["mant"]) and np.array_equal(e, z["e"])
    assert np.array_equal(o8.stack_limbs(q, 2), z["stacked"])
    acc = o8.imm(q, wq)
    y, flag = o8.post(acc, m, fm + 8 - 24, mant, e)
    assert np.array_equal(acc, z["acc"]) and np.array_equal(y, z["y"]) and flag == bool(z["flag"])


def test_gumbel_noise_is_monotone_in_the_uniform():
    """The integer Gumbel noise never decreases when the uniform grows, inside each of its two branches and across
    every power-of-two boundary of 1 - u: the property the GPU sampler's exact pruning rests on."""
    from oracle import exact as ox
    from oracle import sampler as osamp
    lnt = ox.ln_table()
    rng = np.random.RandomState(0)
    for bits in (16, 24):
        us = [rng.randint(osamp.UMIN, 1 << 53, 400000, dtype=np.int64)]
        for j in range(1, 41):                                   # both sides of every bucket boundary
            t = (1 << 53) - (1 << (53 - j))
            us.append(np.arange(max(t - 300, 1), min(t + 300, (1 << 53) - 1), dtype=np.int64))
        us.append(np.arange(1, 20000, dtype=np.int64))
        us.append((1 << 53) - np.arange(1, 20000, dtype=np.int64))
        us.append((1 << 53) - (1 << 45) + np.arange(-5000, 5000, dtype=np.int64))
        u = np.unique(np.concatenate(us))
        g = osamp.gumbel(u << 11, lnt, bits)
        series = ((1 << 53) - np.clip(u, osamp.UMIN, (1 << 53) - osamp.UMIN)) < (1 << 45)
        for part in (g[~series], g[series]):                     # monotone inside each branch
            assert (np.diff(part) >= 0).all()
        for j in range(1, 41):                                   # and bounded by the value at the bucket's top
            t = (1 << 53) - (1 << (53 - j))
            lo = (1 << 53) - (1 << (54 - j)) if j > 1 else 0
            sel = (u > lo) & (u <= t)
            gt = osamp.gumbel(np.array([t], dtype=np.int64) << 11, lnt, bits)[0]
            assert (g[sel] <= gt).all(), j


def test_golden_integer_logp_and_table():
    """oracle.logp against rl.int_logp of the reference (ordinary, flat, peaked, constant and far-below rows, the two
    clamps), the e^x table against the reference's (hash and samples), for the oracle's numpy table and the package's."""
    import torch
    from bitexact_llm_b200.vllm_plugin import rl
    from oracle import logp as ol
    z = np.load(os.path.join(GOLD, "logp.npz"))
    tab = ol.lse_table()
    assert hashlib.sha256(tab.tobytes()).hexdigest() == str(z["tab_sha"])
    assert np.array_equal(tab[::997], z["tab_sample"])
    assert torch.equal(rl.lse_table("cpu"), torch.from_numpy(tab))
    lnt = ox.ln_table(40)
    got = ol.int_logp(z["logits"], z["tok"], lnt, tab)
    assert np.array_equal(got, z["logp"])
    # shards of the vocabulary: integer max of maxima, integer sum of sums -> the same integer
    lg = z["logits"].astype(np.int64)
    q = ol.int_logp_q(lg, z["tok"], lnt, tab)
    mx = lg.max(1, keepdims=True)
    S = sum(ol.shard_sum(lg[:, a:b], mx, tab) for a, b in ((0, 1000), (1000, 1001), (1001, 3001)))
    zt = np.take_along_axis(lg, z["tok"][:, None], 1)[:, 0] - mx[:, 0]
    assert np.array_equal(ol.finish(S, zt, lnt), q)
