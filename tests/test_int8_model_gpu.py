"""int8 mode on the GPU: stages and attention against the oracle on seeded inputs, and the whole decode loop against
the tokens and logits hashes the reference's int8 CPU engine (IntLlama) produced for the tiny model."""

import os
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from oracle import exact as ox
from oracle import int8 as o8

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def T(a, dt=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    return (t if dt is None else t.to(dt)).cuda()


def planes_to_q(a8, M):
    a = a8.cpu().numpy().astype(np.int64)
    return a[:M] + (a[M:2 * M] << 8)


def mdl(D=512, H=4, HKV=2, HD=64, **kw):
    return SimpleNamespace(D=D, H=H, HKV=HKV, HD=HD, dev=torch.device("cuda"),
                           fl=torch.zeros(1, dtype=torch.int32, device="cuda"), **kw)


def test_int8_stages_against_oracle():
    from bitexact_llm_b200.vllm_plugin import tri_fuse as fz
    rng = np.random.RandomState(5)
    M, D = 6, 512
    x = rng.randint(-(1 << 20), 1 << 20, (M, D)).astype(np.int64)
    x[1] >>= 16
    x[2] = 0
    y = rng.randint(-(1 << 18), 1 << 18, (M, D)).astype(np.int64)
    gamma = np.round((1 + 0.3 * rng.randn(D)) * 4096).astype(np.int64)
    m = mdl(D=D)
    xo, a8, mant, e = fz.add_norm(m, T(y), None, None, None, T(x), T(gamma))
    wq, wm, we = o8.pre_norm(x + y, gamma)
    assert np.array_equal(xo.cpu().numpy(), x + y) and np.array_equal(planes_to_q(a8, M), wq)
    assert np.array_equal(mant.cpu().numpy(), wm) and np.array_equal(e.cpu().numpy(), we)
    # raw int_mm form: post applied by the stage
    N = D
    c = rng.randint(-(1 << 20), 1 << 20, (2 * M, N)).astype(np.int32)
    mul = rng.randint(1, 1 << 20, N).astype(np.int64)
    pm = rng.randint(1 << 23, 1 << 24, M).astype(np.int64)
    pe = rng.randint(-24, -12, M).astype(np.int64)
    acc = c[:M].astype(np.int64) + (c[M:].astype(np.int64) << 8)
    yy, _ = o8.post(acc, mul, 9, pm, pe)
    xo2, a82, mant2, e2 = fz.add_norm(m, T(c), (None, T(mul), 9), T(pm), T(pe), T(x), T(gamma))
    wq, wm, we = o8.pre_norm(x + yy, gamma)
    assert np.array_equal(xo2.cpu().numpy(), x + yy) and np.array_equal(planes_to_q(a82, M), wq)
    assert np.array_equal(mant2.cpu().numpy(), wm) and np.array_equal(e2.cpu().numpy(), we)
    # no-norm form sets the 2^42 flag
    xb = x.copy()
    xb[3, 3] = 1 << 42
    fz.add_norm(m, T(np.zeros_like(y)), None, None, None, T(xb), None)
    assert m.fl.item() == 1
    # rope / kv store
    H, HKV, HD, Nt = 4, 2, 64, 5
    yq = rng.randint(-(1 << 20), 1 << 20, (Nt, (H + 2 * HKV) * HD)).astype(np.int64)
    pos = np.array([0, 3, 17, 100, 255])
    ang = np.arange(256)[:, None] * (500000.0 ** (-np.arange(0, HD, 2) / HD))[None]
    cos, sin = np.round(np.cos(ang) * 65536).astype(np.int64), np.round(np.sin(ang) * 65536).astype(np.int64)
    m2 = mdl(H=H, HKV=HKV, HD=HD, cos=T(cos), sin=T(sin))
    cache = torch.zeros(20, HKV, 16, 8 * HD, dtype=torch.int8, device="cuda")
    slot = torch.tensor([16, 17, -1, 40, 95], device="cuda")
    q = fz.qkv(m2, T(yq), None, None, None, T(pos), slot, cache)
    wq, wk, wv, wf = o8.rope_qkv(yq, pos, cos, sin, H, HKV, HD)
    assert np.array_equal(q.cpu().numpy().reshape(Nt, H, HD), wq) and bool(m2.fl.item()) == wf
    want = np.zeros((20, HKV, 16, 8 * HD), dtype=np.int8)
    ox.cache_store(want, slot.cpu().numpy(), wk, wv)
    assert np.array_equal(cache.cpu().numpy(), want)
    # attention output division + silu
    num = rng.randint(-(1 << 40), 1 << 40, (Nt, H, HD)).astype(np.int64)
    den = rng.randint(1 << 20, 1 << 32, (Nt, H, 1)).astype(np.int64)
    a8, mant, e = fz.attn_out(m2, T(num).view(Nt, HKV, H // HKV, HD), T(den).view(Nt, HKV, H // HKV, 1))
    wq, wm, we = o8.attn_out(num, den)
    assert np.array_equal(planes_to_q(a8, Nt), wq) and np.array_equal(mant.cpu().numpy(), wm)
    assert np.array_equal(e.cpu().numpy(), we)
    FF = 1000
    gu = rng.randint(-(40 << 16), 40 << 16, (4, 2 * FF)).astype(np.int64)
    lut = o8.silu_table()
    a8, mant, e, flag = fz.silu_quant(mdl(), T(gu), None, None, None, T(lut))
    wq, wm, we, wf = o8.silu_mul(gu, lut)
    assert np.array_equal(planes_to_q(a8, 4), wq) and np.array_equal(mant.cpu().numpy(), wm)
    assert np.array_equal(e.cpu().numpy(), we) and bool(flag) == wf


def test_int8_paged_attention_against_oracle():
    from bitexact_llm_b200.vllm_plugin import tri_paged
    rng = np.random.RandomState(8)
    nb, bs, HKV, HD = 96, 16, 8, 64
    expt = o8.exp_table()
    ptab = T(o8.weight_table(expt), torch.int32)
    for lim in (8355711, 1 << 9):
        c32 = rng.randint(-lim, lim + 1, (nb, HKV, bs, 2 * HD)).astype(np.int64)
        planes = np.zeros((nb, HKV, bs, 8 * HD), dtype=np.int8)
        for part, o in ((c32[..., :HD], 0), (c32[..., HD:], 3)):
            for i, lo in enumerate(ox.split_limbs(part, 3)[0]):
                planes[..., (o + i) * HD:(o + i + 1) * HD] = lo.astype(np.int8)
        for R, M, P in [(3, 4, 600), (5, 4, 2500), (6, 1, 900), (7, 4, 5)]:
            bt = rng.randint(1, nb, (R, 200)).astype(np.int32)
            qpos = rng.randint(0, P, (R, M)).astype(np.int64)
            q = rng.randint(-lim, lim + 1, (R, HKV, M, HD)).astype(np.int64)
            wnum, wden = o8.paged_attention(q, qpos, planes, bt, np.arange(R), expt)
            for variant, ns in ((1, None), (2, 2), (3, None), (3, 8), (5, None), (6, None)):
                num, den = tri_paged.attend(T(q), T(qpos), T(planes), T(bt), ptab, nsplit=ns, variant=variant)
                assert np.array_equal(num.cpu().numpy(), wnum) and np.array_equal(den.cpu().numpy(), wden), \
                    (lim, R, M, P, variant, ns)


def test_int8_decode_matches_reference_hashes():
    from make_golden import TINY, TINY_PROMPTS, tiny_state_dict
    from bitexact_llm_b200.decode import generate
    from bitexact_llm_b200.int8 import consts
    from bitexact_llm_b200.int8.engine import IntEngine
    z = np.load(os.path.join(GOLD, "tiny_model_int8.npz"))
    tables = {"cos": torch.zeros(2048, 32, dtype=torch.long), "sin": torch.zeros(2048, 32, dtype=torch.long)}
    tables["cos"][:128], tables["sin"][:128] = torch.from_numpy(z["cos"]), torch.from_numpy(z["sin"])
    eng = IntEngine(consts.build(TINY, tiny_state_dict(), tables=tables), "cuda")
    for mode, (tn, td) in (("greedy", (0, 1)), ("t07", (7, 10))):
        for pi, p in enumerate(TINY_PROMPTS):
            toks, shas = generate(eng, torch.tensor([p]), 8, tn, td, seeds=[pi])
            assert toks[0].tolist() == z[f"p{pi}_{mode}_tok"].tolist(), (mode, pi)
            assert shas[0] == z[f"p{pi}_{mode}_sha"].tolist(), (mode, pi)
    order = [2, 0, 1, 1]
    P = max(len(TINY_PROMPTS[i]) for i in order)
    ids = torch.zeros(len(order), P, dtype=torch.long)
    for b, i in enumerate(order):
        ids[b, :len(TINY_PROMPTS[i])] = torch.tensor(TINY_PROMPTS[i])
    lens = torch.tensor([len(TINY_PROMPTS[i]) for i in order])
    toks, shas = generate(eng, ids, 8, 7, 10, seeds=order, lens=lens, perm_seed=3, max_len=64)
    for b, i in enumerate(order):
        assert toks[b].tolist() == z[f"p{i}_t07_tok"].tolist() and shas[b] == z[f"p{i}_t07_sha"].tolist(), b


def test_int8_prefill_tiles_and_head_shims():
    """tri_prefill.attend writes, for the tokens of its tiles, the rows tri_paged.attend gives them one by one;
    tri_sample.head / noisy and tri_logits.argmax_float give the oracle's logits, first argmax and tokens."""
    from bitexact_llm_b200.exact.consts import ln_table
    from bitexact_llm_b200.vllm_plugin import tri_logits, tri_paged, tri_prefill, tri_sample
    rng = np.random.RandomState(11)
    nb, bs, HKV, G, HD = 64, 16, 8, 4, 64
    expt = o8.exp_table()
    ptab = T(o8.weight_table(expt), torch.int32)
    lim = 1 << 13
    c32 = rng.randint(-lim, lim + 1, (nb, HKV, bs, 2 * HD)).astype(np.int64)
    planes = np.zeros((nb, HKV, bs, 8 * HD), dtype=np.int8)
    for part, o in ((c32[..., :HD], 0), (c32[..., HD:], 3)):
        for i, lo in enumerate(ox.split_limbs(part, 3)[0]):
            planes[..., (o + i) * HD:(o + i + 1) * HD] = lo.astype(np.int8)
    # three prefill requests of 37, 5 and 64 new tokens after 10, 0 and 100 cached ones, and 6 decode tokens in between
    pre = [(0, 0, 37, 47), (2, 43, 5, 5), (1, 48, 64, 164)]
    N = 112
    pos = np.zeros(N, dtype=np.int64)
    for r, t0, ql, sl in pre:
        pos[t0:t0 + ql] = np.arange(sl - ql, sl)
    bt = rng.randint(1, nb, (3, 12)).astype(np.int32)
    q = rng.randint(-lim, lim + 1, (N, HKV, G, HD)).astype(np.int64)
    num = torch.full((N, HKV, G, HD), -7, dtype=torch.long, device="cuda")
    den = torch.full((N, HKV, G, 1), -7, dtype=torch.long, device="cuda")
    tiles = tri_prefill.tile_table(pre, G).cuda()
    tri_prefill.attend(T(q), T(pos), T(planes), T(bt), ptab, tiles, num, den)
    for r, t0, ql, sl in pre:
        rows = np.arange(t0, t0 + ql)
        wnum, wden = o8.paged_attention(q[rows], np.repeat(pos[rows][:, None], G, 1), planes, bt, np.full(ql, r), expt)
        assert np.array_equal(num[t0:t0 + ql].cpu().numpy(), wnum) and np.array_equal(den[t0:t0 + ql].cpu().numpy(), wden)
    assert int(num[37:43].max()) == -7 and int(den[37:43].min()) == -7          # rows outside the tiles are untouched

    M, V, K = 5, 1000, 64
    a = rng.randint(-127, 128, (2 * M, K)).astype(np.int8)
    w = rng.randint(-127, 128, (V, K)).astype(np.int8)
    c = a.astype(np.int64) @ w.astype(np.int64).T
    mul = rng.randint(1 << 20, 1 << 24, V).astype(np.int64)
    mant = rng.randint(1 << 23, 1 << 24, M).astype(np.int64)
    e = rng.randint(-6, 2, M).astype(np.int64)
    fmsh = 14
    want, _ = o8.post(c[:M] + (c[M:] << 8), mul, fmsh, mant, e, False)
    h = tri_sample.Head(T(c.astype(np.int32), torch.int32), T(mul), fmsh, T(mant), T(e), rows=4)
    assert np.array_equal(h.logits().cpu().numpy(), want[:4])
    out, y = tri_sample.head(h, "float")
    assert np.array_equal(y.cpu().numpy(), np.argmax(want[:4], 1))
    assert np.array_equal(out.cpu().numpy(), want[:4].astype(np.float32) * np.float32(2.0 ** -16))
    out, y = tri_sample.head(h, "onehot")
    assert np.array_equal(np.isinf(out.cpu().numpy()).sum(1), np.full(4, V - 1)) and float(out[0, y[0]]) == 0.0
    assert tri_sample.head(h, "none")[0] is None
    assert np.array_equal(tri_logits.argmax_float(T(want), mode="none")[1].cpu().numpy(), np.argmax(want, 1))
    assert np.array_equal(tri_logits.first_argmax(T(want)).cpu().numpy(), np.argmax(want, 1))
    from oracle import sampler as osamp
    keys, temps = [(3, 0), (3, 1), (9, 7), (1, 2)], [(7, 10), (0, 1), (13, 10), (1, 1)]
    st = tri_sample.row_state(keys, temps)
    lnt = ln_table(device="cuda")
    vout = torch.zeros(4, V, dtype=torch.float32, device="cuda")
    tok = tri_sample.noisy(h, st, lnt, out=vout).cpu().numpy()
    lnt_np = ox.ln_table()
    for r, ((seed, t), (tn, td)) in enumerate(zip(keys, temps)):
        g = osamp.gumbel(osamp.raw_words(seed, t, V), lnt_np, 16) if tn else None
        assert tok[r] == int(osamp.sample(want[r:r + 1], tn, td, g)[0]), r
        assert float(vout[r, tok[r]]) == 0.0 and int(torch.isinf(vout[r]).sum()) == V - 1
