"""The stage-by-stage API of the reference (`bitexact.exact.segs`, `bitexact.exact.ops`, `bitexact.int8.segs`,
`tri_mlp.silu_quant`, `tri_fuse.mlp_mid / flag_end`, `gpu_pcg.seed_state / raw_from_state`, `Lin` with padded
residual lists) on the GPU: every stage against the CPU oracle, and the stage chains of `Segs` against the fused
kernels the serving path uses (same integers either way)."""

import numpy as np
import pytest
import torch

from oracle import exact as ox
from oracle import int8 as o8
from oracle import sampler as osamp

pytestmark = pytest.mark.gpu


def T(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    return (t if dtype is None else t.to(dtype)).cuda()


def N_(t):
    return t.cpu().numpy()


def test_rms_ndiv_quant_and_the_norm_chain():
    from bitexact_llm_b200.exact import ops, segs
    rng = np.random.RandomState(1)
    for D in (64, 2048, 4096):
        x = rng.randint(-(1 << 30), 1 << 30, (9, D)).astype(np.int64)
        x[0] = 0
        x[1, 3] = (1 << 39) + 5
        gm = rng.randint(100, 256, D).astype(np.int64)
        ge = rng.randint(-9, -5, D).astype(np.int64)
        wr, wer = ox.rms(x)
        r, er = ops.rms(T(x))
        assert np.array_equal(N_(r), wr) and np.array_equal(N_(er), wer)
        wP = ox.div_round(x * gm, ge - ox.FR - wer[:, None] + ox.FN, wr[:, None])
        P = segs.ndiv(T(x), T(gm), T(ge), r, er)
        assert np.array_equal(N_(P), wP)
        wq, wsh = ox.quant(wP, -ox.FN)
        q, sh = segs.quant(P, -ox.FN)
        assert q.dtype == torch.int32 and np.array_equal(N_(q), wq) and np.array_equal(N_(sh), wsh)
        err0 = torch.zeros((), dtype=torch.bool, device="cuda")
        for one in (False, True):
            sg = segs.Segs(dm=(32, 8, 64), one_region=one)
            q2, sh2, err = sg.norm_q(T(x), T(gm), T(ge), err0)
            assert torch.equal(q2, q) and torch.equal(sh2, sh) and not bool(err)
    xb = x.copy()
    xb[2, 0] = 1 << 40
    assert bool(segs.rms(T(xb), err0)[2]) and bool(segs.norm_quant(T(xb), T(gm), T(ge), err0)[2])


def test_rope_group_softmax_attention_division_chain():
    """qkv_y -> scores and p.V through bmm -> softmax -> attn_out: the standalone engine's attention
    (src/bitexact/exact/model.py:106-121) stage by stage against the oracle."""
    from bitexact_llm_b200.bmm import bmm
    from bitexact_llm_b200.exact import consts, segs
    rng = np.random.RandomState(2)
    H, HKV, HD, B, Tn = 4, 2, 64, 2, 5
    G = H // HKV
    y = rng.randint(-(1 << 28), 1 << 28, (B * Tn, (H + 2 * HKV) * HD)).astype(np.int64)
    pos = np.stack([np.arange(3, 3 + Tn), np.arange(0, Tn)]).astype(np.int64)
    cfg = dict(consts.LLAMA_1B)
    cos, sin = consts.rope_tables(cfg, 64)
    sg = segs.Segs(dm=(H, HKV, HD))
    err0 = torch.zeros((), dtype=torch.bool, device="cuda")
    qg, shg, k, v, err = sg.qkv_y(T(y), T(pos), cos.cuda(), sin.cuda(), B, Tn, err0)
    wq, wshq, wk, wv, wflag = ox.rope_qkv(y, pos.reshape(-1), cos.numpy(), sin.numpy(), H, HKV, HD)
    assert np.array_equal(N_(k).reshape(B * Tn, HKV, HD), wk) and np.array_equal(N_(v).reshape(B * Tn, HKV, HD), wv)
    wqg = wq.reshape(B, Tn, HKV, G, HD).transpose(0, 2, 3, 1, 4).reshape(B * HKV, G * Tn, HD)
    wshg = wshq.reshape(B, Tn, HKV, G).transpose(0, 2, 3, 1).reshape(B * HKV, G * Tn, 1)
    assert np.array_equal(N_(qg), wqg) and np.array_equal(N_(shg), wshg) and bool(err) == wflag
    # keys = the tokens themselves (positions 0 .. S - 1 of a fresh cache row per sequence)
    S = 8
    Kc = rng.randint(-(1 << 19), 1 << 19, (B, HKV, S, HD)).astype(np.int64)
    Vc = rng.randint(-(1 << 21), 1 << 21, (B, HKV, S, HD)).astype(np.int64)
    Z = B * HKV
    raw = bmm(qg, T(Kc).transpose(-1, -2).reshape(Z, HD, S))
    wraw = np.einsum("zmd,zsd->zms", wqg, Kc.reshape(Z, S, HD))
    assert np.array_equal(N_(raw), wraw)
    qpos = np.broadcast_to(pos[:, None, None, :], (B, HKV, G, Tn)).reshape(Z, G * Tn, 1)
    lut = ox.exp2_table()
    p, den = sg.softmax(raw, T(qpos), shg, T(lut))
    ok = np.arange(S)[None, None, :] <= qpos
    wp, wden = ox.softmax_w(wraw, ok, wshg, lut, ox.L2E28_HD[HD])
    assert p.dtype == torch.int32 and np.array_equal(N_(p), wp) and np.array_equal(N_(den), wden)
    num = bmm(p, T(Vc).reshape(Z, S, HD))
    wnum = np.einsum("zms,zsd->zmd", wp, Vc.reshape(Z, S, HD))
    assert np.array_equal(N_(num), wnum)
    qo, sho = sg.attn_out(num, den, Tn)
    wo = ox.div_round(wnum, ox.FR - ox.FV, wden).reshape(B, HKV, G, Tn, HD).transpose(0, 3, 1, 2, 4).reshape(B * Tn, H * HD)
    wqo, wsho = ox.quant(wo, -ox.FR)
    assert np.array_equal(N_(qo), wqo) and np.array_equal(N_(sho), wsho)
    # ops.softmax_w with an arbitrary mask
    from bitexact_llm_b200.exact import ops
    okr = rng.rand(Z, G * Tn, S) < 0.6
    okr[..., 0] = True
    p2, d2 = ops.softmax_w(raw, T(okr), shg, 17, T(lut), 22, ox.L2E28_HD[HD])
    wp2, wd2 = ox.softmax_w(wraw, okr, wshg, lut, ox.L2E28_HD[HD])
    assert np.array_equal(N_(p2), wp2) and np.array_equal(N_(d2), wd2)


def test_silu_stages_equal_the_fused_kernel_and_the_oracle():
    from types import SimpleNamespace
    from bitexact_llm_b200.exact import segs
    from bitexact_llm_b200.vllm_plugin import exact_fuse
    rng = np.random.RandomState(3)
    N, FF = 5, 8192
    gu = rng.randint(-(6 << 24), 6 << 24, (N, 2 * FF)).astype(np.int64)
    lut = ox.exp2_table()
    sg = segs.Segs()
    err0 = torch.zeros((), dtype=torch.bool, device="cuda")
    q, sh, err = sg.gu_silu_y(T(gu), T(lut), err0)
    wq, wsh, wflag = ox.silu_quant(gu, lut)
    assert np.array_equal(N_(q), wq) and np.array_equal(N_(sh), wsh) and bool(err) == wflag
    m = SimpleNamespace(dev=torch.device("cuda"))
    fl = torch.zeros(1, dtype=torch.int32, device="cuda")
    q2, sh2 = exact_fuse.silu_quant(m, T(gu), T(lut), fl)
    assert torch.equal(q2, q) and torch.equal(sh2, sh)
    gu[1, 7] = (1 << 32) + 1                                      # |g| beyond the table clamp: the bound flag
    assert bool(sg.gu_silu_y(T(gu), T(lut), err0)[2])


def test_lin_with_padded_residual_lists_and_lin_out():
    from bitexact_llm_b200.exact import segs
    from bitexact_llm_b200.exact.consts import decompose
    from bitexact_llm_b200.exact.model import Lin
    g = torch.Generator().manual_seed(9)
    w = (torch.randn(384, 256, generator=g) * 0.02).to(torch.bfloat16)
    dec = decompose(w.cuda())
    assert dec["rr"].numel() > 0
    q = torch.randint(-(1 << 22), (1 << 22) + 1, (11, 256), generator=g)
    sh = torch.randint(-30, -10, (11,), generator=g)
    want, wflag = ox.linear(q.numpy(), sh.numpy(), {k: v.cpu().numpy() for k, v in dec.items()}, checked=True)
    sg = segs.Segs()
    for ell in (False, True):
        lin = Lin({f"l.{k}": v for k, v in dec.items()}, "l", "cuda", "triton", ell, 6)
        y, flag = sg.lin_out(*lin(q.cuda()), sh.cuda())
        assert np.array_equal(N_(y), want) and bool(flag) == wflag
    x = torch.randint(-(1 << 30), 1 << 30, (11, 384), generator=g).cuda()
    x2, f2 = segs.lin_add(*lin(q.cuda()), sh.cuda(), x)
    assert np.array_equal(N_(x2), N_(x) + want)


def test_int8_post_softmax_and_mlp_mid():
    from types import SimpleNamespace
    from bitexact_llm_b200.int8 import segs as isegs
    from bitexact_llm_b200.int8.gemm_skinny import int_mm
    from bitexact_llm_b200.vllm_plugin import tri_fuse, tri_mlp
    rng = np.random.RandomState(4)
    M, N = 7, 300
    acc = rng.randint(-(1 << 30), 1 << 30, (M, N)).astype(np.int64)
    mul = rng.randint(1, 1 << 24, N).astype(np.int64)
    mant = rng.randint(1 << 23, (1 << 24) + 1, M).astype(np.int64)
    e = rng.randint(-30, -5, M).astype(np.int64)
    for fmsh in (20, 12):
        want, wflag = o8.post(acc, mul, fmsh, mant, e)
        y, flag = isegs.post(T(acc), T(mul), fmsh, T(mant), T(e))
        assert np.array_equal(N_(y), want) and bool(flag) == wflag
    assert isegs.post(T(acc), T(mul), 20, T(mant), T(e), check=False)[1] is None
    # dense-score softmax of int8 mode
    B, HKV, gT, S = 2, 2, 6, 37
    raw = rng.randint(-(1 << 34), 1 << 34, (B, HKV, gT, S)).astype(np.int64)
    qpos = rng.randint(0, S, (B, 1, gT, 1)).astype(np.int64)
    expt = o8.exp_table()
    p, den = isegs.softmax(T(raw), T(qpos), T(expt))
    wp, wden = o8.softmax(raw, np.arange(S) <= qpos, expt)
    assert np.array_equal(N_(p), wp) and np.array_equal(N_(den), wden)
    # tri_mlp.silu_quant / tri_fuse.mlp_mid / flag_end(m) on a raw gate-up GEMM output
    K, FF = 128, 96
    w8 = rng.randint(-127, 128, (2 * FF, K)).astype(np.int8)
    qa = rng.randint(-32512, 32513, (M, K)).astype(np.int64)
    mgu = rng.randint(1 << 20, 1 << 23, 2 * FF).astype(np.int64)
    fm = 24
    a = T(o8.stack_limbs(qa, 2))
    c = int_mm(a, T(w8), M=M)
    silu_t = o8.silu_table()
    gu, pflag = o8.post(o8.imm(qa, w8), mgu, fm, mant, e)
    wa, wmant, we, wfl = o8.silu_mul(gu, silu_t)
    q8, m2, e2, flag = tri_mlp.silu_quant(c, T(mgu), fm, T(mant), T(e), T(silu_t), True)
    assert q8.shape[0] == max(24, (2 * M + 7) // 8 * 8) and not bool(q8[2 * M:].any())
    assert np.array_equal(N_(q8[:2 * M]), o8.stack_limbs(wa, 2)[:2 * M])
    assert np.array_equal(N_(m2), wmant) and np.array_equal(N_(e2), we) and bool(flag) == (wfl or pflag)
    m = SimpleNamespace(dev=torch.device("cuda"), L=3, silu_t=T(silu_t), fl=torch.zeros(1, dtype=torch.int32, device="cuda"))
    out = tri_fuse.mlp_mid(m, {"wgu": (T(w8), T(mgu), fm)}, c, T(mant), T(e), 1)
    assert torch.equal(out[0], q8) and torch.equal(out[1], m2) and int(m.scr[1, 0]) > 0 and int(m.scr[0, 0]) == 0
    tri_fuse.flag_end(m)
    assert not bool(m.scr.any()) and int(m.fl) == int(wfl)
    m.scr[2] = torch.tensor([1 << 31, 1 << 31])                     # product 2^62: the bound
    tri_fuse.flag_end(m)
    assert int(m.fl) == 1


def test_pcg_state_round_trip():
    from bitexact_llm_b200.vllm_plugin import gpu_pcg
    keys = [(0, 0), (5, 77), (2 ** 33 + 1, 2 ** 35)]
    st = gpu_pcg.seed_state(keys)
    assert st.device.type == "cpu" and st.shape == (3, 4)
    for r, (s, t) in enumerate(keys):
        state, inc = osamp.pcg_state(s, t)
        got = [int(v) & ((1 << 64) - 1) for v in st[r]]
        assert got == [state >> 64, state & ((1 << 64) - 1), inc >> 64, inc & ((1 << 64) - 1)]
    raw = gpu_pcg.raw_from_state(st, "cuda", n_out=3000)
    assert torch.equal(raw, gpu_pcg.raw_rows(keys, "cuda", n_out=3000))
    want = np.random.default_rng([osamp.SEED_BASE, 5, 77]).bit_generator.random_raw(3000)
    assert np.array_equal(N_(raw[1]).view(np.uint64), want)
