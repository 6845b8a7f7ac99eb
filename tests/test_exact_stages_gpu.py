"""Exact-mode element-wise stages, paged attention and sampler on the GPU (through the C ABI) against the
golden vectors made by the reference and against the CPU oracle on seeded inputs. Modelled on the reference's
tests/test_vllm_exact_fuse.py, tests/test_vllm_exact_attn.py and tests/test_vllm_kernels.py."""

import os
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from oracle import exact as ox
from oracle import sampler as osamp

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def T(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    return (t if dtype is None else t.to(dtype)).cuda()


def N_(t):
    return t.cpu().numpy()


def flag0():
    return torch.zeros(1, dtype=torch.int32, device="cuda")


def model(D=2048, H=32, HKV=8, HD=64, emb=None, cos=None, sin=None):
    return SimpleNamespace(D=D, H=H, HKV=HKV, HD=HD, emb=emb, cos=cos, sin=sin, dev=torch.device("cuda"))


def test_norm_golden_and_modes():
    from bitexact_llm_b200.vllm_plugin import exact_fuse as fz
    z = np.load(os.path.join(GOLD, "exact_ops.npz"))
    x, gm, ge = T(z["norm_x"]), T(z["norm_gm"]), T(z["norm_ge"])
    m = model(D=x.shape[1])
    fl = flag0()
    q, sh = fz.pre_norm(m, x, (gm, ge), fl)
    assert np.array_equal(N_(q), z["norm_q"]) and np.array_equal(N_(sh), z["norm_sh"]) and fl.item() == 0
    # x + y mode and the 2^40 bound flag
    y = torch.randint(-(1 << 20), 1 << 20, x.shape, device="cuda")
    xo, q2, sh2 = fz.add_norm(m, y, x, (gm, ge), fl)
    wq, wsh, wflag = ox.norm_quant(N_(x + y), z["norm_gm"], z["norm_ge"])
    assert torch.equal(xo, x + y) and np.array_equal(N_(q2), wq) and np.array_equal(N_(sh2), wsh)
    xbig = x.clone()
    xbig[0, 5] = 1 << 40
    fl2 = flag0()
    fz.pre_norm(m, xbig, (gm, ge), fl2)
    assert fl2.item() == 1
    xo, q3, sh3 = fz.add_norm(m, y, x, None, fl)
    assert torch.equal(xo, x + y) and q3 is None
    # embedding gather mode
    emb = torch.randint(-(1 << 26), 1 << 26, (50, x.shape[1]), dtype=torch.int32, device="cuda")
    ids = torch.tensor([3, 49, 0, 3], device="cuda")
    m.emb = emb
    xe, qe, she = fz.embed_norm(m, ids, (gm, ge), fl)
    wq, wsh, _ = ox.norm_quant(N_(emb[ids].long()), z["norm_gm"], z["norm_ge"])
    assert torch.equal(xe, emb[ids].long()) and np.array_equal(N_(qe), wq) and np.array_equal(N_(she), wsh)


@pytest.mark.parametrize("D", [64, 2048, 4096])
def test_norm_seeded(D):
    from bitexact_llm_b200.vllm_plugin import exact_fuse as fz
    rng = np.random.RandomState(D)
    x = rng.randint(-(1 << 30), 1 << 30, (7, D)).astype(np.int64)
    x[1] >>= 25
    x[2] <<= 8
    gbits = (torch.from_numpy(1 + 0.4 * rng.randn(D)).to(torch.bfloat16).view(torch.int16).numpy()).astype(np.uint16)
    gm, ge = ox.bf16_parts(gbits)
    wq, wsh, _ = ox.norm_quant(x, gm, ge)
    q, sh = fz.pre_norm(model(D=D), T(x), (T(gm), T(ge)), flag0())
    assert np.array_equal(N_(q), wq) and np.array_equal(N_(sh), wsh)


def test_qkv_rope_golden_and_cache_store():
    from bitexact_llm_b200.vllm_plugin import exact_fuse as fz
    z = np.load(os.path.join(GOLD, "exact_ops.npz"))
    H, HKV, HD = 4, 2, 64
    m = model(H=H, HKV=HKV, HD=HD, cos=T(z["rope_cos"]), sin=T(z["rope_sin"]))
    y, pos = T(z["rope_y"]), T(z["rope_pos"])
    n = y.shape[0]
    cache = torch.zeros(6, HKV, 16, 8 * HD, dtype=torch.int8, device="cuda")
    slot = torch.tensor([16, 17, -1, 40, 95], device="cuda")
    fl = flag0()
    q, sh = fz.qkv(m, y, pos, slot, cache, fl)
    assert np.array_equal(N_(q).reshape(n, H, HD), z["rope_q"]) and np.array_equal(N_(sh), z["rope_sh"])
    want = np.zeros((6, HKV, 16, 8 * HD), dtype=np.int8)
    ox.cache_store(want, N_(slot), z["rope_k"], z["rope_v"])
    assert np.array_equal(N_(cache), want)
    _, _, _, _, wflag = ox.rope_qkv(z["rope_y"], z["rope_pos"], z["rope_cos"], z["rope_sin"], H, HKV, HD)
    assert bool(fl.item()) == wflag
    q2, sh2 = fz.qkv(m, y, pos, None, None, flag0())
    assert torch.equal(q, q2) and torch.equal(sh, sh2)
    # stand-alone store
    from bitexact_llm_b200.vllm_plugin import tri_paged
    c2 = torch.zeros_like(cache)
    tri_paged.store(c2, slot, T(z["rope_k"]), T(z["rope_v"]))
    assert torch.equal(c2, cache)
    ybig = y.clone()
    ybig[1, 7] = 1 << 31
    fl3 = flag0()
    fz.qkv(m, ybig, pos, None, None, fl3)
    assert fl3.item() == 1


def test_silu_golden_and_full_width():
    from bitexact_llm_b200.vllm_plugin import exact_fuse as fz
    z = np.load(os.path.join(GOLD, "exact_ops.npz"))
    lut = T(ox.exp2_table())
    fl = flag0()
    q, sh = fz.silu_quant(model(), T(z["silu_y"]), lut, fl)
    assert np.array_equal(N_(q), z["silu_q"]) and np.array_equal(N_(sh), z["silu_sh"])
    assert bool(fl.item()) == bool(z["silu_err"])
    rng = np.random.RandomState(3)
    y = rng.randint(-(20 << 24), 20 << 24, (3, 2 * 8192)).astype(np.int64)
    wq, wsh, werr = ox.silu_quant(y, ox.exp2_table())
    fl = flag0()
    q, sh = fz.silu_quant(model(), T(y), lut, fl)
    assert np.array_equal(N_(q), wq) and np.array_equal(N_(sh), wsh) and bool(fl.item()) == werr
    y[1, 5] = (1 << 32) + 1                                    # gate bound
    fl = flag0()
    fz.silu_quant(model(), T(y), lut, fl)
    assert fl.item() == 1


def test_attention_golden_all_cluster_sizes():
    from bitexact_llm_b200 import _native as nv
    from bitexact_llm_b200.vllm_plugin import exact_fuse as fz
    from bitexact_llm_b200.vllm_plugin import tri_exact_attn
    z = np.load(os.path.join(GOLD, "exact_ops.npz"))
    lut = T(ox.exp2_table())
    R = z["attn_q"].shape[0]
    args = (T(z["attn_q"], torch.int32), T(z["attn_sh"]), T(z["attn_qpos"]), T(z["attn_cache"]), T(z["attn_bt"]),
            torch.arange(R, device="cuda"), lut, ox.L2E28)
    # direct-load, TMA-staged, TMA + tcgen05 p.V (8 / 4 warps), persistent streaming (8 / 4 warps)
    for variant in (1, 2, 3, 4, 5, 6):
        for ns in (None, 1, 2, 5, 64):
            num, den = tri_exact_attn.attend(*args, nsplit=ns, variant=variant)
            assert np.array_equal(N_(num), z["attn_num"]) and np.array_equal(N_(den), z["attn_den"]), (variant, ns)
    m = model(H=8, HKV=2, HD=64)
    qo, sho = fz.attn_out(m, num, den)
    assert np.array_equal(N_(qo), z["attn_qo"]) and np.array_equal(N_(sho), z["attn_sho"])
    assert nv.device_status() == 0


@pytest.mark.parametrize("lim", [8355711, 1 << 13, 1 << 10])
def test_attention_seeded_random_masks_and_padding(lim):
    """Random per-query positions (causal masks), M in 1..4, int64 block tables, shared block-table rows (rmap),
    junk keys beyond qpos, contexts from 5 to 3000 keys."""
    from bitexact_llm_b200.vllm_plugin import tri_exact_attn
    rng = np.random.RandomState(lim % 1000)
    nb, bs, HKV, HD = 96, 16, 8, 64
    c32 = rng.randint(-lim, lim + 1, (nb, HKV, bs, 2 * HD)).astype(np.int64)
    planes = np.zeros((nb, HKV, bs, 8 * HD), dtype=np.int8)
    for part, o in ((c32[..., :HD], 0), (c32[..., HD:], 3)):
        for i, lo in enumerate(ox.split_limbs(part, 3)[0]):
            planes[..., (o + i) * HD:(o + i + 1) * HD] = lo.astype(np.int8)
    planes[..., 6 * HD:] = rng.randint(-128, 128, planes[..., 6 * HD:].shape)      # unused tail: junk
    lut_np = ox.exp2_table()
    lut = T(lut_np)
    for R, M, P, bt_dtype in [(3, 4, 600, np.int32), (5, 4, 3000, np.int64), (6, 1, 900, np.int32), (2, 3, 50, np.int32),
                              (7, 4, 5, np.int64)]:
        bt = rng.randint(1, nb, (R + 2, 200)).astype(bt_dtype)
        rmap = rng.randint(0, R + 2, R).astype(np.int64)
        qpos = rng.randint(0, P, (R, M)).astype(np.int64)
        q = rng.randint(-(1 << 22), (1 << 22) + 1, (R, HKV, M, HD)).astype(np.int64)
        sh = rng.randint(-40, -10, (R, HKV, M)).astype(np.int64)
        wnum, wden = ox.paged_attention(q, sh, qpos, planes, bt, rmap, lut_np)
        for variant, ns in ((1, None), (1, 8), (2, None), (2, 4), (3, None), (3, 4), (4, None), (4, 1), (4, 2), (4, 8), (5, None), (6, None)):
            num, den = tri_exact_attn.attend(T(q, torch.int32), T(sh), T(qpos), T(planes), T(bt), T(rmap), lut,
                                             ox.L2E28, nsplit=ns, variant=variant)
            assert np.array_equal(N_(num), wnum) and np.array_equal(N_(den), wden), (R, M, P, variant, ns)


@pytest.mark.parametrize("lim", [8355711, 1 << 10])
def test_attention_persistent_streaming(lim):
    """The persistent kernels (a CTA walks many (request, KV head) pairs with one TMA ring): more pairs than CTAs,
    page sizes 8 / 16 / 32, block tables just wide enough and much wider than the contexts, ragged positions."""
    from bitexact_llm_b200.vllm_plugin import tri_exact_attn
    rng = np.random.RandomState(7 + lim % 1000)
    HKV, HD = 8, 64
    lut_np = ox.exp2_table()
    lut = T(lut_np)
    for bs in (16, 8, 32):
        nb = 1536 // bs
        c32 = rng.randint(-lim, lim + 1, (nb, HKV, bs, 2 * HD)).astype(np.int64)
        planes = np.zeros((nb, HKV, bs, 8 * HD), dtype=np.int8)
        for part, o in ((c32[..., :HD], 0), (c32[..., HD:], 3)):
            for i, lo in enumerate(ox.split_limbs(part, 3)[0]):
                planes[..., (o + i) * HD:(o + i + 1) * HD] = lo.astype(np.int8)
        planes[..., 6 * HD:] = rng.randint(-128, 128, planes[..., 6 * HD:].shape)
        for R, M, P, width in [(3, 4, 600, 640), (5, 4, 2040, 2048), (90, 1, 300, 1024), (2, 3, 50, 64), (7, 4, 5, 32),
                               (80, 4, 544, 544), (3, 2, 100, 4000)]:
            bt = rng.randint(1, nb, (R + 2, -(-width // bs))).astype(np.int32)
            rmap = rng.randint(0, R + 2, R).astype(np.int64)
            qpos = rng.randint(0, P, (R, M)).astype(np.int64)
            q = rng.randint(-(1 << 22), (1 << 22) + 1, (R, HKV, M, HD)).astype(np.int64)
            sh = rng.randint(-40, -10, (R, HKV, M)).astype(np.int64)
            wnum, wden = ox.paged_attention(q, sh, qpos, planes, bt, rmap, lut_np)
            for variant in (5, 6):
                num, den = tri_exact_attn.attend(T(q, torch.int32), T(sh), T(qpos), T(planes), T(bt), T(rmap), lut,
                                                 ox.L2E28, variant=variant)
                assert np.array_equal(N_(num), wnum) and np.array_equal(N_(den), wden), (bs, R, M, P, width, variant)
    from bitexact_llm_b200 import _native as nv
    assert nv.device_status() == 0


def test_attention_long_contexts_with_score_scratch():
    """Enough pairs for the persistent kernel and block tables wider than its shared-memory score buffer: the scores of
    long pairs live in the scratch buffer and sweep 2 runs in chunks of 512 keys (contexts from 3 to 3000 keys in one
    batch, chunk boundaries hit exactly, requests ranked by length)."""
    from bitexact_llm_b200.vllm_plugin import tri_exact_attn, tri_paged
    rng = np.random.RandomState(77)
    nb, bs, HKV, HD = 220, 16, 8, 64
    lim = 1 << 12
    c32 = rng.randint(-lim, lim + 1, (nb, HKV, bs, 2 * HD)).astype(np.int64)
    planes = np.zeros((nb, HKV, bs, 8 * HD), dtype=np.int8)
    for part, o in ((c32[..., :HD], 0), (c32[..., HD:], 3)):
        for i, lo in enumerate(ox.split_limbs(part, 3)[0]):
            planes[..., (o + i) * HD:(o + i + 1) * HD] = lo.astype(np.int8)
    lut_np = ox.exp2_table()
    R, M = 40, 4
    bt = rng.randint(1, nb, (R, 192)).astype(np.int32)                     # 3072 keys wide
    ctx = rng.randint(3, 3001, R)
    ctx[:6] = [512, 513, 1024, 1025, 3000, 511]
    qpos = np.repeat((ctx - 1)[:, None], M, 1).astype(np.int64)
    qpos[7, 1] = 5                                                          # one query of a long row sees few keys
    q = rng.randint(-(1 << 22), (1 << 22) + 1, (R, HKV, M, HD)).astype(np.int64)
    sh = rng.randint(-40, -10, (R, HKV, M)).astype(np.int64)
    wnum, wden = ox.paged_attention(q, sh, qpos, planes, bt, np.arange(R), lut_np)
    for variant in (0, 6, 5):
        num, den = tri_exact_attn.attend(T(q, torch.int32), T(sh), T(qpos), T(planes), T(bt), None, T(lut_np), ox.L2E28,
                                         variant=variant)
        assert np.array_equal(N_(num), wnum) and np.array_equal(N_(den), wden), variant
    from oracle import int8 as o8
    expt = o8.exp_table()
    w8n, w8d = o8.paged_attention(q >> 9, qpos, planes, bt, np.arange(R), expt)
    num, den = tri_paged.attend(T(q >> 9), T(qpos), T(planes), T(bt), T(o8.weight_table(expt), torch.int32))
    assert np.array_equal(N_(num), w8n) and np.array_equal(N_(den), w8d)
    from bitexact_llm_b200 import _native as nv
    assert nv.device_status() == 0


def test_attention_decode_batch_with_contexts_up_to_8192_keys():
    """A decode batch of 48 requests x 8 KV heads (enough pairs for the persistent streaming kernel) whose contexts
    run from 64 to 8192 keys, a few at 4096 .. 8192 among short ones, random pages, per-query positions that differ
    inside a request: the automatic choice and both streaming variants, exact and int8 weight rule, full-range
    values (|K|, |V| up to three limbs)."""
    from bitexact_llm_b200.vllm_plugin import tri_exact_attn, tri_paged
    rng = np.random.RandomState(8192)
    nb, bs, HKV, HD = 640, 16, 8, 64
    lim = 8355711
    c32 = np.clip(np.rint(rng.standard_normal((nb, HKV, bs, 2 * HD)) * (1 << 19)), -lim, lim).astype(np.int64)
    c32[5] = lim
    c32[6] = -lim
    planes = np.zeros((nb, HKV, bs, 8 * HD), dtype=np.int8)
    for part, o in ((c32[..., :HD], 0), (c32[..., HD:], 3)):
        for i, lo in enumerate(ox.split_limbs(part, 3)[0]):
            planes[..., (o + i) * HD:(o + i + 1) * HD] = lo.astype(np.int8)
    planes[..., 6 * HD:] = rng.randint(-128, 128, planes[..., 6 * HD:].shape)
    lut_np = ox.exp2_table()
    R, M = 48, 4
    bt = rng.randint(1, nb, (R, 512)).astype(np.int32)                     # 8192 keys wide
    ctx = rng.randint(64, 700, R)
    ctx[[3, 11, 19, 30, 41]] = [8192, 4096, 4097, 6000, 7681]
    qpos = np.repeat((ctx - 1)[:, None], M, 1).astype(np.int64)
    qpos[3, 2], qpos[30, 0] = 100, 5999 - 513
    q = rng.randint(-(1 << 22), (1 << 22) + 1, (R, HKV, M, HD)).astype(np.int64)
    sh = rng.randint(-34, -16, (R, HKV, M)).astype(np.int64)
    wnum, wden = ox.paged_attention(q, sh, qpos, planes, bt, np.arange(R), lut_np)
    for variant in (0, 6, 5):
        num, den = tri_exact_attn.attend(T(q, torch.int32), T(sh), T(qpos), T(planes), T(bt), None, T(lut_np), ox.L2E28,
                                         variant=variant)
        assert np.array_equal(N_(num), wnum) and np.array_equal(N_(den), wden), variant
    from oracle import int8 as o8
    expt = o8.exp_table()
    q8 = q >> 8
    w8n, w8d = o8.paged_attention(q8, qpos, planes, bt, np.arange(R), expt)
    for variant in (0, 6, 5):
        num, den = tri_paged.attend(T(q8), T(qpos), T(planes), T(bt), T(o8.weight_table(expt), torch.int32),
                                    variant=variant)
        assert np.array_equal(N_(num), w8n) and np.array_equal(N_(den), w8d), variant
    from bitexact_llm_b200 import _native as nv
    assert nv.device_status() == 0


def test_attention_bound_stress_equal_scores_at_limb_extremes():
    """All K, V at +LIM3, all q at 2^22, 8192 equal-score keys (the p.V partial-sum bound case)."""
    from bitexact_llm_b200.vllm_plugin import tri_exact_attn
    nb, bs, HKV, HD, S = 520, 16, 1, 64, 8192
    c32 = np.full((nb, HKV, bs, 2 * HD), 8355711, dtype=np.int64)
    planes = np.zeros((nb, HKV, bs, 8 * HD), dtype=np.int8)
    for part, o in ((c32[..., :HD], 0), (c32[..., HD:], 3)):
        for i, lo in enumerate(ox.split_limbs(part, 3)[0]):
            planes[..., (o + i) * HD:(o + i + 1) * HD] = lo.astype(np.int8)
    bt = np.arange(1, 513, dtype=np.int32)[None]
    q = np.full((1, HKV, 4, HD), 1 << 22, dtype=np.int64)
    sh = np.full((1, HKV, 4), -30, dtype=np.int64)
    qpos = np.full((1, 4), S - 1, dtype=np.int64)
    for variant in (1, 2, 3, 4):
        num, den = tri_exact_attn.attend(T(q, torch.int32), T(sh), T(qpos), T(planes), T(bt), None,
                                         T(ox.exp2_table()), ox.L2E28, variant=variant)
        assert int(den.min()) == S << 22 and int(num.min()) == (S << 22) * 8355711 and int(num.max()) == int(num.min())
    assert int(den.min()) == S << 22 and int(num.min()) == (S << 22) * 8355711 and int(num.max()) == int(num.min())


def test_pcg_words_and_sampler():
    from bitexact_llm_b200.exact.consts import ln_table
    from bitexact_llm_b200.vllm_plugin import gpu_pcg, sampler
    keys = [(0, 0), (1, 0), (7, 33), (123456, 255), (2 ** 31 + 5, 4000), (2 ** 40 + 3, 2 ** 33)]
    raw = gpu_pcg.raw_rows(keys, "cuda", n_out=5000)
    for r, (s, t) in enumerate(keys):
        want = np.random.default_rng([osamp.SEED_BASE, s, t]).bit_generator.random_raw(5000)
        assert np.array_equal(N_(raw[r]).view(np.uint64), want), (s, t)
    z = np.load(os.path.join(GOLD, "sampler.npz"))
    lnt = ln_table(device="cuda")
    li = T(z["logits"])
    gk = [tuple(int(v) for v in k) for k in z["keys"]]
    assert np.array_equal(N_(sampler.first_argmax(li)), z["tok_greedy"])
    # golden row 0 has patched raw words, so compare rows 1.. of the golden and every row with the oracle
    tok = sampler.integer_sample(li, [k[0] for k in gk], [k[1] for k in gk], [(7, 10)] * 4, lnt)
    assert np.array_equal(N_(tok)[1:], z["tok_t07"][1:])
    V = 128256
    rng = np.random.RandomState(9)
    logits = rng.randint(-(25 << 24), 25 << 24, (5, V)).astype(np.int64)
    logits[3, 777] = logits[3, 90000] = logits[3].max() + 11
    seeds, ts = [0, 1, 2, 3, 4], [0, 5, 255, 9, 1]
    temps = [(7, 10), (0, 1), (13, 10), (0, 1), (1, 1)]
    lnt_np = ox.ln_table()
    want = []
    for r in range(5):
        tn, td = temps[r]
        g = osamp.gumbel(osamp.raw_words(seeds[r], ts[r], V), lnt_np, 24) if tn else None
        want.append(int(osamp.sample(logits[r:r + 1], tn, td, g)[0]))
    tok = sampler.integer_sample(T(logits), seeds, ts, temps, lnt)
    assert N_(tok).tolist() == want and want[3] == 777


def test_sharded_sampler_pairs_combine_to_the_full_row_token():
    """Eight vocabulary shards, each reduced to (max, first global index) by bx_sample_shard, combine to exactly the
    token bx_sample picks on the full row (greedy and T = 0.7; a tie across shards resolves to the first index)."""
    from bitexact_llm_b200 import _native as nv
    from bitexact_llm_b200.exact.consts import ln_table
    from bitexact_llm_b200.vllm_plugin import sampler
    lib = nv.lib()
    V, M, W = 128256, 6, 8
    g = torch.Generator(device="cuda").manual_seed(4)
    li = torch.randint(-(25 << 24), 25 << 24, (M, V), device="cuda", generator=g)
    li[2, 100] = li[2, 90000] = li[2].max() + 7
    rows = torch.tensor([[r, 3 + r, (0 if r % 2 else 7), (1 if r % 2 else 10)] for r in range(M)], device="cuda")
    lnt = ln_table(device="cuda")
    want = sampler.sample_rows(li, rows, lnt)
    per = V // W
    best = torch.empty(W, M, dtype=torch.long, device="cuda")
    idx = torch.empty(W, M, dtype=torch.long, device="cuda")
    scratch = torch.empty(lib.bx_sample_scratch_bytes(M, per), dtype=torch.uint8, device="cuda")
    for s in range(W):
        loc = li[:, s * per:(s + 1) * per]                              # a strided view: ld = V
        rc = lib.bx_sample_shard(loc.data_ptr(), loc.stride(0), rows.data_ptr(), lnt.data_ptr(), scratch.data_ptr(),
                                 best[s].data_ptr(), idx[s].data_ptr(), M, per, s * per, 24, nv.stream())
        assert rc == 0
    top = best.amax(0, keepdim=True)
    tok = torch.where(best == top, idx, torch.full_like(idx, 1 << 62)).amin(0)
    assert torch.equal(tok, want) and int(tok[2]) in (100, int(want[2]))


def test_sampler_pruning_keeps_the_first_maximum():
    """Rows built to stress the exact pruning of the sampler: flat logits (the noise alone decides), a narrow band,
    a dominant logit, huge spread, duplicated maxima of logit + noise, 16 and 24 fractional bits, many temperatures,
    vocabulary sizes that leave ragged warps."""
    from bitexact_llm_b200.exact.consts import ln_table
    from bitexact_llm_b200.vllm_plugin import sampler
    lnt = ln_table(device="cuda")
    lnt_np = ox.ln_table()
    rng = np.random.RandomState(21)
    for V, bits in ((128256, 24), (50001, 16), (777, 24)):
        rows = []
        for kind in range(6):
            if kind == 0:
                li = np.zeros(V, dtype=np.int64)
            elif kind == 1:
                li = rng.randint(-(1 << (bits - 4)), 1 << (bits - 4), V).astype(np.int64)
            elif kind == 2:
                li = rng.randint(-(3 << bits), 3 << bits, V).astype(np.int64)
                li[V // 3] = 40 << bits
            elif kind == 3:
                li = rng.randint(-(1 << 40), 1 << 40, V).astype(np.int64)
            elif kind == 4:
                li = np.full(V, 5 << bits, dtype=np.int64)
                li[::7] -= 1
            else:
                li = (rng.standard_normal(V) * (1 << bits)).astype(np.int64)
            rows.append(li)
        logits = np.stack(rows)
        seeds = [3, 1 << 33, 5, 6, 7, 123456789]
        ts = [0, 1, 2, 70000, 4, 5]
        temps = [(7, 10), (1, 1), (13, 10), (1, 3), (5, 2), (7, 10)]
        want = []
        for r in range(len(rows)):
            raw = np.random.default_rng([osamp.SEED_BASE, seeds[r], ts[r]]).bit_generator.random_raw(V).view(np.int64)
            g = osamp.gumbel(raw, lnt_np, bits)
            want.append(int(osamp.sample(logits[r:r + 1], temps[r][0], temps[r][1], g)[0]))
        tok = sampler.integer_sample(T(logits), seeds, ts, temps, lnt, fr=bits)
        assert N_(tok).tolist() == want, (V, bits)


def test_two_step_silu_equals_the_fused_kernel_for_any_column_split():
    """bx_exact_silu_prod per column shard + the maximum of the shard row maxima + bx_exact_quant_rows give the q and
    sh of exact_fuse.silu_quant on the full row (what the column-sharded MLP does across GPUs)."""
    from bitexact_llm_b200 import _native as nv
    from bitexact_llm_b200.vllm_plugin import exact_fuse as fz
    lib = nv.lib()
    rng = np.random.RandomState(31)
    lut = T(ox.exp2_table())
    for N, FF, parts in ((5, 8192, 4), (3, 256, 2), (9, 48, 3)):
        y = rng.randint(-(1 << 27), 1 << 27, (N, 2 * FF)).astype(np.int64)
        y[0, :FF] = 0                                                     # a row whose product is all zero
        y[1, 3] = 70 << 24                                                # beyond the clamp of |g|
        fl = flag0()
        q_full, sh_full = fz.silu_quant(model(), T(y), lut, fl)
        wq, wsh, wflag = ox.silu_quant(y, ox.exp2_table())
        assert np.array_equal(N_(q_full), wq) and np.array_equal(N_(sh_full), wsh)
        bounds = np.linspace(0, FF, parts + 1).astype(int)
        Ps, rmaxes = [], []
        fl2 = flag0()
        for a, b in zip(bounds[:-1], bounds[1:]):
            yl = T(np.concatenate([y[:, a:b], y[:, FF + a:FF + b]], 1))
            P = torch.empty(N, b - a, dtype=torch.long, device="cuda")
            rmax = torch.empty(N, dtype=torch.long, device="cuda")
            nv.check(lib.bx_exact_silu_prod(yl.data_ptr(), lut.data_ptr(), P.data_ptr(), rmax.data_ptr(), fl2.data_ptr(),
                                            N, b - a, nv.stream()), "prod")
            Ps.append(P)
            rmaxes.append(rmax)
        rmax = torch.stack(rmaxes).amax(0).contiguous()
        q = torch.empty(N, FF, dtype=torch.int32, device="cuda")
        planes = torch.zeros(3, N, FF, dtype=torch.int8, device="cuda")
        sh = torch.empty(N, dtype=torch.long, device="cuda")
        for (a, b), P in zip(zip(bounds[:-1], bounds[1:]), Ps):
            nv.check(lib.bx_exact_quant_rows(P.data_ptr(), rmax.data_ptr(), 48, q[:, a:].data_ptr(), FF, sh.data_ptr(),
                                             planes[:, :, a:].data_ptr(), N * FF, N, int(b - a), nv.stream()), "quant")
        assert np.array_equal(N_(q), wq) and np.array_equal(N_(sh), wsh) and int(fl2) == int(fl)
        assert np.array_equal(N_(planes), N_(fz.planes_of(q_full, N, FF)))


def test_limb_planes_attached_to_q_are_dropped_when_q_is_edited_in_place():
    """A stage kernel hands its limb planes to the next fused linear through q. A caller that edits q in place
    afterwards (masking, padding rows) must get the product of the edited q, not of the stale planes."""
    from bitexact_llm_b200.exact.consts import decompose
    from bitexact_llm_b200.exact.model import Lin
    from bitexact_llm_b200.vllm_plugin import exact_fuse
    from bitexact_llm_b200.vllm_plugin.exact_gemm import FusedLin
    g = torch.Generator().manual_seed(4)
    dec = decompose((torch.randn(256, 128, generator=g) * 0.02).to(torch.bfloat16).cuda())
    lin = FusedLin(Lin(dec, None, "cuda"))
    m = model(D=128)
    x = torch.randint(-(1 << 30), 1 << 30, (6, 128), generator=g).cuda()
    gm, ge = torch.full((128,), 128, device="cuda"), torch.full((128,), -7, device="cuda")
    q, sh = exact_fuse.pre_norm(m, x, (gm, ge), flag0())
    assert exact_fuse.planes_of(q, 6, 128) is not None
    y0 = lin(q, sh, flag0(), True)
    q[2:4] = 0                                                     # in-place edit: the planes no longer describe q
    assert exact_fuse.planes_of(q, 6, 128) is None
    y1 = lin(q, sh, flag0(), True)
    assert bool((y1[2:4] == 0).all()) and torch.equal(y1[:2], y0[:2]) and torch.equal(y1[4:], y0[4:])
    want, _ = ox.linear(N_(q).astype(np.int64), N_(sh), {k: N_(v) for k, v in dec.items()}, checked=True)
    assert np.array_equal(N_(y1), want)
