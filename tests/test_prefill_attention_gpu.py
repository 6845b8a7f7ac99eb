"""Prefill attention tile kernel (bx_prefill_attention) against the CPU oracle: prompts of 128 and 2048 tokens
(BASELINE config 3), exact and int8 weight rule, tiles that start mid-prompt (a chunk of a longer prompt: the
cache already holds earlier keys), ragged last tiles, padding rows outside every tile, junk keys beyond the
prompts, scattered pages, page sizes 8 / 16 / 32, G = 1 / 2 / 4, and equality with the per-row decode kernel.
The oracle is row-local, so the 2048-token case checks a seeded sample of token rows over all heads."""

import numpy as np
import pytest
import torch

from oracle import exact as ox
from oracle import int8 as o8

pytestmark = pytest.mark.gpu
HD = 64


def T(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    return (t if dtype is None else t.to(dtype)).cuda()


def _cache(rng, nb, HKV, bs, lim):
    c32 = np.clip(np.rint(rng.standard_normal((nb, HKV, bs, 2 * HD)) * (lim / 3.5)), -lim, lim).astype(np.int64)
    c32[1] = lim
    c32[2] = -lim
    planes = np.zeros((nb, HKV, bs, 8 * HD), dtype=np.int8)
    for part, o in ((c32[..., :HD], 0), (c32[..., HD:], 3)):
        for i, lo in enumerate(ox.split_limbs(part, 3)[0]):
            planes[..., (o + i) * HD:(o + i + 1) * HD] = lo.astype(np.int8)
    planes[..., 6 * HD:] = rng.randint(-128, 128, planes[..., 6 * HD:].shape)          # unused tail of a row: junk
    return planes


def _case(rng, prompts, HKV, G, bs, nb, width):
    """prompts: [(first position, tokens)] per request. Token rows are request-major with `pad` padding rows
    (never in a tile) after every request."""
    from bitexact_llm_b200.vllm_plugin import tri_prefill
    R = len(prompts)
    bt = rng.randint(1, nb, (R, -(-width // bs))).astype(np.int32)
    pre, pos, req, row0 = [], [], [], 0
    for r, (p0, n) in enumerate(prompts):
        pre.append((r, row0, n, p0 + n))
        pos += list(range(p0, p0 + n)) + [0, 0]
        req += [r] * (n + 2)
        row0 += n + 2
    N = row0
    pos, req = np.array(pos, np.int64), np.array(req, np.int64)
    tiles = tri_prefill.tile_table(pre, G)
    live = np.ones(N, bool)
    for r, t0, n, _ in pre:
        live[t0 + n:t0 + n + 2] = False
    return bt, pos, req, tiles, live, N


def _oracle_rows(rows, q, sh, pos, req, planes, bt, lut_np, mode, expt):
    """num / den of the sampled token rows (each row = G queries at one position)."""
    qs = q[rows]
    qpos = np.repeat(pos[rows][:, None], q.shape[2], 1)
    if mode == "exact":
        return ox.paged_attention(qs, sh[rows], qpos, planes, bt, req[rows], lut_np)
    return o8.paged_attention(qs, qpos, planes, bt, req[rows], expt)


@pytest.mark.parametrize("mode", ["exact", "int8"])
@pytest.mark.parametrize("S,HKV,G,bs", [(128, 8, 4, 16), (2048, 2, 4, 16), (77, 3, 2, 8), (300, 2, 1, 32)])
def test_tiles_equal_the_oracle_and_the_row_kernel(mode, S, HKV, G, bs):
    from bitexact_llm_b200.vllm_plugin import tri_exact_attn, tri_paged, tri_prefill
    rng = np.random.RandomState(S + 7 * G + (mode == "int8"))
    nb = 96 if S <= 300 else 400
    lim = 8355711
    planes = _cache(rng, nb, HKV, bs, lim)
    # request 0: the whole prompt; request 1: a chunk that starts mid-prompt; request 2: a short ragged one
    prompts = [(0, S), (S // 3, min(S, 41)), (5, 3)]
    width = max(p0 + n for p0, n in prompts) + 3 * bs
    bt, pos, req, tiles, live, N = _case(rng, prompts, HKV, G, bs, nb, width)
    qlim = 1 << 22 if mode == "exact" else 1 << 13
    q = rng.randint(-qlim, qlim + 1, (N, HKV, G, HD)).astype(np.int64)
    q[0] = qlim
    sh = rng.randint(-34, -16, (N, HKV, G)).astype(np.int64)
    lut_np, expt = ox.exp2_table(), o8.exp_table()
    tl = T(tiles)
    if mode == "exact":
        num, den = tri_prefill.attend_exact(T(q, torch.int32), T(sh), T(pos), T(planes), T(bt), tl, T(lut_np), ox.L2E28)
        n32, d32 = tri_prefill.attend_exact(T(q, torch.int32), T(sh), T(pos), T(planes), T(bt), tl, T(lut_np), ox.L2E28,
                                            rows=32)                      # the 32-row tile height: same integers
        assert torch.equal(n32, num) and torch.equal(d32, den)
    else:
        num = torch.zeros(N, HKV, G, HD, dtype=torch.long, device="cuda")
        den = torch.ones(N, HKV, G, 1, dtype=torch.long, device="cuda")
        tri_prefill.attend(T(q), T(pos), T(planes), T(bt), T(o8.weight_table(expt), torch.int32), tl, num, den)
    torch.cuda.synchronize()
    num, den = num.cpu().numpy(), den.cpu().numpy()
    # padding rows are never written
    assert not num[~live].any() and (den[~live] == 1).all()
    rows = np.flatnonzero(live)
    if len(rows) > 160:                                       # first / last tiles and a seeded sample in between
        pick = np.unique(np.concatenate([rows[:20], rows[-60:], rng.choice(rows, 80, replace=False)]))
    else:
        pick = rows
    wnum, wden = _oracle_rows(pick, q, sh, pos, req, planes, bt, lut_np, mode, expt)
    assert np.array_equal(num[pick], wnum) and np.array_equal(den[pick].reshape(wden.shape), wden), (mode, S)
    # every live row against the per-row decode kernel
    qpos = np.repeat(pos[:, None], G, 1)
    if mode == "exact":
        n2, d2 = tri_exact_attn.attend(T(q, torch.int32), T(sh), T(qpos), T(planes), T(bt), T(req), T(lut_np), ox.L2E28)
    else:
        n2, d2 = tri_paged.attend(T(q), T(qpos), T(planes), T(bt), T(o8.weight_table(expt), torch.int32), rmap=T(req))
    lv = torch.from_numpy(live)
    assert np.array_equal(num[live], n2.cpu()[lv].numpy()) and np.array_equal(den[live], d2.cpu()[lv].numpy())
    from bitexact_llm_b200 import _native as nv
    assert nv.device_status() == 0


def test_tall_tiles_are_cut_and_empty_tile_lists_are_accepted():
    from bitexact_llm_b200.vllm_plugin import tri_prefill
    rng = np.random.RandomState(3)
    HKV, G, bs, nb = 2, 4, 16, 40
    planes = _cache(rng, nb, HKV, bs, 1 << 12)
    bt = rng.randint(1, nb, (1, 8)).astype(np.int32)
    N = 50
    pos = np.arange(N, dtype=np.int64)
    q = rng.randint(-(1 << 13), 1 << 13, (N, HKV, G, HD)).astype(np.int64)
    expt = o8.exp_table()
    ptab = T(o8.weight_table(expt), torch.int32)
    outs = []
    for tiles in (torch.tensor([[0, 0, 50]], dtype=torch.int32),                  # one tile of 50 tokens: cut into 8s
                  tri_prefill.tile_table([(0, 0, 50, 50)], G)):
        num = torch.zeros(N, HKV, G, HD, dtype=torch.long, device="cuda")
        den = torch.ones(N, HKV, G, 1, dtype=torch.long, device="cuda")
        tri_prefill.attend(T(q), T(pos), T(planes), T(bt), ptab, tiles.cuda(), num, den)
        outs.append((num, den))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    wnum, wden = o8.paged_attention(q, np.repeat(pos[:, None], G, 1), planes, bt, np.zeros(N, np.int64), expt)
    assert np.array_equal(outs[0][0].cpu().numpy(), wnum)
    num = torch.zeros(N, HKV, G, HD, dtype=torch.long, device="cuda")
    den = torch.ones(N, HKV, G, 1, dtype=torch.long, device="cuda")
    tri_prefill.attend(T(q), T(pos), T(planes), T(bt), ptab, torch.zeros(0, 3, dtype=torch.int32, device="cuda"), num, den)
    assert not bool(num.any())
