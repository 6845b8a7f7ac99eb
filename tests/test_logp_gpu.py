"""Integer log p on the GPU (through the C ABI) against the reference's golden vectors and the CPU oracle on seeded
rows. Modelled on the reference's tests/test_vllm_kernels.py::test_tri_logp_matches_int_logp."""

import os

import numpy as np
import pytest
import torch

from oracle import exact as ox
from oracle import logp as ol

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def T(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_golden_rows():
    from bitexact_llm_b200.vllm_plugin import rl
    z = np.load(os.path.join(GOLD, "logp.npz"))
    lnt = T(ox.ln_table(40))
    got = rl.int_logp(T(z["logits"]), T(z["tok"]), lnt)
    assert got.dtype == torch.float64 and np.array_equal(got.cpu().numpy(), z["logp"])
    one = rl.int_logp(T(z["logits"][2:3]), T(z["tok"][2:3]), lnt)                 # one row: many column chunks
    assert np.array_equal(one.cpu().numpy(), z["logp"][2:3])


@pytest.mark.parametrize("M,V,fr", [(1, 128256, 16), (5, 128256, 24), (64, 9000, 16), (300, 1000, 13), (3, 1, 16)])
def test_seeded_rows_vs_oracle(M, V, fr):
    from bitexact_llm_b200.vllm_plugin import rl
    g = np.random.default_rng(M * 1000 + V + fr)
    span = 30 << fr
    lg = g.integers(-span, span, (M, V), dtype=np.int64)
    lg[0] = lg[0] >> 9
    if V > 100:
        lg[M // 2, 7] = span * 4                                                   # a peaked row
        lg[-1, ::5] = -(1 << 50)
    tok = g.integers(0, V, M, dtype=np.int64)
    lnt = ox.ln_table(40)
    want = ol.int_logp_q(lg, tok, lnt, fr=fr)
    buf = torch.zeros(M, V + 3, dtype=torch.long, device="cuda")                   # a row stride above V
    buf[:, :V] = T(lg)
    got = rl.int_logp_q(buf[:, :V], T(tok), T(lnt), fr)
    assert np.array_equal(got.cpu().numpy(), want)


def test_token_out_of_range_gives_nan():
    from bitexact_llm_b200.vllm_plugin import rl
    lg = torch.randint(-(1 << 20), 1 << 20, (3, 500), device="cuda")
    got = rl.int_logp(lg, torch.tensor([0, 500, -1], device="cuda"), T(ox.ln_table(40)))
    assert bool(torch.isfinite(got[0])) and bool(torch.isnan(got[1])) and bool(torch.isnan(got[2]))


def test_column_shards_give_the_full_rows_bits():
    """The stepwise entry points over three column shards of one GPU's rows, combined the way the ranks would
    (integer max, integer sum), against the one-call result."""
    from bitexact_llm_b200 import _native as nv
    from bitexact_llm_b200.vllm_plugin import rl
    g = torch.Generator(device="cuda").manual_seed(3)
    M, V = 9, 40000
    lg = torch.randint(-(20 << 16), 20 << 16, (M, V), generator=g, device="cuda")
    tok = torch.randint(0, V, (M,), generator=g, device="cuda")
    lnt, tab = T(ox.ln_table(40)), rl.pair_table(torch.device("cuda"))
    want = rl.int_logp_q(lg, tok, lnt)
    lib, st = nv.lib(), nv.stream()
    shards = [lg[:, a:b].contiguous() for a, b in ((0, 13000), (13000, 13001), (13001, V))]
    scr = [torch.empty(max(1, lib.bx_logp_scratch_bytes(M, s.shape[1])), dtype=torch.uint8, device="cuda") for s in shards]
    mxs = []
    for s, w in zip(shards, scr):
        mx = torch.empty(M, dtype=torch.long, device="cuda")
        nv.check(lib.bx_logp_rowmax(s.data_ptr(), s.stride(0), w.data_ptr(), mx.data_ptr(), M, s.shape[1], st), "rowmax")
        mxs.append(mx)
    mx = torch.stack(mxs).amax(0)
    assert torch.equal(mx, lg.amax(1))
    S = torch.zeros(M, dtype=torch.long, device="cuda")
    for s, w in zip(shards, scr):
        part = torch.empty(M, dtype=torch.long, device="cuda")
        nv.check(lib.bx_logp_rowsum(s.data_ptr(), s.stride(0), mx.data_ptr(), tab.data_ptr(), tab.shape[0], w.data_ptr(),
                                    part.data_ptr(), M, s.shape[1], 16, st), "rowsum")
        S += part
    zt = lg.gather(1, tok[:, None])[:, 0] - mx
    out = torch.empty(M, dtype=torch.long, device="cuda")
    nv.check(lib.bx_logp_finish(S.data_ptr(), zt.data_ptr(), lnt.data_ptr(), out.data_ptr(), M, 16, st), "finish")
    assert torch.equal(out, want)


def test_tri_logp_from_the_head():
    """tri_logp.logp on a Head that carries raw int32 GEMM products (segs.post applied on the way) equals int_logp
    of its logits."""
    from bitexact_llm_b200.vllm_plugin import rl, tri_logp, tri_sample
    g = torch.Generator().manual_seed(9)
    M, V = 6, 5000
    c = torch.randint(-(1 << 24), 1 << 24, (M, V), generator=g, dtype=torch.int32).cuda()
    m = torch.randint(1 << 20, 1 << 23, (V,), generator=g).cuda()
    mant = torch.randint(1 << 23, 1 << 24, (M,), generator=g).cuda()
    e = torch.randint(-6, 2, (M,), generator=g).cuda()
    h = tri_sample.Head(c, m, 10, mant, e)
    tok = torch.randint(0, V, (M,), generator=g).cuda()
    lnt = T(ox.ln_table(40))
    got = tri_logp.logp(h, tok, lnt)
    want = ol.int_logp(h.logits().cpu().numpy(), tok.cpu().numpy(), ox.ln_table(40))
    assert np.array_equal(got.cpu().numpy(), want)
