"""One decoder layer + final norm + LM head + sampler at the full Llama-3.2-1B geometry (hidden 2048, 32 : 8 heads,
FF 8192, vocabulary 128,256) on the GPU against the CPU oracle: residual rows, every logits row and the tokens
(greedy and T = 0.7) must be equal bit for bit, and the same rows must give the same bits alone, inside a batch of
256 with other sequences, and in a permuted order (the reference's batch verification, src/bitexact/repro.py:190-212,
and tests/test_invariance.py:47-61). Exact and int8 mode."""

import numpy as np
import pytest
import torch

from oracle import step_sample
from oracle.model import OracleInt8Model, OracleModel

pytestmark = pytest.mark.gpu
ROWS, CTX = 64, 640


def _np(c):
    return {k: (v.cpu().numpy() if torch.is_tensor(v) else v) for k, v in c.items()}


def _load(ses, sample, seqs):
    for r, b in enumerate(seqs):
        ses.import_kv(int(b), torch.from_numpy(sample["k"][r]), torch.from_numpy(sample["v"][r]))


def _step(eng, ses, sample, seqs, B):
    """One decode step of the session's B sequences; rows `seqs` carry the sample, the rest their own filler."""
    ids = torch.zeros(B, dtype=torch.long, device="cuda")
    ids[torch.as_tensor(seqs, device="cuda")] = torch.from_numpy(sample["ids"]).cuda()
    x = ses.step(ids)
    return x, eng.logits(x)


@pytest.fixture(scope="module")
def exact_1b():
    from bitexact_llm_b200.exact import consts
    from bitexact_llm_b200.vllm_plugin.exact_run import ExactEngine
    cfg = dict(consts.LLAMA_1B)
    cfg["num_hidden_layers"] = 1
    c = consts.build(cfg, consts.random_state_dict(cfg, seed=0, device="cuda"), n_pos=CTX + 512)
    eng = ExactEngine(c, "cuda")
    m = OracleModel(_np(c))
    sample = step_sample.make_sample(cfg, ROWS, CTX, seed=0)
    x, lg = step_sample.run_oracle(m, sample)
    assert not m.flag
    return eng, m, cfg, sample, x, lg


def test_exact_layer_and_head_equal_the_oracle(exact_1b):
    from bitexact_llm_b200.decode import Session
    from bitexact_llm_b200.vllm_plugin import sampler
    eng, m, cfg, sample, wx, wlg = exact_1b
    ses = Session(eng, ROWS, CTX + 64)
    _load(ses, sample, range(ROWS))
    x, lg = _step(eng, ses, sample, list(range(ROWS)), ROWS)
    assert np.array_equal(x.cpu().numpy(), wx)
    assert np.array_equal(lg.cpu().numpy(), wlg)
    seeds = list(range(100, 100 + ROWS))
    for tn, td in ((0, 1), (7, 10)):
        rows = torch.tensor([[s, 3, tn, td] for s in seeds], device="cuda")
        tok = sampler.sample_rows(lg, rows, eng.ln, eng.FR)
        assert tok.cpu().tolist() == step_sample.oracle_tokens(m, wlg, seeds, 3, tn, td).tolist(), (tn, td)
    eng.check()


def test_exact_rows_inside_a_batch_of_256_and_permuted(exact_1b):
    from bitexact_llm_b200.decode import Session
    eng, m, cfg, sample, wx, wlg = exact_1b
    B = 256
    filler = step_sample.make_sample(cfg, B - ROWS, CTX, seed=7, spread=300)
    perm = np.random.RandomState(3).permutation(B)
    seqs, others = perm[:ROWS], perm[ROWS:]
    ses = Session(eng, B, CTX + 400, perm_seed=5)                  # scattered pages
    _load(ses, sample, seqs)
    _load(ses, filler, others)
    ids = torch.zeros(B, dtype=torch.long)
    ids[torch.from_numpy(seqs)] = torch.from_numpy(sample["ids"])
    ids[torch.from_numpy(others)] = torch.from_numpy(filler["ids"])
    x = ses.step(ids.cuda())
    lg = eng.logits(x)
    sel = torch.from_numpy(seqs).cuda()
    assert np.array_equal(x[sel].cpu().numpy(), wx)
    assert np.array_equal(lg[sel].cpu().numpy(), wlg)
    eng.check()


def test_int8_layer_and_head_equal_the_oracle():
    from bitexact_llm_b200.decode import Session
    from bitexact_llm_b200.exact import consts
    from bitexact_llm_b200.int8 import consts as consts8
    from bitexact_llm_b200.int8.engine import IntEngine
    from bitexact_llm_b200.vllm_plugin import sampler
    cfg = dict(consts.LLAMA_1B)
    cfg["num_hidden_layers"] = 1
    c = consts8.build(cfg, consts.random_state_dict(cfg, seed=1, device="cuda"), n_pos=2048)
    eng = IntEngine(c, "cuda")
    m = OracleInt8Model(_np(c))
    sample = step_sample.make_sample(cfg, 32, 300, seed=2)
    sample["k"] = [k >> 3 for k in sample["k"]]                    # int8 mode keeps k and v at 14 fractional bits
    sample["v"] = [v >> 5 for v in sample["v"]]
    wx, wlg = step_sample.run_oracle(m, sample)
    assert not m.flag
    for B, seqs in ((32, np.arange(32)), (96, np.random.RandomState(1).permutation(96)[:32])):
        ses = Session(eng, B, 400, perm_seed=B)
        _load(ses, sample, seqs)
        x, lg = _step(eng, ses, sample, seqs.tolist(), B)
        sel = torch.from_numpy(seqs).cuda()
        assert np.array_equal(x[sel].cpu().numpy(), wx), B
        assert np.array_equal(lg[sel].cpu().numpy(), wlg), B
    rows = torch.tensor([[s, 0, 0, 1] for s in range(32)], device="cuda")
    tok = sampler.sample_rows(lg[sel], rows, eng.ln, eng.FR)
    assert tok.cpu().tolist() == np.argmax(wlg, 1).tolist()
    eng.check()
