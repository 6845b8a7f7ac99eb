"""IntSampler.apply on the GPU against the CPU oracle's sampler: one logits row per request (host-side generated
index), speculative rows (device positions), the hash log and the RL log-p hook. vLLM's step context and request
state are faked with the attributes the hook reads (src/bitexact/vllm_plugin/sampler.py:153-212)."""

import hashlib
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from oracle import exact as ox
from oracle import sampler as osamp

pytestmark = pytest.mark.gpu


def _want(logits, seeds, ts, temps, lnt, bits):
    out = []
    for r in range(len(seeds)):
        tn, td = temps[r]
        g = osamp.gumbel(osamp.raw_words(int(seeds[r]), int(ts[r]), logits.shape[1]), lnt, bits) if tn else None
        out.append(int(osamp.sample(logits[r:r + 1], tn, td, g)[0]))
    return out


def test_apply_forces_the_integer_token(tmp_path):
    from bitexact_llm_b200.exact.consts import ln_table
    from bitexact_llm_b200.vllm_plugin import rl, sampler as S
    rng = np.random.RandomState(3)
    V, nslot = 5000, 16
    lnt_np = ox.ln_table()
    view = SimpleNamespace(max_num_reqs=nslot, total_len=np.zeros(nslot, dtype=np.int64),
                           prompt_len=SimpleNamespace(np=rng.randint(1, 50, nslot).astype(np.int32)))
    old = (S.STASH.active, S.STASH.logits, S.STASH.head, S.STASH.lnt, S.STASH.fr)
    try:
        S.STASH.active, S.STASH.head, S.STASH.fr = True, None, 16
        S.STASH.lnt = ln_table(device="cuda")
        smp = S.IntSampler(None, view)
        temps = {}
        for slot in range(nslot):
            T = [0.0, 0.7, 1.0, 1.3][slot % 4]
            smp.add_request(slot, SimpleNamespace(seed=(slot * 7919 if slot % 3 else None), temperature=T, logprobs=None))
            temps[slot] = S.temp_ratio(T)
        # ---- one row per request, slots in batch order ----
        slots = np.array([5, 2, 9, 0, 14, 7], dtype=np.int32)
        n = len(slots)
        gen = rng.randint(0, 300, n)
        logits = rng.randint(-(20 << 16), 20 << 16, (n, V)).astype(np.int64)
        logits[3, 100] = logits[3, 4000] = logits[3].max() + 3                       # greedy tie: first index
        S.STASH.logits = torch.from_numpy(logits).cuda()
        ctx = SimpleNamespace(idx_mapping_np=slots,
                              seq_lens_upper_bound_np=(view.prompt_len.np[slots] + gen).astype(np.int32))
        out = torch.randn(n, V, device="cuda")
        smp.lp = []
        res = smp.apply(out, ctx)
        seeds = [int(smp.seed[s]) for s in slots]
        want = _want(logits, seeds, gen, [temps[int(s)] for s in slots], lnt_np, 16)
        got = res.argmax(1).cpu().tolist()
        assert got == want and want[3] == 100
        assert torch.equal((res == 0).sum(1).cpu(), torch.ones(n, dtype=torch.long))
        assert bool(torch.isinf(res).sum() == n * (V - 1))
        lp_seeds, lp_ts, lp = smp.lp[0]
        assert lp_seeds.tolist() == seeds and lp_ts.tolist() == gen.tolist()
        assert torch.equal(lp, rl.int_logp(S.STASH.logits, torch.tensor(want).cuda(), S.STASH.lnt, 16))
        smp.lp = None
        # ---- speculative decoding: several rows per request, t from the device positions; hash log on ----
        rows = np.array([5, 5, 5, 2, 2, 9], dtype=np.int64)
        pos = view.prompt_len.np[rows].astype(np.int64) + np.array([3, 4, 5, -6, 0, 17]) - 1     # one row mid-prompt
        ctx = SimpleNamespace(idx_mapping_np=np.array([5, 2, 9], dtype=np.int32), seq_lens_upper_bound_np=None,
                              expanded_idx_mapping=torch.from_numpy(rows).cuda(), pos=torch.from_numpy(pos).cuda())
        smp.log = str(tmp_path / "hash.log")
        res = smp.apply(torch.zeros(n, V, device="cuda"), ctx)
        ts = pos + 1 - view.prompt_len.np[rows]
        want = _want(logits, [int(smp.seed[s]) for s in rows], np.maximum(ts, 0), [temps[int(s)] for s in rows],
                     lnt_np, 16)
        assert res.argmax(1).cpu().tolist() == want
        lines = open(smp.log).read().split("\n")[:-1]
        assert len(lines) == 5                                                       # the mid-prompt row is left out
        keep = [r for r in range(n) if ts[r] >= 0]
        for line, r in zip(lines, keep):
            sha = hashlib.sha256(logits[r].tobytes()).hexdigest()[:16]
            assert line == "%d %d %s %d" % (smp.seed[rows[r]], ts[r], sha, want[r])
        # ---- switched off: logits untouched ----
        S.STASH.active = False
        x = torch.randn(2, V, device="cuda")
        assert smp.apply(x, ctx) is x
    finally:
        S.STASH.active, S.STASH.logits, S.STASH.head, S.STASH.lnt, S.STASH.fr = old
        S.STASH.sampler = None
