"""A generation driven the way vLLM drives the plugin (src/bitexact/vllm_plugin/model.py, sampler.py): flat token
batches with attention metadata -> ModelGlue.forward -> compute_logits -> IntSampler.apply on vLLM's float rows ->
argmax. Mixed prompt chunks and decode rows in one step, padding rows, greedy / temperature / strict requests: the
tokens equal the reference's for the tiny model (tests/golden/tiny_model.npz)."""

import os
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


class _Table:
    """Stands for the model runner's request table: shares `total_len` with the processor's view."""

    def __init__(self, total_len, index):
        self.total_len = total_len
        self.req_id_to_index = index


def _engine():
    from make_golden import TINY, TINY_PROMPTS, tiny_state_dict
    from bitexact_llm_b200.exact import consts
    from bitexact_llm_b200.vllm_plugin.exact_run import ExactEngine
    z = np.load(os.path.join(GOLD, "tiny_model.npz"))
    tables = {"cos": torch.zeros(4096, 32, dtype=torch.long), "sin": torch.zeros(4096, 32, dtype=torch.long)}
    tables["cos"][:128], tables["sin"][:128] = torch.from_numpy(z["cos"]), torch.from_numpy(z["sin"])
    return ExactEngine(consts.build(TINY, tiny_state_dict(), tables=tables), "cuda"), z, TINY_PROMPTS


@pytest.mark.parametrize("mode,strict", [("greedy", False), ("t07", False), ("t07", True)])
def test_generation_through_the_vllm_hooks(mode, strict):
    from bitexact_llm_b200.vllm_plugin import sampler as S
    from bitexact_llm_b200.vllm_plugin.model import ModelGlue
    eng, z, prompts = _engine()
    old = (S.STASH.active, S.STASH.sampler)
    try:
        glue = ModelGlue(eng)
        R, bs, nblk, NEW = len(prompts), 16, 4, 8
        plen = np.array([len(p) for p in prompts], dtype=np.int32)
        view = SimpleNamespace(max_num_reqs=R, total_len=np.zeros(R, dtype=np.int64), prompt_len=SimpleNamespace(np=plen))
        table = _Table(view.total_len, {f"r{i}": i for i in range(R)})
        smp = S.IntSampler(None, view)
        for i in range(R):
            smp.add_request(i, SimpleNamespace(seed=i, temperature=0.0 if mode == "greedy" else 0.7,
                                               logprobs=1 if strict else None))
        assert smp.any_strict() == strict and smp.any_noisy() == (mode != "greedy")
        kvs = [torch.zeros(1 + R * nblk, eng.HKV, bs, 8 * eng.HD, dtype=torch.int8, device="cuda") for _ in range(eng.L)]
        perm = torch.randperm(R * nblk, generator=torch.Generator().manual_seed(4)) + 1      # block 0 is the null block
        bt = perm.view(R, nblk).cuda()
        done = np.zeros(R, dtype=np.int64)                 # tokens of each request already in the cache
        seqs = [list(p) for p in prompts]
        out_tok = [[] for _ in range(R)]
        chunk = 5                                           # prompt tokens per request and step: chunked prompts
        while min(len(t) for t in out_tok) < NEW:
            ids, pos, slot, qsl, lens, live = [], [], [], [0], [], []
            for r in range(R):
                if len(out_tok[r]) >= NEW:
                    continue
                take = min(chunk, len(seqs[r]) - done[r])
                for t in range(done[r], done[r] + take):
                    ids.append(seqs[r][t]); pos.append(t)
                    slot.append(int(perm[r * nblk + t // bs]) * bs + t % bs)
                done[r] += take
                qsl.append(len(ids)); lens.append(int(done[r])); live.append(r)
            n, pad = len(ids), 3                            # three padding rows behind the real ones
            T = lambda v: torch.tensor(v + [0] * pad, dtype=torch.long, device="cuda")
            meta = SimpleNamespace(query_start_loc=torch.tensor(qsl), seq_lens=lens, slot_mapping=T(slot),
                                   block_table=bt[live])
            x = glue.forward(T(ids), T(pos), meta, kvs)
            last = torch.tensor([q - 1 for q in qsl[1:]], device="cuda")
            f = glue.compute_logits(x[last])
            if strict:                                      # vLLM's real float logits: li * 2^-24
                assert torch.equal(f, S.STASH.logits.to(torch.float32) * 2.0 ** -24)
            elif mode == "greedy":                          # one-hot at the greedy token, no sampler pass needed
                assert bool(((f == 0).sum(1) == 1).all())
            ctx = SimpleNamespace(idx_mapping_np=np.array(live, dtype=np.int32),
                                  seq_lens_upper_bound_np=np.array(lens, dtype=np.int32))
            if mode != "greedy" or strict:
                f = smp.apply(f, ctx)
            tok = f.argmax(1).cpu().tolist()
            glue.check_output()
            for r, t in zip(live, tok):
                if done[r] == len(seqs[r]):                 # the whole sequence is in the cache: a token was sampled
                    out_tok[r].append(t)
                    seqs[r].append(t)
        for r in range(R):
            assert out_tok[r][:NEW] == z[f"p{r}_{mode}_tok"].tolist(), r
        eng.check()
        del table
    finally:
        S.STASH.active, S.STASH.sampler = old
