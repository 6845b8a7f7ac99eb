"""A vLLM-style mixed step (a whole prefill, a prefill chunk behind an earlier chunk, a decode) laid out by
vllm_plugin.paged.make_plan and run as token rows through the int8 engine: the last row of every request hashes to
the reference's logits hash for that position."""

import os
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
sys.path.insert(0, GOLD)


def test_mixed_step_through_the_plan():
    from make_golden import TINY, TINY_PROMPTS, tiny_state_dict
    from bitexact_llm_b200.decode import logits_sha
    from bitexact_llm_b200.int8 import consts
    from bitexact_llm_b200.int8.engine import IntEngine
    from bitexact_llm_b200.vllm_plugin import paged
    z = np.load(os.path.join(GOLD, "tiny_model_int8.npz"))
    tables = {"cos": torch.zeros(2048, 32, dtype=torch.long), "sin": torch.zeros(2048, 32, dtype=torch.long)}
    tables["cos"][:128], tables["sin"][:128] = torch.from_numpy(z["cos"]), torch.from_numpy(z["sin"])
    eng = IntEngine(consts.build(TINY, tiny_state_dict(), tables=tables), "cuda")
    dev, bs = eng.dev, 16
    kvs = [torch.zeros(13, eng.HKV, bs, 8 * eng.HD, dtype=torch.int8, device=dev) for _ in range(eng.L)]
    bt = torch.tensor([[7, 2, 9, 4], [1, 12, 3, 8], [5, 10, 6, 11]], dtype=torch.int32, device=dev)
    seqs = [list(TINY_PROMPTS[0]), list(TINY_PROMPTS[1]), list(TINY_PROMPTS[2]) + [int(z["p2_greedy_tok"][0])]]

    def step(spans, pad=0):
        """spans: per request (first position, one past the last position) of its query tokens in this step."""
        ids, pos, slots, qsl = [], [], [], [0]
        for r, (a, b) in enumerate(spans):
            ids += seqs[r][a:b]
            pos += list(range(a, b))
            slots += [int(bt[r, p // bs]) * bs + p % bs for p in range(a, b)]
            qsl.append(qsl[-1] + b - a)
        n, N = len(ids), len(ids) + pad
        meta = SimpleNamespace(query_start_loc=torch.tensor(qsl, dtype=torch.int32), block_table=bt,
                               seq_lens=torch.tensor([b for _, b in spans], dtype=torch.int32),
                               slot_mapping=torch.tensor(slots + [0] * pad, device=dev))
        positions = torch.tensor(pos + [0] * pad, device=dev)
        plan = paged.make_plan(meta, N, positions)
        slot, table, rmap = plan.rows(N)
        x = eng.forward(kvs, torch.tensor(ids + [0] * pad, device=dev), positions, slot, table, rmap)
        return x, qsl

    step([(0, 0), (0, 10), (0, 40)])                                   # earlier step: B's first chunk, C's prompt
    x, qsl = step([(0, 5), (10, 17), (40, 41)], pad=3)                 # the mixed step, with three padding rows
    lg = eng.logits(x[[qsl[1] - 1, qsl[2] - 1, qsl[3] - 1]])
    eng.check()
    assert logits_sha(lg[0]) == z["p0_greedy_sha"][0]
    assert logits_sha(lg[1]) == z["p1_greedy_sha"][0]
    assert logits_sha(lg[2]) == z["p2_greedy_sha"][1]
