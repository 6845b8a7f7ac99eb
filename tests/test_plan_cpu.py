"""Batch layout of a forward call (vllm_plugin.paged.make_plan / Plan.groups) against the reference's own output on
the same step description (tests/golden/plan.npz), and the token-row form the kernels of this package take."""

import os
import sys

import numpy as np
import torch

GOLD = os.path.join(os.path.dirname(__file__), "golden")
sys.path.insert(0, GOLD)


def test_plan_matches_the_reference_and_gives_token_rows():
    from make_golden import plan_meta
    from bitexact_llm_b200.vllm_plugin import paged
    z = np.load(os.path.join(GOLD, "plan.npz"))
    meta, N, pos = plan_meta()
    default_cap = paged.GROUP_BYTES
    try:
        for tag, cap in (("a", default_cap), ("b", 2 * 17 * 2048 * 8 - 1)):
            paged.GROUP_BYTES = cap
            p = paged.make_plan(meta, N, pos)
            assert p.n == int(z[f"{tag}_n"])
            for name, got in (("slot", p.slot), ("bt", p.block_table), ("dec_req", p.dec_req), ("dec_tok", p.dec_tok)):
                assert got.dtype == torch.int64 and np.array_equal(got.numpy(), z[f"{tag}_{name}"]), name
            assert [list(t) for t in p.pre] == z[f"{tag}_pre"].tolist()
            groups = p.groups()
            assert len(groups) == int(z[f"{tag}_ngroups"]) and p.groups() is groups
            for i, g in enumerate(groups):
                for name in ("req", "idx", "pos", "valid", "dst"):
                    assert np.array_equal(getattr(g, name).numpy(), z[f"{tag}_g{i}_{name}"]), (i, name)
    finally:
        paged.GROUP_BYTES = default_cap
    # token rows: every real token belongs to the request whose query range holds it
    qsl = meta.query_start_loc.tolist()
    for t in range(p.n):
        r = int(p.rmap[t])
        assert qsl[r] <= t < qsl[r + 1]
    slot, bt, rmap = p.rows(N)
    assert slot.shape == (N,) and rmap.shape == (N,) and bt is p.block_table
    assert slot[p.n:].tolist() == [-1] * (N - p.n) and rmap[p.n:].tolist() == [0] * (N - p.n)
    assert torch.equal(slot[:p.n], p.slot) and p.rows()[0].shape == (p.n,)


def test_kv_view():
    from bitexact_llm_b200.vllm_plugin import paged
    kv = torch.zeros(3, 8, 16, 256, dtype=torch.bfloat16)
    v = paged.kv_view(kv)
    assert v.dtype == torch.int8 and v.shape == (3, 8, 16, 512) and v.data_ptr() == kv.data_ptr()
