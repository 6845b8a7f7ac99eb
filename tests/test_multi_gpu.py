"""2, 4 or 8 ranks over NCCL (the largest of these that the box has GPUs for; skipped below 2): the column-sharded LM head gathers to the single-GPU
logits bit for bit, the sharded sampler picks the single-GPU tokens and the sharded integer log p gives the
single-GPU integers; the column-sharded MLP (gate / up and down
split by output column, integer all-reduce MAX of the SiLU row maxima) gives the single-GPU output; sequence-sharded decode of a batch split
over the ranks reproduces the reference's tokens and logits hashes of every sequence."""

import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    try:
        from make_golden import TINY, TINY_PROMPTS, tiny_state_dict
        from bitexact_llm_b200 import parallel as par
        from bitexact_llm_b200.decode import generate
        from bitexact_llm_b200.exact import consts
        from bitexact_llm_b200.vllm_plugin import exact_fuse, sampler
        from bitexact_llm_b200.vllm_plugin.exact_run import ExactEngine
        z = np.load(os.path.join(ROOT, "tests", "golden", "tiny_model.npz"))
        tables = {"cos": torch.zeros(4096, 32, dtype=torch.long), "sin": torch.zeros(4096, 32, dtype=torch.long)}
        tables["cos"][:128], tables["sin"][:128] = torch.from_numpy(z["cos"]), torch.from_numpy(z["sin"])
        dev = torch.device("cuda", rank)
        c = consts.build(TINY, {k: v.to(dev) for k, v in tiny_state_dict().items()}, tables=tables)   # device decompose
        eng = ExactEngine(c, dev)
        ok = True
        # (1) column-sharded head: same hidden rows on every rank
        g = torch.Generator().manual_seed(5)
        h = torch.randint(-(1 << 26), 1 << 26, (7, eng.D), generator=g).to(dev)
        q, sh = exact_fuse.pre_norm(eng, h, eng.gf, eng.fl)
        full = eng.lm(q, sh, eng.fl, True)
        head = par.ShardedHead(c, dev)
        ok &= torch.equal(head.full_logits(q, sh, eng.fl), full)
        rows = torch.tensor([[r, 2 * r, (7 if r % 2 else 0), (10 if r % 2 else 1)] for r in range(7)], device=dev)
        ok &= torch.equal(head.sample(q, sh, eng.fl, rows, eng.ln), sampler.sample_rows(full, rows, eng.ln))
        # (1a) integer log p from the column shard of the logits: the bits of the full rows
        from bitexact_llm_b200.vllm_plugin import rl
        tk = torch.tensor([0, 5, 128255, 70000, 16032, 16031, 99], device=dev)
        ok &= torch.equal(par.sharded_logp_q(head.local_logits(q, sh, eng.fl), head.v0, tk, eng.ln, 24),
                          rl.int_logp_q(full, tk, eng.ln, 24))
        # (1b) column-sharded MLP of layer 0: the single-GPU wgu -> silu_quant -> wd output on every rank
        hq = torch.randint(-(1 << 22), (1 << 22) + 1, (6, eng.D), generator=g).to(torch.int32).to(dev)
        hs = torch.randint(-40, -30, (6,), generator=g).to(dev)
        ly = eng.layers[0]
        q1, sh1 = exact_fuse.silu_quant(eng, ly["wgu"](hq, hs, eng.fl, False), eng.exp2, eng.fl)
        want = ly["wd"](q1, sh1, eng.fl, True)
        mlp = par.ShardedMLP(c, 0, eng.FF, dev)
        ok &= torch.equal(mlp(hq, hs, eng.exp2, eng.fl), want)
        # (2) sequence sharding: every rank decodes its block of the sequences (at least one each)
        order = [0, 1, 2, 1, 2, 0, 1, 2][:max(4, world)]
        lo, hi = par.shard_bounds(len(order), world, rank)
        mine = order[lo:hi]
        P = max(len(TINY_PROMPTS[i]) for i in mine)
        ids = torch.zeros(len(mine), P, dtype=torch.long)
        for b, i in enumerate(mine):
            ids[b, :len(TINY_PROMPTS[i])] = torch.tensor(TINY_PROMPTS[i])
        lens = torch.tensor([len(TINY_PROMPTS[i]) for i in mine])
        toks, shas = generate(eng, ids, 8, 7, 10, seeds=mine, lens=lens, max_len=64)
        for b, i in enumerate(mine):
            ok &= toks[b].tolist() == z[f"p{i}_t07_tok"].tolist() and shas[b] == z[f"p{i}_t07_sha"].tolist()
        eng.check()
        # (3) int8 mode: sequence-sharded decode against the reference's hashes, column-sharded LM head and sampler
        from bitexact_llm_b200.int8 import consts as consts8
        from bitexact_llm_b200.int8.engine import IntEngine
        from bitexact_llm_b200.vllm_plugin import tri_fuse
        z8 = np.load(os.path.join(ROOT, "tests", "golden", "tiny_model_int8.npz"))
        t8 = {"cos": torch.zeros(2048, 32, dtype=torch.long), "sin": torch.zeros(2048, 32, dtype=torch.long)}
        t8["cos"][:128], t8["sin"][:128] = torch.from_numpy(z8["cos"]), torch.from_numpy(z8["sin"])
        c8 = consts8.build(TINY, tiny_state_dict(), tables=t8)
        eng8 = IntEngine(c8, dev)
        toks, shas = generate(eng8, ids, 8, 7, 10, seeds=mine, lens=lens, max_len=64)
        for b, i in enumerate(mine):
            ok &= toks[b].tolist() == z8[f"p{i}_t07_tok"].tolist() and shas[b] == z8[f"p{i}_t07_sha"].tolist()
        h8 = torch.randint(-(1 << 18), 1 << 18, (7, eng8.D), generator=g).to(dev)
        pre = tri_fuse.pre_norm(eng8, h8, eng8.gf)
        full8 = eng8.logits(h8)
        head8 = par.ShardedHeadInt8(c8, dev)
        ok &= torch.equal(head8.full_logits(*pre, eng8.fl), full8)
        ok &= torch.equal(head8.sample(*pre, eng8.fl, rows, eng8.ln), sampler.sample_rows(full8, rows, eng8.ln, 16))
        eng8.check()
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_ranks_nccl():
    import torch.multiprocessing as mp
    world = max(w for w in (2, 4, 8) if w <= torch.cuda.device_count())
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = 29700 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=600)
    assert all(p.exitcode == 0 for p in procs) and dict(ret) == {r: True for r in range(world)}
