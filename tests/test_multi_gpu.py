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


# ---- BASELINE config 5: int8 mode, sequences sharded over the ranks, MLP and LM head + sampler sharded by column ----

def _config5_worker(rank, world, port, order, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import hashlib
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    try:
        from bitexact_llm_b200 import parallel as par
        from bitexact_llm_b200.decode import Session
        from bitexact_llm_b200.exact import consts
        from bitexact_llm_b200.int8 import consts as consts8
        dev = torch.device("cuda", rank)
        cfg = dict(consts.LLAMA_1B)
        cfg["num_hidden_layers"] = 1
        c = consts8.build(cfg, consts.random_state_dict(cfg, seed=3, device=dev), n_pos=4200)
        eng = par.ColumnShardedIntEngine(c, dev)
        per = len(order) // world
        mine = order[rank * per:(rank + 1) * per]
        # sequence s: its own seeded prompt (length U[16, 4096] for a few, short for the rest) and sampler key s
        rng = [np.random.RandomState(1000 + s) for s in mine]
        lens = [int(r.randint(16, 4097)) if s % 8 == 0 else int(r.randint(16, 200)) for r, s in zip(rng, mine)]
        P = max(lens)
        ids = torch.zeros(per, P, dtype=torch.long)
        for b, (r, n) in enumerate(zip(rng, lens)):
            ids[b, :n] = torch.from_numpy(r.randint(0, cfg["vocab_size"], n))
        ses = Session(eng, per, 4200)
        eng.sharded = False                                     # prompts: every rank on its own
        h = ses.prefill(ids, torch.tensor(lens), chunk_rows=2048)
        eng.sharded = True
        rows_all = torch.zeros(len(order), 4, dtype=torch.long, device=dev)
        rows_all[:, 0] = torch.tensor(order, device=dev)
        rows_all[:, 2], rows_all[:, 3] = 7, 10
        out = {s: [] for s in mine}
        for t in range(3):
            lg = eng.logits(h)                                  # test mode: the gathered rows, for the hashes
            tok = eng.sample(h, rows_all)
            for b, s in enumerate(mine):
                out[s].append((hashlib.sha256(lg[b].cpu().numpy().tobytes()).hexdigest(), int(tok[b])))
            rows_all[:, 1] += 1
            h = ses.step(tok)
        eng.check()
        ret[rank] = out
    finally:
        dist.destroy_process_group()


def _config5_run(world, order, port):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_config5_worker, args=(r, world, port, order, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=900)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    merged = {}
    for r in range(world):
        merged.update(ret[r])
    return merged


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_config5_int8_column_sharded_decode_is_identical_at_every_gpu_count_and_order():
    """One int8-mode decoder layer + LM head at Llama-3.2-1B geometry, 16 sequences with mixed prompt lengths (two of
    them drawn from U[16, 4096]): per-step logits hashes and T = 0.7 tokens of every sequence are the same on 1 GPU
    and on 2 / 4 / 8 GPUs with the MLP and the LM head + sampler sharded by column, and under a permuted batch."""
    order = list(range(16))
    port = 29900 + os.getpid() % 1000
    want = _config5_run(1, order, port)
    worlds = [w for w in (2, 4, 8) if w <= torch.cuda.device_count()]
    for i, w in enumerate(worlds):
        assert _config5_run(w, order, port + 1 + i) == want, w
    perm = [int(v) for v in np.random.RandomState(5).permutation(16)]
    assert _config5_run(worlds[-1], perm, port + 9) == want
