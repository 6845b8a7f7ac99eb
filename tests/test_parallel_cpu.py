"""Multi-rank host logic on CPU (gloo, world size 2): sequence and column shard bounds, the int64 all-gather of
column-sharded linear outputs, and the (max, first index) combine of the sharded sampler - each checked against the
unsharded oracle result bit for bit."""

import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from bitexact_llm_b200 import parallel as par
        from oracle import exact as ox
        from oracle import sampler as osamp
        rng = np.random.RandomState(3)                                    # same data on every rank
        N, K, M = 96, 64, 5
        w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
        w[3, :4] = [1e-9, -3e-8, 2.0, -0.5]
        bits = torch.from_numpy(w).to(torch.bfloat16).view(torch.int16).numpy().astype(np.uint16)
        dec = ox.decompose(bits)
        q = rng.randint(-(1 << 22), 1 << 22, (M, K)).astype(np.int64)
        sh = rng.randint(-20, -8, M).astype(np.int64)
        full, _ = ox.linear(q, sh, dec)
        # column shard of the constants, local product with the oracle, int64 all-gather
        c = {f"lm.{k}": torch.from_numpy(np.ascontiguousarray(v)) for k, v in dec.items()}
        n0, n1 = par.column_bounds(N, world, rank)
        loc = {k: v.numpy() for k, v in par.shard_linear_constants(c, "lm", n0, n1).items()}
        y_loc, _ = ox.linear(q, sh, loc)
        y = par.gather_columns(torch.from_numpy(y_loc))
        ok = bool(np.array_equal(y.numpy(), full))
        # sharded sampler: (max, first idx) of the shard with global indices, then the combine
        lnt = ox.ln_table()
        for tn, td in ((0, 1), (7, 10)):
            g = osamp.gumbel(osamp.raw_rows([(r, 2) for r in range(M)], N), lnt, 24) if tn else None
            v = full if tn == 0 else ox.rdiv(full * td, np.int64(tn)) + g
            v[1, 10] = v[1, 70] = v[1].max() + 3                          # tie across shards: first index wins
            want = ox.first_argmax(v)
            vl = v[:, n0:n1]
            best = torch.from_numpy(vl.max(1))
            idx = torch.from_numpy(ox.first_argmax(vl) + n0)
            tok = par.combine_argmax(best, idx)
            ok = ok and bool(np.array_equal(tok.numpy(), want)) and int(tok[1]) == 10
        # column-sharded gate / up: shard constants, local SiLU products, integer all-reduce MAX of the row maxima,
        # quantisation with the common exponent, all-gather of the shards = the full-row silu_quant
        FF = 64
        wgu = (rng.standard_normal((2 * FF, K)) * 0.05).astype(np.float32)
        dgu = ox.decompose(torch.from_numpy(wgu).to(torch.bfloat16).view(torch.int16).numpy().astype(np.uint16))
        lut = ox.exp2_table()
        y_full, _ = ox.linear(q, sh, dgu)
        wq, wsh, _ = ox.silu_quant(y_full, lut)
        cgu = {f"0.wgu.{k}": torch.from_numpy(np.ascontiguousarray(v)) for k, v in dgu.items()}
        f0, f1 = par.column_bounds(FF, world, rank, 16)
        sgu = {k: v.numpy() for k, v in par.shard_gate_up_constants(cgu, "0.wgu", FF, f0, f1).items()}
        y_loc, _ = ox.linear(q, sh, sgu)
        ok = ok and bool(np.array_equal(y_loc, np.concatenate([y_full[:, f0:f1], y_full[:, FF + f0:FF + f1]], 1)))
        P_loc, _ = ox.silu_mul(y_loc[:, :f1 - f0], y_loc[:, f1 - f0:], lut)
        rmax = par.allreduce_max(torch.from_numpy(np.abs(P_loc).max(1)))
        _, sh_c = ox.quant(rmax.numpy()[:, None], -48)
        q_loc = ox.rshc(P_loc, sh_c[:, None] + 48)
        qg = par.gather_columns(torch.from_numpy(q_loc))
        ok = ok and bool(np.array_equal(qg.numpy(), wq)) and bool(np.array_equal(sh_c, wsh))
        # sequence shards partition the batch
        lo, hi = par.shard_bounds(11, world, rank)
        rows = par.gather_rows(torch.arange(lo, lo + 5))                   # equal-size blocks gather in rank order
        ok = ok and rows.tolist() == [*range(0, 5), *range(par.shard_bounds(11, world, 1)[0],
                                                            par.shard_bounds(11, world, 1)[0] + 5)]
        # packed row exchange of an int8-mode linear input: planes + row scales in one all-gather
        a8 = torch.from_numpy(rng.randint(-128, 128, (2, 3, 8)).astype(np.int8)) + rank
        mant = torch.arange(3) + 100 * rank + (1 << 40)
        ee = -torch.arange(3) - 7 * rank
        A, Mg, Eg = par.gather_scaled_rows(a8, mant, ee)
        want_a = torch.cat([a8 - rank + r for r in range(world)], 1)
        ok = ok and torch.equal(A, want_a) and Mg.tolist() == [v + 100 * r + (1 << 40) for r in range(world) for v in range(3)]
        ok = ok and Eg.tolist() == [-v - 7 * r for r in range(world) for v in range(3)]
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


def test_shard_bounds_cover_everything():
    from bitexact_llm_b200 import parallel as par
    for n in (0, 1, 7, 256, 513):
        for world in (1, 2, 4, 8):
            spans = [par.shard_bounds(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    assert par.column_bounds(128256, 8, 3) == (3 * 16032, 4 * 16032)


def test_two_ranks_gloo():
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    assert all(p.exitcode == 0 for p in procs) and dict(ret) == {0: True, 1: True}
