"""Kernel micro-benchmarks through the C ABI (CUDA-event timing, inputs larger than L2 or L2 flushed).

    python microbench.py gemm [--m 1,16,256,4096] [--tile 0] [--iters 20] [--shapes decode|all]
    python microbench.py gemmr [--m 256] [--iters 10]
    python microbench.py attn [--batch 256] [--ctx 4128] [--iters 10]
    python microbench.py stages [--batch 256] [--iters 10]
    python microbench.py prefill [--batch 4] [--ctx 2048] [--iters 10]
    python microbench.py prompt [--batch 4] [--ctx 2048] [--chunk 4096] [--iters 3]
    python microbench.py bmm [--ctx 2048] [--iters 5]

gemm: the exact-mode fused linear on the projection shapes of one Llama-3.2-1B layer and the LM head
      (int8-equivalent ops = 2 * 9 * M * N * K; algorithmic bytes = 3 N K + 4 M K + 8 M N).
gemmr: the fused projections of one layer with REAL constants (bf16 weights from N(0, 0.02^2), decomposed into limbs
      and the sparse residual lists, as the engine holds them) through `FusedLin` with producer-written limb planes,
      timed as a CUDA graph over enough weight sets to exceed L2, with and without the residual lists.
attn: exact-mode paged decode attention, 8 KV heads x 4 query heads, head_dim 64, 16-token pages, context lengths
      uniform in [64, 2 ctx - 64] (algorithmic bytes = 384 per key and KV head).
stages (the last line: integer log p, two passes of 8 V bytes per row): add + RMSNorm + quant (D 2048: 16 D read + 15 D written per row), SiLU * up + quant (FF 8192: 16 FF read,
      7 FF written), attention output division (2048 columns: 8 read, 7 written per element) and the seeded
      Gumbel-max sampler (V 128256: 8 V read per row), on random in-range rows.
"""

import argparse
import json

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from bitexact_llm_b200 import _native as nv  # noqa: E402

SHAPES = {"q": (2048, 2048), "k": (512, 2048), "v": (512, 2048), "o": (2048, 2048), "gate": (8192, 2048),
          "up": (8192, 2048), "down": (2048, 8192)}
FUSED = {"wqkv": (3072, 2048), "wo": (2048, 2048), "wgu": (16384, 2048), "wd": (2048, 8192), "lm": (128256, 2048)}


def _flush(buf):
    buf.add_(1)                                    # > L2 capacity: evicts everything


def gemm(args):
    lib, dev = nv.lib(), "cuda"
    flush = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)
    shapes = dict(FUSED) if args.shapes == "decode" else {**SHAPES, **FUSED}
    out = []
    for M in [int(v) for v in args.m.split(",")]:
        for name, (N, K) in shapes.items():
            q = torch.randint(-(1 << 22), (1 << 22) + 1, (M, K), dtype=torch.int32, device=dev)
            sh = torch.full((M,), -14, dtype=torch.long, device=dev)
            limbs = torch.randint(-128, 128, (3, N, K), dtype=torch.int8, device=dev)
            d = torch.zeros(N, dtype=torch.long, device=dev)
            g = torch.full((N,), -30, dtype=torch.long, device=dev)
            scratch = torch.empty(3 * M * K, dtype=torch.int8, device=dev)
            y = torch.empty(M, N, dtype=torch.long, device=dev)
            flag = torch.zeros(1, dtype=torch.int32, device=dev)
            st = torch.cuda.current_stream().cuda_stream

            def run():
                rc = lib.bx_exact_linear(q.data_ptr(), K, sh.data_ptr(), limbs.data_ptr(), d.data_ptr(), g.data_ptr(),
                                         None, None, None, 0, scratch.data_ptr(), y.data_ptr(), flag.data_ptr(),
                                         M, N, K, 1, args.tile, st)
                nv.check(rc, "bx_exact_linear")
            for _ in range(3):
                run()
            ms = 0.0
            for _ in range(args.iters):
                if 3 * N * K < (200 << 20):
                    _flush(flush)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                run()
                e1.record()
                torch.cuda.synchronize()
                ms += e0.elapsed_time(e1) / args.iters
            ops, byts = 18.0 * M * N * K, 3.0 * N * K + 4.0 * M * K + 8.0 * M * N
            rec = {"kernel": "exact_linear", "proj": name, "M": M, "N": N, "K": K, "us": ms * 1e3,
                   "int8_tops": ops / ms / 1e9, "GBps": byts / ms / 1e6}
            out.append(rec)
            print(json.dumps(rec), flush=True)
            del limbs, y, q, scratch
    return out


def gemmr(args):
    from bitexact_llm_b200.exact.consts import decompose
    from bitexact_llm_b200.exact.model import Lin
    from bitexact_llm_b200.vllm_plugin import exact_fuse
    from bitexact_llm_b200.vllm_plugin.exact_gemm import FusedLin
    lib, dev = nv.lib(), "cuda"
    g = torch.Generator().manual_seed(0)
    out = []
    for M in [int(v) for v in args.m.split(",")]:
        for name, (N, K) in FUSED.items():
            if name == "lm" and args.shapes != "all":
                continue
            if args.proj and name != args.proj:
                continue
            w = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
            d0 = decompose(w.to(dev))
            nsets = max(2, (200 << 20) // (3 * N * K) + 1)
            sets = [FusedLin(Lin({k: (v.clone() if torch.is_tensor(v) else v) for k, v in d0.items()}, None, dev))
                    for _ in range(nsets)]
            for f in sets:
                f.cfg = args.tile or None
            q = torch.randint(-(1 << 22), (1 << 22) + 1, (M, K), dtype=torch.int32, device=dev)
            planes = torch.empty(3, M, K, dtype=torch.int8, device=dev)
            nv.check(lib.bx_split_limbs(q.data_ptr(), K, planes.data_ptr(), M, K, nv.stream()), "bx_split_limbs")
            exact_fuse.attach_planes(q, planes)
            sh = torch.full((M,), -14, dtype=torch.long, device=dev)
            fl = torch.zeros(1, dtype=torch.int32, device=dev)
            if args.eager:                      # plain launches, one per weight set (for a profiler capture)
                for i in range(nsets):
                    sets[i](q, sh, fl, False)
                torch.cuda.synchronize()
                print(json.dumps({"kernel": "exact_linear", "proj": name, "M": M, "eager_launches": nsets}), flush=True)
                del sets
                continue
            for tag in ("residual", "none"):
                saved = [f.cnt for f in sets]
                if tag == "none":
                    for f in sets:
                        f.cnt = None
                ms = _graph_time(lambda i: sets[i](q, sh, fl, False), nsets, args.iters)
                for f, c in zip(sets, saved):
                    f.cnt = c
                rec = {"kernel": "exact_linear", "proj": name, "M": M, "N": N, "K": K, "residual": tag,
                       "entries": int(d0["rr"].numel()), "us": ms * 1e3, "int8_tops": 18.0 * M * N * K / ms / 1e9}
                out.append(rec)
                print(json.dumps(rec), flush=True)
            del sets
    return out


def gemm8(args):
    """int8-mode fused linear (GEMM + post) on the model's projections: CUDA-graph timing over weight sets larger than
    L2. int8 ops = 2 * 2 * M * N * K (two activation limbs)."""
    lib, dev = nv.lib(), "cuda"
    g = torch.Generator().manual_seed(0)
    out = []
    for M in [int(v) for v in args.m.split(",")]:
        for name, (N, K) in FUSED.items():
            if (name == "lm" and args.shapes != "all") or (args.proj and name != args.proj):
                continue
            nsets = max(2, (200 << 20) // (N * K) + 1)
            ws = [torch.randint(-127, 128, (N, K), dtype=torch.int8, generator=g).to(dev) for _ in range(nsets)]
            a = torch.randint(-128, 128, (2 * M, K), dtype=torch.int8, generator=g).to(dev)
            mul = torch.randint(1 << 20, 1 << 24, (N,), generator=g).to(dev)
            mant = torch.randint(1 << 7, 1 << 8, (M,), generator=g).to(dev)
            e = torch.randint(-12, -4, (M,), generator=g).to(dev)
            y = torch.empty(M, N, dtype=torch.long, device=dev)
            fl = torch.zeros(1, dtype=torch.int32, device=dev)

            def run(i):
                nv.check(lib.bx_int8_linear_post(a.data_ptr(), ws[i].data_ptr(), mul.data_ptr(), 30, mant.data_ptr(),
                                                 e.data_ptr(), y.data_ptr(), fl.data_ptr(), M, N, K, 0, args.tile,
                                                 nv.stream()), "bx_int8_linear_post")
            if args.eager:                      # plain launches, one per weight set (for a profiler capture)
                for i in range(nsets):
                    run(i)
                torch.cuda.synchronize()
                print(json.dumps({"kernel": "int8_linear", "proj": name, "M": M, "eager_launches": nsets}), flush=True)
                del ws
                continue
            ms = _graph_time(run, nsets, args.iters)
            rec = {"kernel": "int8_linear", "proj": name, "M": M, "N": N, "K": K, "residual": "residual",
                   "us": ms * 1e3, "int8_tops": 4.0 * M * N * K / ms / 1e9}
            out.append(rec)
            print(json.dumps(rec), flush=True)
            del ws
    return out


def attn(args):
    from bitexact_llm_b200.exact.consts import exp2_table
    lib, dev = nv.lib(), "cuda"
    B, HKV, G, HD, bs = args.batch, 8, 4, 64, 16
    gen = torch.Generator(device=dev).manual_seed(0)
    lo, hi = 64, max(65, 2 * args.ctx - 64)
    ctx = torch.randint(lo, hi + 1, (B,), generator=gen, device=dev)
    if args.fixed:
        ctx = torch.full((B,), args.ctx, device=dev)
    nblk = (int(ctx.max()) + bs) // bs
    nb = 1 + B * nblk
    cache = torch.randint(-128, 128, (nb, HKV, bs, 8 * HD), dtype=torch.int8, device=dev, generator=gen)
    bt = (1 + torch.randperm(nb - 1, device=dev, generator=gen)).view(B, nblk).to(torch.int32)
    q = torch.randint(-(1 << 22), (1 << 22) + 1, (B, HKV, G, HD), dtype=torch.int32, device=dev, generator=gen)
    sh = torch.randint(-40, -30, (B, HKV, G), device=dev, generator=gen)
    qpos = (ctx - 1)[:, None].expand(B, G).contiguous()
    lut = exp2_table(dev)
    num = torch.empty(B, HKV, G, HD, dtype=torch.long, device=dev)
    den = torch.empty(B, HKV, G, dtype=torch.long, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    ws = None
    if not args.no_scratch:
        ws = torch.empty(lib.bx_attention_scratch_bytes(nblk, bs), dtype=torch.uint8, device=dev)

    def run(variant=None, outs=None):
        n_, d_ = outs if outs is not None else (num, den)
        rc = lib.bx_exact_attention_ws(q.data_ptr(), sh.data_ptr(), qpos.data_ptr(), cache.data_ptr(), cache.shape[0],
                                       cache.stride(0), cache.stride(1), cache.stride(2), bs, bt.data_ptr(), 0,
                                       bt.stride(0), nblk, None, lut.data_ptr(), 387270501, n_.data_ptr(), d_.data_ptr(), B,
                                       HKV, G, HD, args.cluster if variant is None else 0,
                                       args.variant if variant is None else variant,
                                       ws.data_ptr() if (ws is not None and variant is None) else None,
                                       ws.numel() if (ws is not None and variant is None) else 0, st)
        nv.check(rc, "bx_exact_attention_ws")
    flush = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(2):
        run()
    ms = 0.0
    for _ in range(args.iters):
        _flush(flush)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run()
        e1.record()
        torch.cuda.synchronize()
        ms += e0.elapsed_time(e1) / args.iters
    # every timed variant must give the integers of the direct-load kernel
    want = (torch.empty_like(num), torch.empty_like(den))
    run(1, want)
    torch.cuda.synchronize()
    if not (torch.equal(num, want[0]) and torch.equal(den, want[1])):
        raise SystemExit("variant %d differs from the direct-load kernel" % args.variant)
    byts = 384.0 * HKV * float(ctx.sum())
    rec = {"kernel": "exact_attention", "variant": args.variant, "cluster": args.cluster, "batch": B, "mean_ctx": float(ctx.float().mean()), "us": ms * 1e3,
           "GBps": byts / ms / 1e6, "bytes": byts}
    print(json.dumps(rec), flush=True)
    return rec


def prefill(args):
    """Prefill attention of whole prompts, Llama-3.2-1B geometry (8 KV heads x 4 query heads, head_dim 64, 16-token
    pages): --batch prompts of --ctx tokens each through the tile kernel and, for comparison, through the per-row
    decode kernel (every token a row). Algorithmic int8 ops = 2 products x 2 * 9 * (S^2 / 2) * H * HD per prompt."""
    from bitexact_llm_b200.exact.consts import exp2_table
    from bitexact_llm_b200.vllm_plugin import tri_exact_attn, tri_prefill
    dev = "cuda"
    R, S, HKV, G, HD, bs = args.batch, args.ctx, 8, 4, 64, 16
    gen = torch.Generator(device=dev).manual_seed(0)
    nblk = (S + bs - 1) // bs
    nb = 1 + R * nblk
    cache = torch.randint(-128, 128, (nb, HKV, bs, 8 * HD), dtype=torch.int8, device=dev, generator=gen)
    bt = (1 + torch.randperm(nb - 1, device=dev, generator=gen)).view(R, nblk).to(torch.int32)
    N = R * S
    q = torch.randint(-(1 << 22), (1 << 22) + 1, (N, HKV, G, HD), dtype=torch.int32, device=dev, generator=gen)
    sh = torch.randint(-30, -20, (N, HKV, G), device=dev, generator=gen)
    pos = torch.arange(S, device=dev).repeat(R)
    req = torch.arange(R, device=dev).repeat_interleave(S)
    tiles = tri_prefill.tile_table([(r, r * S, S, S) for r in range(R)], G).to(dev)
    lut = exp2_table(dev)
    num = torch.zeros(N, HKV, G, HD, dtype=torch.long, device=dev)
    den = torch.ones(N, HKV, G, 1, dtype=torch.long, device=dev)
    qpos = pos[:, None].expand(N, G).contiguous()

    def timed(fn):
        for _ in range(2):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.iters

    rows = args.tile or tri_prefill.ROWS
    tiles = tri_prefill.tile_table([(r, r * S, S, S) for r in range(R)], G, rows).to(dev)
    ms_tile = timed(lambda: tri_prefill.attend_exact(q, sh, pos, cache, bt, tiles, lut, 387270501, num, den, rows))
    n2, d2 = tri_exact_attn.attend(q, sh, qpos, cache, bt, req, lut, 387270501)
    if not (torch.equal(num, n2) and torch.equal(den, d2)):
        raise SystemExit("tile kernel differs from the per-row kernel")
    ms_row = timed(lambda: tri_exact_attn.attend(q, sh, qpos, cache, bt, req, lut, 387270501))
    ops = R * 2.0 * 18.0 * (S * (S + 1) / 2.0) * HKV * G * HD
    rec = {"kernel": "prefill_attention", "tile_rows": rows, "prompts": R, "S": S, "tiles": int(tiles.shape[0]), "us": ms_tile * 1e3,
           "int8_tops": ops / ms_tile / 1e9, "tokens_per_s_one_layer": N / ms_tile * 1e3,
           "per_row_kernel_us": ms_row * 1e3, "speedup_vs_rows": ms_row / ms_tile}
    print(json.dumps(rec), flush=True)
    return rec


def bmm_bench(args):
    """`bmm` (the exact batched product of the reference's standalone engine) on the shapes of a --ctx-token prompt of
    one sequence: q.K (Z = 8 KV heads, M = 4 T, K = 64, N = S) and p.V (K = S, N = 64), on the tensor pipe (limb planes
    packed per call + the tcgen05 limb main loop) and on the CUDA-core int64 tile kernel. The serving path never calls
    it (its attention kernels form these products themselves)."""
    from bitexact_llm_b200.bmm import bmm
    dev = "cuda"
    S = args.ctx
    g = torch.Generator(device=dev).manual_seed(0)
    q = torch.randint(-(1 << 22), 1 << 22, (8, 4 * S, 64), dtype=torch.int32, device=dev, generator=g)
    k = torch.randint(-(1 << 22), 1 << 22, (8, 64, S), dtype=torch.int64, device=dev, generator=g)
    p = torch.randint(0, 1 << 22, (8, 4 * S, S), dtype=torch.int32, device=dev, generator=g)
    v = torch.randint(-(1 << 22), 1 << 22, (8, S, 64), dtype=torch.int64, device=dev, generator=g)
    for name, a, b in (("q.K", q, k), ("p.V", p, v)):
      for path in ("tensor", "cuda"):
        for _ in range(2):
            bmm(a, b, path=path)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.iters):
            bmm(a, b, path=path)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.iters
        macs = 8.0 * a.shape[1] * a.shape[2] * b.shape[2]
        print(json.dumps({"kernel": "bmm", "path": path, "product": name, "S": S, "us": ms * 1e3,
                          "int64_gmac_per_s": macs / ms / 1e6, "int8_equivalent_tops": 18.0 * macs / ms / 1e9}),
              flush=True)


def prompt(args):
    """Prompt processing of the whole model (random-init Llama-3.2-1B, exact mode): --batch prompts of --ctx tokens
    through `Session.prefill`, with the tile kernel and with every token as a row of the decode kernel."""
    from bitexact_llm_b200.decode import Session
    from bitexact_llm_b200.exact import consts
    from bitexact_llm_b200.vllm_plugin.exact_run import ExactEngine
    dev = torch.device("cuda")
    cfg = dict(consts.LLAMA_1B)
    c = consts.build(cfg, consts.random_state_dict(cfg, seed=0, device=dev), n_pos=args.ctx + 64)
    eng = ExactEngine(c, dev)
    del c
    g = torch.Generator().manual_seed(1)
    prompts = torch.randint(0, cfg["vocab_size"], (args.batch, args.ctx), generator=g)
    out = {}
    for tiles in (True, False):
        times, last = [], None
        for _ in range(1 + args.iters):
            ses = Session(eng, args.batch, args.ctx + 16)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            last = ses.prefill(prompts, chunk_rows=args.chunk, tiles=tiles)
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
            del ses
        out[tiles] = (min(times[1:]), last)
    eng.check()
    if not torch.equal(out[True][1], out[False][1]):
        raise SystemExit("prefill with tiles differs from prefill by rows")
    toks = args.batch * args.ctx
    rec = {"what": "prompt processing, 16 layers", "prompts": args.batch, "S": args.ctx, "chunk_rows": args.chunk,
           "ms_tiles": out[True][0], "tok_per_s_tiles": toks / out[True][0] * 1e3, "ms_rows": out[False][0],
           "tok_per_s_rows": toks / out[False][0] * 1e3}
    print(json.dumps(rec), flush=True)
    return rec


def _graph_time(run, nsets, iters, reps=4):
    """Mean device time of one call: `reps` rounds over `nsets` input sets captured in one CUDA graph (no host gaps;
    the sets together exceed L2, so every call reads its inputs from HBM)."""
    for i in range(nsets):
        run(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(reps):
            for i in range(nsets):
                run(i)
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (iters * reps * nsets)


def stages(args):
    from types import SimpleNamespace
    from bitexact_llm_b200.exact.consts import exp2_table, ln_table
    from bitexact_llm_b200.vllm_plugin import exact_fuse
    from bitexact_llm_b200.vllm_plugin.sampler import sample_rows
    dev, M, D, FF, V = "cuda", args.batch, 2048, 8192, 128256
    gen = torch.Generator(device=dev).manual_seed(0)
    fl = torch.zeros(1, dtype=torch.int32, device=dev)
    m = SimpleNamespace(D=D, H=32, HKV=8, HD=64, dev=dev, exp2=exp2_table(dev))
    R = lambda lo, hi, *shape: torch.randint(lo, hi, shape, dtype=torch.long, device=dev, generator=gen)
    gamma = (R(1 << 22, 1 << 24, D), R(-24, -20, D))
    lnt = ln_table(device=dev)

    def sets(n, make):
        return [make() for _ in range(n)]
    out = []

    def report(name, ms, byts):
        rec = {"kernel": name, "rows": M, "us": ms * 1e3, "GBps": byts / ms / 1e6}
        out.append(rec)
        print(json.dumps(rec), flush=True)

    n = max(2, (160 << 20) // (16 * M * D) + 1)
    xs = sets(n, lambda: (R(-(1 << 30), 1 << 30, M, D), R(-(1 << 28), 1 << 28, M, D)))
    report("add_norm", _graph_time(lambda i: exact_fuse.add_norm(m, xs[i][1], xs[i][0], gamma, fl), n, args.iters),
           31.0 * M * D)
    del xs
    n = max(2, (160 << 20) // (16 * M * FF) + 1)
    ys = sets(n, lambda: R(-(1 << 27), 1 << 27, M, 2 * FF))
    report("silu_quant", _graph_time(lambda i: exact_fuse.silu_quant(m, ys[i], m.exp2, fl), n, args.iters),
           23.0 * M * FF)
    del ys
    n = max(2, (160 << 20) // (8 * M * D) + 1)
    nd = sets(n, lambda: (R(-(1 << 40), 1 << 40, M, 8, 4, 64), R(1 << 20, 1 << 30, M, 8, 4, 1)))
    report("attn_out", _graph_time(lambda i: exact_fuse.attn_out(m, nd[i][0], nd[i][1]), n, args.iters),
           (15.0 + 8.0 / 64) * M * D)
    del nd
    n = max(2, (160 << 20) // (8 * M * V) + 1)
    ls = sets(n, lambda: R(-(1 << 28), 1 << 28, M, V))
    rows = torch.stack([R(0, 1 << 40, M), R(0, 1000, M), R(1, 9, M), R(1, 9, M)], 1)
    report("sample", _graph_time(lambda i: sample_rows(ls[i], rows, lnt, 24), n, args.iters), 8.0 * M * V)
    from bitexact_llm_b200.vllm_plugin.rl import int_logp_q
    toks = R(0, V, M)
    l16 = [x >> 8 for x in ls]                                                     # logits at 16 bits in (-16, 16)
    del ls
    report("int_logp", _graph_time(lambda i: int_logp_q(l16[i], toks, lnt, 16), n, args.iters), 16.0 * M * V)
    print(json.dumps({"bound_flag": int(fl)}))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "gemmr", "gemm8", "attn", "stages", "prefill", "prompt", "bmm"])
    ap.add_argument("--m", default="1,16,256,4096")
    ap.add_argument("--tile", type=int, default=0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--shapes", default="all", choices=["all", "decode"])
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--ctx", type=int, default=4128)
    ap.add_argument("--cluster", type=int, default=0)
    ap.add_argument("--variant", type=int, default=0)
    ap.add_argument("--no-scratch", action="store_true", help="attn: no scratch buffer (long contexts: cluster kernels)")
    ap.add_argument("--fixed", action="store_true", help="attn: every request has exactly --ctx keys")
    ap.add_argument("--proj", default="", help="gemmr / gemm8: only this projection (wqkv, wo, wgu, wd, lm)")
    ap.add_argument("--eager", action="store_true", help="gemmr / gemm8: one plain launch per weight set, no timing")
    ap.add_argument("--chunk", type=int, default=4096, help="prompt: token rows per forward call")
    args = ap.parse_args()
    {"gemm": gemm, "gemmr": gemmr, "gemm8": gemm8, "attn": attn, "stages": stages, "prefill": prefill, "prompt": prompt, "bmm": bmm_bench}[args.what](args)
    if nv.device_status() != 0:
        raise SystemExit("device-side wait timed out")


if __name__ == "__main__":
    main()
