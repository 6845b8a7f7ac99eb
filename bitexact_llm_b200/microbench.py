"""Kernel micro-benchmarks through the C ABI (CUDA-event timing, inputs larger than L2 or L2 flushed).

    python -m bitexact_llm_b200.microbench gemm [--m 1,16,256,4096] [--tile 0] [--iters 20] [--shapes decode|all]
    python -m bitexact_llm_b200.microbench attn [--batch 256] [--ctx 4128] [--iters 10]

gemm: the exact-mode fused linear on the projection shapes of one Llama-3.2-1B layer and the LM head
      (int8-equivalent ops = 2 * 9 * M * N * K; algorithmic bytes = 3 N K + 4 M K + 8 M N).
attn: exact-mode paged decode attention, 8 KV heads x 4 query heads, head_dim 64, 16-token pages, context lengths
      uniform in [64, 2 ctx - 64] (algorithmic bytes = 384 per key and KV head).
"""

import argparse
import json

import torch

from . import _native as nv

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


def attn(args):
    from .exact.consts import exp2_table
    lib, dev = nv.lib(), "cuda"
    B, HKV, G, HD, bs = args.batch, 8, 4, 64, 16
    gen = torch.Generator(device=dev).manual_seed(0)
    lo, hi = 64, max(65, 2 * args.ctx - 64)
    ctx = torch.randint(lo, hi + 1, (B,), generator=gen, device=dev)
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

    def run():
        rc = lib.bx_exact_attention(q.data_ptr(), sh.data_ptr(), qpos.data_ptr(), cache.data_ptr(), cache.shape[0], cache.stride(0),
                                    cache.stride(1), cache.stride(2), bs, bt.data_ptr(), 0, bt.stride(0), nblk, None,
                                    lut.data_ptr(), 387270501, num.data_ptr(), den.data_ptr(), B, HKV, G, HD,
                                    args.cluster, args.variant, st)
        nv.check(rc, "bx_exact_attention")
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
    byts = 384.0 * HKV * float(ctx.sum())
    rec = {"kernel": "exact_attention", "batch": B, "mean_ctx": float(ctx.float().mean()), "us": ms * 1e3,
           "GBps": byts / ms / 1e6, "bytes": byts}
    print(json.dumps(rec), flush=True)
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "attn"])
    ap.add_argument("--m", default="1,16,256,4096")
    ap.add_argument("--tile", type=int, default=0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--shapes", default="all", choices=["all", "decode"])
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--ctx", type=int, default=4128)
    ap.add_argument("--cluster", type=int, default=0)
    ap.add_argument("--variant", type=int, default=0)
    args = ap.parse_args()
    {"gemm": gemm, "attn": attn}[args.what](args)
    if nv.device_status() != 0:
        raise SystemExit("device-side wait timed out")


if __name__ == "__main__":
    main()
