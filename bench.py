#!/usr/bin/env python
"""Benchmark of the exact-mode decode path: random-init Llama-3.2-1B, 512-token prompts, batched decode.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--repeats R] [--batch B] [--prompt P] [--mode exact|int8]
                    [--impl reference]

A step is one decode step of the whole batch: 16 layers (4 limb GEMMs, RoPE/KV store, paged attention, attention
division, two RMSNorms, SiLU per layer), final norm, LM head and the integer Gumbel-max sampler at T = 0.7.
One process per GPU; with N > 1 (torchrun) every rank decodes its own B sequences (sequence sharding, no
collective on the data path), every timed region is bracketed by a barrier and its time is the max over ranks.
The region of exactly K steps is timed R times (on contexts that keep growing); the line reports the median region
with the minimum and maximum beside it. Before timing, one decoder layer + LM head of the SAME engine is compared bit
for bit with the CPU oracle on a seeded 64-row sample (`parity`); a difference ends the run with a non-zero status.
Prints ONE JSON line. `--impl reference` times the CPU restatement of the reference's float64-GEMM path (the
oracle) on the host cores for the same metric; it never touches CUDA or this package's shared library.
"""

import argparse
import contextlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "Llama-3.2-1B exact-mode decode tok/s (bit-exact)"
LAYER_NK = 60817408                             # weight entries of the four fused projections of one layer
HEAD_NK = 262668288                             # LM head
SAMPLE_ROWS, SAMPLE_CTX = 64, 640               # the CPU sample: config 4's mean context (512 + 256 / 2)
PARITY_BATCH = 256                              # the engine runs the sample repeated to this many rows


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--repeats", type=int, default=9, help="timed regions of --steps steps each (median reported)")
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--mode", default="exact", choices=["exact", "int8"],
                    help="exact: original bf16 weights as 3 limbs (the headline); int8: int8 weights, 2-limb activations")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-int8-extra", action="store_true", help="skip the int8-mode pass reported under `extra`")
    ap.add_argument("--no-column-sharded", action="store_true",
                    help="N > 1: skip the int8-mode column-sharded pass reported under `extra.column_sharded`")
    ap.add_argument("--no-graph", dest="graph", action="store_false", help="launch kernel by kernel instead of replaying a CUDA graph")
    return ap.parse_args()


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def workload(args, mode=None):
    mode = mode or args.mode
    return (f"BASELINE config {4 if mode == 'exact' else 5}: random-init Llama-3.2-1B {mode}-mode decode, "
            f"{args.prompt}-token uniform random prompts, batch {args.batch} per GPU, T=0.7 integer Gumbel sampler")


# ---------------------------------------------------------------------------------------------------------
# CPU leg: the oracle (numpy restatement of the reference's CPU path) on a bounded sample of the workload:
# one decoder layer + final norm + LM head on SAMPLE_ROWS token rows at contexts near SAMPLE_CTX.

def oracle_model(c_np, mode):
    from oracle.model import OracleInt8Model, OracleModel
    if mode == "int8":
        return OracleInt8Model(c_np)
    m = OracleModel(c_np)
    for lin in list(m.lin.values()) + [m.lm]:
        lin["keep_w64"] = True                                     # the reference keeps its float64 weight copy
    return m


def one_layer_view(c, to_numpy):
    """The constants of layer 0 + embedding + final norm + LM head + tables as a 1-layer constants dict."""
    keep = {}
    for k, v in c.items():
        head = k.split(".")[0]
        if head.isdigit() and head != "0":
            continue
        keep[k] = to_numpy(v)
    keep["n_layers"] = 1
    keep["cfg"] = dict(c["cfg"], num_hidden_layers=1)
    return keep


def make_sample(cfg, mode):
    from oracle import step_sample
    s = step_sample.make_sample(cfg, SAMPLE_ROWS, SAMPLE_CTX, seed=0)
    if mode == "int8":                                              # int8 mode keeps k and v at 14 fractional bits
        s["k"], s["v"] = [k >> 3 for k in s["k"]], [v >> 5 for v in s["v"]]
    return s


def time_oracle(m, sample, reps, warm=1):
    """[(t_layer, t_head)] of `reps` sample steps, and the last step's residual rows and logits."""
    from oracle import step_sample
    out, x, lg = [], None, None
    for i in range(warm + reps):
        cache = step_sample.fill_cache(m, sample)
        rows = len(sample["ids"])
        t0 = time.perf_counter()
        x = m.forward(cache, sample["ids"].tolist(), [int(n) for n in sample["lens"]], list(range(rows)))
        t1 = time.perf_counter()
        lg = m.logits(x)
        t2 = time.perf_counter()
        if i >= warm:
            out.append((t1 - t0, t2 - t1))
    return out, x, lg


def cpu_summary(times, layers, cores):
    t_layer = statistics.median(t for t, _ in times)
    t_head = statistics.median(t for _, t in times)
    step_s = layers * t_layer + t_head
    return {"value": SAMPLE_ROWS / step_s, "unit": "tok/s", "cores": cores, "kind": "port",
            "sample": f"oracle (numpy float64-GEMM port of the reference CPU path): 1 decoder layer + final norm + LM "
                      f"head on {SAMPLE_ROWS} token rows at contexts {SAMPLE_CTX} +- 40, 1B geometry, {len(times)} "
                      f"timed sample steps; scaled to {layers} layers (layer {t_layer * 1e3:.1f} ms, head "
                      f"{t_head * 1e3:.1f} ms): tok/s = {SAMPLE_ROWS} / ({layers} t_layer + t_head)",
            "ms_sample_step": (t_layer + t_head) * 1e3}, step_s


def run_reference(args, rank):
    """The CPU arm. Host only: weights are generated and decomposed on the host, nothing here imports the shared
    library or initialises CUDA. Thread count pinned to the host cores (a launcher's OMP_NUM_THREADS=1 is overridden)."""
    if rank != 0:
        return
    cores = host_cores()
    for var in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[var] = str(cores)                                # before numpy / torch load their BLAS
    os.environ["CUDA_VISIBLE_DEVICES"] = ""
    import threadpoolctl
    import torch

    from bitexact_llm_b200.exact import consts
    torch.set_num_threads(cores)
    cfg = dict(consts.LLAMA_1B)
    cfg["num_hidden_layers"] = 1
    sd = consts.random_state_dict(cfg, seed=0, device="cpu")
    if args.mode == "exact":
        c = consts.build(cfg, sd, n_pos=SAMPLE_CTX + 64)
    else:
        from bitexact_llm_b200.int8 import consts as consts8
        c = consts8.build(cfg, sd, n_pos=2048)
    del sd
    c_np = {k: (v.numpy() if torch.is_tensor(v) else v) for k, v in c.items()}
    m = oracle_model(c_np, args.mode)
    sample = make_sample(cfg, args.mode)
    with threadpoolctl.threadpool_limits(limits=cores):
        used = max([p["num_threads"] for p in threadpoolctl.threadpool_info() if p.get("user_api") == "blas"] or [cores])
        times, _, _ = time_oracle(m, sample, reps=max(1, args.steps), warm=max(1, args.warmup))
    base, step_s = cpu_summary(times, args.layers, used)
    metric = METRIC if args.mode == "exact" else METRIC.replace("exact-mode", "int8-mode")
    line = {"metric": metric, "value": base["value"], "unit": "tok/s", "n_gpus": args.gpus, "steps": len(times),
            "warmup": max(1, args.warmup), "ms_per_step": base["ms_sample_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int64 (float64 GEMM of int8 limbs)", "data": "synthetic",
            "impl": "reference",
            "config": {"workload": workload(args), "batch_per_gpu": args.batch, "prompt": args.prompt,
                       "layers": args.layers, "page": 16,
                       "sample": "each step = one decoder layer + LM head on 64 token rows of this workload "
                                 "(ms_per_step is that sample step); value scales it to the full "
                                 f"{args.layers}-layer step (see cpu_baseline.sample)",
                       "ms_per_full_step_extrapolated": step_s * 1e3},
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------

class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed regions run."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([f.strip() for f in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            self.th.join(timeout=2)

    def summary(self):
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


class LinTimer:
    """CUDA-event pairs around every fused-linear call of an instrumented pass (on the launching stream)."""

    def __init__(self):
        self.pairs, self.on = [], False

    @contextlib.contextmanager
    def __call__(self, M, N, K):
        import torch
        if not self.on:
            yield
            return
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        yield
        e1.record()
        self.pairs.append((e0, e1, M, N, K))

    def totals(self):
        ms = sum(a.elapsed_time(b) for a, b, *_ in self.pairs)
        mnk = sum(float(M) * N * K for *_, M, N, K in self.pairs)
        return ms, mnk, len(self.pairs)


def build_engine(mode, cfg, dev, n_pos, timer):
    """(engine, 1-layer numpy constants for the oracle)."""
    import torch

    from bitexact_llm_b200.exact import consts
    sd = consts.random_state_dict(cfg, seed=0, device=dev)          # same weights on every rank
    to_np = lambda v: v.cpu().numpy() if torch.is_tensor(v) else v
    if mode == "exact":
        from bitexact_llm_b200.vllm_plugin.exact_run import ExactEngine
        c = consts.build(cfg, sd, n_pos=n_pos)
        del sd
        eng = ExactEngine(c, dev)
        for ly in eng.layers:
            for n in ("wqkv", "wo", "wgu", "wd"):
                ly[n].timer = timer
        eng.lm.timer = timer
    else:
        from bitexact_llm_b200.int8 import consts as consts8
        from bitexact_llm_b200.int8.engine import IntEngine
        c = consts8.build(cfg, sd, n_pos=max(2048, n_pos))
        del sd
        eng = IntEngine(c, dev)
        eng.timer = timer
    return eng, c


def parity_leg(eng, c, cfg, mode, cpu_reps):
    """One decoder layer + final norm + LM head of the benchmark's own engine (its layer 0) on the seeded sample,
    against the oracle on the same constants and rows. Returns (parity dict, oracle timings)."""
    import hashlib

    import numpy as np
    import torch

    from bitexact_llm_b200.decode import Session
    from bitexact_llm_b200.vllm_plugin import sampler
    from oracle import step_sample
    to_np = lambda v: v.cpu().numpy() if torch.is_tensor(v) else v
    c1 = one_layer_view(c, to_np)
    sample = make_sample(cfg, mode)
    m = oracle_model(c1, mode)
    times, wx, wlg = time_oracle(m, sample, reps=cpu_reps, warm=1)
    full_L = eng.L
    eng.L = 1                                                        # the same engine object, first layer only
    try:
        # The engine runs the sample inside a batch of the benchmark's size (the sample rows repeated), so that the
        # kernels the timed steps use (chosen by batch size) are the ones compared; the copies must give the same bits.
        R = max(SAMPLE_ROWS, (PARITY_BATCH // SAMPLE_ROWS) * SAMPLE_ROWS)
        ses = Session(eng, R, SAMPLE_CTX + 64, perm_seed=11)
        for r in range(R):
            ses.import_kv(r, torch.from_numpy(sample["k"][r % SAMPLE_ROWS]), torch.from_numpy(sample["v"][r % SAMPLE_ROWS]))
        x = ses.step(torch.from_numpy(np.tile(sample["ids"], R // SAMPLE_ROWS)).to(eng.dev))
        lg = eng.logits(x)
        copies_equal = all(bool(torch.equal(x[i:i + SAMPLE_ROWS], x[:SAMPLE_ROWS])) and
                           bool(torch.equal(lg[i:i + SAMPLE_ROWS], lg[:SAMPLE_ROWS]))
                           for i in range(SAMPLE_ROWS, R, SAMPLE_ROWS))
        x, lg = x[:SAMPLE_ROWS], lg[:SAMPLE_ROWS]
        seeds = list(range(SAMPLE_ROWS))
        rows = torch.tensor([[s, 0, 7, 10] for s in seeds], device=eng.dev)
        tok = sampler.sample_rows(lg, rows, eng.ln, eng.FR).cpu().numpy()
        eng.check()
    finally:
        eng.L = full_L
    if mode == "exact":
        wtok = step_sample.oracle_tokens(m, wlg, seeds, 0, 7, 10)
    else:
        from oracle import sampler as osamp
        g = np.stack([osamp.gumbel(osamp.raw_words(s, 0, wlg.shape[1]), m.c["ln"], m.FR) for s in seeds])
        wtok = osamp.sample(wlg, 7, 10, g)
    xg, lgg = x.cpu().numpy(), lg.cpu().numpy()
    sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()
    par = {"rows": SAMPLE_ROWS, "batch": R, "copies_equal": copies_equal, "context": SAMPLE_CTX, "layers_compared": 1,
           "equal": bool(copies_equal and np.array_equal(xg, wx) and np.array_equal(lgg, wlg) and
                         np.array_equal(tok, wtok)),
           "residual_equal": bool(np.array_equal(xg, wx)), "logits_equal": bool(np.array_equal(lgg, wlg)),
           "tokens_equal": bool(np.array_equal(tok, wtok)), "oracle_flag": bool(m.flag),
           "logits_sha_first": sha(lgg[0]), "oracle_logits_sha_first": sha(wlg[0]),
           "what": "layer 0 + final norm + LM head + T=0.7 sampler of this run's engine, run on the sample rows "
                   "repeated to a batch of `batch` rows, vs the CPU oracle (float64-GEMM port of the reference) on "
                   "the same constants and seeded rows"}
    del ses
    return par, times


class DecodeRun:
    """A session of B sequences after prompt processing, its captured decode step and its host-driven step."""

    def __init__(self, args, eng, cfg, dev, rank, total_steps):
        import torch

        from bitexact_llm_b200.decode import Session
        from bitexact_llm_b200.vllm_plugin import sampler
        self.args, self.eng, self.dev, self.sampler = args, eng, dev, sampler
        B, P = args.batch, args.prompt
        g = torch.Generator().manual_seed(1000 + rank)              # every rank its own sequences
        prompts = torch.randint(0, cfg["vocab_size"], (B, P), generator=g)
        self.ses = Session(eng, B, P + total_steps, perm_seed=rank)
        self.h = self.ses.prefill(prompts, chunk_rows=8192)
        self.rows = torch.zeros(B, 4, dtype=torch.long, device=dev)
        self.rows[:, 0] = torch.arange(B, device=dev) + rank * B    # noise key (seed = global sequence index, t)
        self.rows[:, 2], self.rows[:, 3] = 7, 10                    # T = 0.7

    def eager_step(self):
        lg = self.eng.logits(self.h)
        tok = self.sampler.sample_rows(lg, self.rows, self.eng.ln, self.eng.FR)
        self.rows[:, 1] += 1
        self.h = self.ses.step(tok)
        return tok


def run_b200(args, rank, world):
    import torch
    import torch.distributed as dist

    from bitexact_llm_b200 import _native as nv
    from bitexact_llm_b200.decode import GraphDecoder, GraphHostStep
    from bitexact_llm_b200.exact import consts

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback); use --impl reference for the CPU leg")
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    lib = nv.lib()
    B, P, K, W, R = args.batch, args.prompt, args.steps, args.warmup, max(1, args.repeats)
    exact = args.mode == "exact"

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    cfg = dict(consts.LLAMA_1B)
    cfg["num_hidden_layers"] = args.layers
    span = R * K + 3 * W + K + 24                                   # decode steps any phase runs from the prompt's end
    timer = LinTimer()
    eng, c = build_engine(args.mode, cfg, dev, max(P + span, SAMPLE_CTX + 40) + 64, timer)

    # ---- parity of this engine against the oracle (rank 0), and the CPU baseline timing at N = 1 ----
    parity, cpu_times = None, None
    if rank == 0:
        want_cpu = world == 1 and not args.no_cpu_baseline
        parity, cpu_times = parity_leg(eng, c, cfg, args.mode, cpu_reps=5 if want_cpu else 1)
        if not want_cpu:
            cpu_times = None
    del c
    ok = torch.tensor([1 if (parity is None or parity["equal"]) else 0], device=dev)
    if world > 1:
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if int(ok.item()) == 0:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "error": "GPU result differs from the CPU oracle", "parity": parity}),
                  flush=True)
        raise SystemExit(3)

    peak_best, peak_mean = nv.i8_tensor_peak(1 << 16, 24)           # about 0.4 s of back-to-back kind::i8 MMAs

    run = DecodeRun(args, eng, cfg, dev, rank, span)
    ses, rows = run.ses, run.rows
    for _ in range(W):
        run.eager_step()
    lens0, t0 = ses.lens.clone(), rows[:, 1].clone()
    h0 = run.h.clone()

    def rewind():
        """Back to the state after warm-up: every phase decodes over the same range of context lengths (the cache
        rows beyond are simply rewritten)."""
        ses.lens.copy_(lens0)
        rows[:, 1] = t0
        run.h = h0.clone()

    # ---- timed: R regions of exactly K steps, the whole step replayed from one CUDA graph ----
    dec = GraphDecoder(ses, rows, run.h, warmup=0) if args.graph else None
    step = dec.step if dec else run.eager_step
    for _ in range(W):
        step()
    rewind()
    if dec:
        dec.h.copy_(h0)
    region_ms, e2e_ms = [], []
    with ClockSampler(local) as clk:
        torch.cuda.profiler.start()                                  # capture range for `ncu --profile-from-start off`
        for _ in range(R):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(K):
                step()
            e1.record()
            barrier()
            region_ms.append(e0.elapsed_time(e1))
        torch.cuda.profiler.stop()

        # ---- end to end: every step's inputs (token ids, positions, sampler rows) come from pinned host memory
        # and the sampled tokens are read back to the host; the device work of the step is one graph replay ----
        rewind()
        host_tok = torch.zeros(B, dtype=torch.long).pin_memory()
        host_pos = torch.zeros(B, dtype=torch.long).pin_memory()
        host_rows = rows.cpu().pin_memory()
        host_tok.copy_(run.eager_step())
        torch.cuda.synchronize()
        host_pos.copy_(ses.lens)
        host_rows.copy_(rows)
        hs = GraphHostStep(ses, rows) if args.graph else None

        def step_e2e():
            if hs:
                hs.tok_in.copy_(host_tok, non_blocking=True)
                hs.pos_in.copy_(host_pos, non_blocking=True)
                hs.rows_in.copy_(host_rows, non_blocking=True)
                tok = hs.step()
            else:
                tok_dev = host_tok.to(dev, non_blocking=True)
                pos_dev = host_pos.to(dev, non_blocking=True)
                rows_dev = host_rows.to(dev, non_blocking=True)
                lg = eng.logits(ses.step(tok_dev, pos_dev))
                tok = run.sampler.sample_rows(lg, rows_dev, eng.ln, eng.FR)
            host_tok.copy_(tok, non_blocking=True)
            torch.cuda.current_stream().synchronize()                # the host has the tokens
            host_pos.add_(1)
            host_rows[:, 1] += 1

        for _ in range(W):
            step_e2e()
        for _ in range(R):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(K):
                step_e2e()
            e1.record()
            barrier()
            e2e_ms.append(e0.elapsed_time(e1))

    # kernels per step are the same whether replayed or launched one by one: count them on an eager step
    rewind()
    n0 = lib.bx_launch_count()
    run.eager_step()
    launches_per_step = lib.bx_launch_count() - n0
    # ---- instrumented eager pass: CUDA-event pairs around every limb GEMM of K steps (roofline) ----
    barrier()
    timer.on = True
    for _ in range(K):
        run.eager_step()
    barrier()
    timer.on = False
    lin_ms, lin_mnk, lin_calls = timer.totals()
    eng.check()

    # ---- int8 mode beside the exact-mode headline: decode rate and the GEMM rate at 4 M N K ops ----
    int8_extra = None
    if exact and world == 1 and not args.no_int8_extra:
        dec = hs = None
        int8_extra = int8_pass(args, cfg, dev, peak_mean)

    # ---- N > 1: the column-sharded configuration, the one place where the data path crosses NVLink ----
    sharded_extra = None
    if world > 1 and not args.no_column_sharded:
        dec = hs = run = ses = eng = None                      # free the exact-mode engine and its cache
        torch.cuda.empty_cache()
        sharded_extra = column_sharded_pass(args, cfg, dev, rank, world)

    times = torch.tensor(region_ms + e2e_ms, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    times = times.tolist()
    region_ms, e2e_ms = times[:R], times[R:]
    if rank != 0:
        return

    peaks = {}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except OSError:
        pass
    bf16 = peaks.get("bf16_tflops_sustained")
    proxy = 2.0 * bf16 if bf16 else 2.0 * 1400.0
    ops_per_mnk = 18.0 if exact else 4.0
    achieved = ops_per_mnk * lin_mnk / (lin_ms * 1e-3) / 1e12
    ms, ms_e2e = statistics.median(region_ms), statistics.median(e2e_ms)
    tok = lambda t: world * B * K / (t * 1e-3)
    # algorithmic bytes of a launch: weight limbs once + activations + int64 outputs (exact: 3 N K + 4 M K + 8 M N;
    # int8: N K + 2 M K + 8 M N), mean over the GEMM launches of the instrumented pass
    wb, ab = (3, 4) if exact else (1, 2)
    alg_bytes_per_launch = sum(wb * N * Kk + ab * M * Kk + 8 * M * N for *_, M, N, Kk in timer.pairs) / lin_calls
    metric = METRIC if exact else METRIC.replace("exact-mode", "int8-mode")
    kernel = ("exact_linear_kernel / exact_linear_persistent_kernel (tcgen05 kind::i8 limb GEMM, 3 x 3 limbs, fused epilogue)"
              if exact else "int8_linear_kernel (tcgen05 kind::i8, 1 x 2 limbs, fused post epilogue)")
    line = {
        "metric": metric, "value": tok(ms), "unit": "tok/s", "n_gpus": world, "steps": K,
        "warmup": W, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 limbs -> int32 -> int64", "data": "synthetic",
        "config": {"workload": workload(args), "batch_per_gpu": B, "prompt": P, "layers": args.layers, "page": 16,
                   "parallelism": f"sequence-sharded x{world}, no data-path collective",
                   "l2": "inputs larger than L2 (3.7 GB of weight limbs + KV pages read per step)",
                   "launch": "one CUDA graph replay per step" if args.graph else "kernel by kernel",
                   "contexts": f"{P + W + 1}..{P + W + R * K} keys over the {R} regions (config 4 decodes 512..768)"},
        "repeats": {"regions": R, "steps_per_region": K, "ms_per_step_median": ms / K,
                    "ms_per_step_min": min(region_ms) / K, "ms_per_step_max": max(region_ms) / K,
                    "value_min": tok(max(region_ms)), "value_max": tok(min(region_ms)),
                    "timed_seconds": (sum(region_ms) + sum(e2e_ms)) * 1e-3},
        "e2e": {"value": tok(ms_e2e), "unit": "tok/s", "h2d_bytes_per_step": 48 * B, "d2h_bytes_per_step": 8 * B,
                "ms_per_step": ms_e2e / K, "ms_per_step_min": min(e2e_ms) / K, "ms_per_step_max": max(e2e_ms) / K},
        "gpu_launches": int(launches_per_step * K),
        "clocks": clk.summary(),
        "parity": parity,
        "roofline": {"bound": "tensor", "kernel": kernel,
                     "achieved": achieved, "peak": peak_mean, "unit": "TFLOP/s",
                     "ops": f"int8 ({'2*9' if exact else '2*2'}*M*N*K per call)",
                     "frac": achieved / peak_mean,
                     "peak_source": "measured in this run: tcgen05.mma kind::i8 M128 N256 K32 loop on shared-memory "
                                    "operands, one CTA per SM, mean of 24 back-to-back launches (about 0.4 s)",
                     "peak_i8_measured": peak_mean, "peak_i8_measured_burst": peak_best,
                     "peak_proxy_2x_bf16_sustained": proxy, "frac_of_proxy": achieved / proxy,
                     "frac_of_nominal_4500": achieved / 4500.0,
                     "calls": lin_calls, "ms_per_step": lin_ms / K,
                     "traffic": 1.02 * alg_bytes_per_launch,
                     "traffic_note": "1.02 x the algorithmic bytes per launch computed in this run (weight limbs once + "
                                     "activation planes + int64 outputs, mean over the step's GEMM launches); the factor "
                                     "is the ncu dram read+write / algorithmic ratio of profiles/"
                                     "exact_linear_limb_gemm_ncu.md (102.6 MB measured vs 100.7 MB for gate/up)",
                     "algorithmic_bytes_per_launch": alg_bytes_per_launch},
        "extra": {"limb_gemm_int8_tops": achieved, "limb_gemm_ms_per_step_eager": lin_ms / K},
    }
    if int8_extra:
        line["extra"]["int8_mode"] = int8_extra
    if sharded_extra:
        line["extra"]["column_sharded"] = sharded_extra
    if cpu_times:
        line["cpu_baseline"], _ = cpu_summary(cpu_times, args.layers, host_cores())
    print(json.dumps(line), flush=True)


class CollectiveTimer:
    """CUDA-event pairs around every collective of `bitexact_llm_b200.parallel` while `on`."""

    def __init__(self):
        self.on, self.spans = False, []

    @contextlib.contextmanager
    def span(self, name, nbytes):
        import torch
        if not self.on:
            yield
            return
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        yield
        e1.record()
        self.spans.append((name, nbytes, e0, e1))

    def summary(self, steps):
        out = {}
        for name, nbytes, e0, e1 in self.spans:
            d = out.setdefault(name, {"calls_per_step": 0.0, "ms_per_step": 0.0, "bytes_per_step": 0.0})
            d["calls_per_step"] += 1.0 / steps
            d["ms_per_step"] += e0.elapsed_time(e1) / steps
            d["bytes_per_step"] += nbytes / steps
        return out


def column_sharded_pass(args, cfg, dev, rank, world):
    """BASELINE config 5: int8 mode, 64 sequences per GPU (512 on 8) with prompt lengths U[16, 4096], sequences
    sharded over the ranks, MLP and LM head + sampler sharded by output column (NCCL all-gathers of the int8 limb
    planes and the int64 outputs, integer all-reduce MAX of the SiLU row maxima, all-gather of the (max, index)
    pairs). Returns the decode rate over all ranks and the per-step time of every collective."""
    import torch
    import torch.distributed as dist

    from bitexact_llm_b200 import parallel as par
    from bitexact_llm_b200.decode import Session
    from bitexact_llm_b200.exact import consts
    from bitexact_llm_b200.int8 import consts as consts8
    K, W = args.steps, args.warmup
    per = 64
    span = 3 * K + 2 * W + 8
    sd = consts.random_state_dict(cfg, seed=0, device=dev)
    c = consts8.build(cfg, sd, n_pos=4096 + span + 64)
    del sd
    eng = par.ColumnShardedIntEngine(c, dev)
    del c
    g = torch.Generator().manual_seed(5000 + rank)
    lens = torch.randint(16, 4097, (per,), generator=g)
    P = int(lens.max())
    prompts = torch.randint(0, cfg["vocab_size"], (per, P), generator=g)
    ses = Session(eng, per, 4096 + span, perm_seed=rank)
    eng.sharded = False
    h = ses.prefill(prompts, lens, chunk_rows=8192)
    eng.sharded = True
    rows_all = torch.zeros(per * world, 4, dtype=torch.long, device=dev)
    rows_all[:, 0] = torch.arange(per * world, device=dev)
    rows_all[:, 2], rows_all[:, 3] = 7, 10
    state = {"h": h}

    def step():
        tok = eng.sample(state["h"], rows_all)
        rows_all[:, 1] += 1
        state["h"] = ses.step(tok)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    for _ in range(W):
        step()
    regions = []
    for _ in range(2):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            step()
        e1.record()
        barrier()
        regions.append(e0.elapsed_time(e1))
    timer = CollectiveTimer()
    par.TIMER = timer
    timer.on = True
    for _ in range(K):
        step()
    barrier()
    timer.on = False
    par.TIMER = None
    eng.check()
    t = torch.tensor([min(regions)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    coll = timer.summary(K)
    return {"workload": "BASELINE config 5: int8 mode, 64 sequences per GPU, prompt lengths U[16, 4096] (seeded), "
                        "sequence-sharded attention, MLP and LM head + sampler sharded by output column",
            "value": world * per * K / (ms * 1e-3), "unit": "tok/s", "ms_per_step": ms / K,
            "launch": "kernel by kernel (NCCL collectives between the kernels)",
            "collectives": coll, "collective_ms_per_step": sum(d["ms_per_step"] for d in coll.values()),
            "mean_context": float(lens.float().mean()) + W + K}


def int8_pass(args, cfg, dev, peak):
    """int8 mode on the same workload: decode rate from R short regions and the GEMM rate (2 * 2 * M * N * K ops) from
    an instrumented eager pass."""
    import torch

    from bitexact_llm_b200.decode import GraphDecoder
    K, W = args.steps, args.warmup
    R = min(3, max(1, args.repeats))
    timer = LinTimer()
    eng, c = build_engine("int8", cfg, dev, args.prompt + (R + 2) * K + 2 * W + 80, timer)
    del c
    run = DecodeRun(args, eng, cfg, dev, 0, (R + 2) * K + 2 * W + 16)
    for _ in range(W):
        run.eager_step()
    dec = GraphDecoder(run.ses, run.rows, run.h, warmup=0)
    for _ in range(W):
        dec.step()
    regions = []
    for _ in range(R):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            dec.step()
        e1.record()
        torch.cuda.synchronize()
        regions.append(e0.elapsed_time(e1))
    run.h = dec.h
    timer.on = True
    for _ in range(K):
        run.eager_step()
    torch.cuda.synchronize()
    timer.on = False
    eng.check()
    lin_ms, lin_mnk, calls = timer.totals()
    ms = statistics.median(regions)
    tops = 4.0 * lin_mnk / (lin_ms * 1e-3) / 1e12
    return {"value": args.batch * K / (ms * 1e-3), "unit": "tok/s", "ms_per_step": ms / K,
            "roofline": {"kernel": "int8_linear_kernel (tcgen05 kind::i8, 1 x 2 limbs, fused post epilogue)",
                         "achieved": tops, "unit": "TFLOP/s", "ops": "int8 (2*2*M*N*K per call)", "peak": peak,
                         "frac": tops / peak, "calls": calls, "ms_per_step": lin_ms / K}}


def main():
    args = parse()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
        dist.init_process_group("nccl")
    try:
        run_b200(args, rank, world)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
