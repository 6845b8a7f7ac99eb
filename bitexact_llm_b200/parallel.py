"""Multi-GPU layout of the hot path: one process per GPU, `torch.distributed` for the plumbing.

Two shardings, both exact (no value is ever reduced in floating point, so every GPU count gives the same bits):

* sequence sharding  - every rule of the engine is row-local, so rank r simply owns a contiguous block of the
                       batch (its own KV cache, no communication).
* column sharding    - a large-N projection (LM head, gate/up) is split by OUTPUT columns: y[m, n] depends only on
                       row m and weight row n. Each rank computes y[:, n0:n1]; one all-gather of the int64 outputs
                       rebuilds y. The sampler needs no full row at all: each rank reduces its shard to a
                       (max, first index) pair per row and the pairs are all-gathered.

The reference is single-GPU (README "TP = 1, PP = 1"); these helpers are the new part the multi-GPU configs need.
The collective wrappers take any process group (NCCL on GPUs; the unit tests run them on CPU tensors over gloo).
"""

import contextlib

import torch
import torch.distributed as dist

# Optional timing of the collectives: set TIMER to an object with a context-manager method
# `span(name, payload_bytes)` (bench.py does, to report the per-step time of each exchange); None = no timing.
TIMER = None


def _span(name, nbytes):
    return TIMER.span(name, nbytes) if TIMER is not None else contextlib.nullcontext()


def shard_bounds(n, world, rank):
    """Contiguous near-equal split of n items: [lo, hi) of `rank` (the first n % world ranks get one more)."""
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def column_bounds(N, world, rank, align=1):
    """[n0, n1) of `rank` when N output columns are split evenly (N % (world * align) must be 0)."""
    if N % (world * align):
        raise ValueError(f"{N} columns do not split over {world} ranks in multiples of {align}")
    per = N // world
    return rank * per, (rank + 1) * per


def shard_linear_constants(c, name, n0, n1):
    """The constants of weight rows [n0, n1) of linear `name` (reference key layout), residual rows re-based."""
    rr = c[f"{name}.rr"]
    keep = (rr >= n0) & (rr < n1)
    return {"limbs": c[f"{name}.limbs"][:, n0:n1].contiguous(), "g": c[f"{name}.g"][n0:n1].contiguous(),
            "d": c[f"{name}.d"][n0:n1].contiguous(), "rr": rr[keep] - n0, "rc": c[f"{name}.rc"][keep],
            "rv": c[f"{name}.rv"][keep]}


def gather_columns(y_local, group=None):
    """y_local int [M, n_local] on every rank (equal shapes) -> y [M, world * n_local] (rank-major columns)."""
    world = dist.get_world_size(group)
    if world == 1:
        return y_local
    y_local = y_local.contiguous()
    M, nl = y_local.shape
    out = torch.empty((world * M, nl), dtype=y_local.dtype, device=y_local.device)      # rank-major blocks of rows
    with _span("all_gather_columns", out.numel() * out.element_size()):
        dist.all_gather_into_tensor(out, y_local, group=group)
    return out.view(world, M, nl).permute(1, 0, 2).reshape(M, world * nl)


def gather_rows(x_local, group=None):
    """x_local [m_local, ...] (equal m_local on every rank) -> [world * m_local, ...] in rank order."""
    world = dist.get_world_size(group)
    if world == 1:
        return x_local
    x_local = x_local.contiguous()
    out = torch.empty((world * x_local.shape[0],) + tuple(x_local.shape[1:]), dtype=x_local.dtype,
                      device=x_local.device)
    with _span("all_gather_rows", out.numel() * out.element_size()):
        dist.all_gather_into_tensor(out, x_local, group=group)
    return out


def gather_planes(a8, group=None):
    """Limb planes [P, m_local, K] of every rank's rows -> [P, world * m_local, K] (rows in rank order)."""
    world = dist.get_world_size(group)
    if world == 1:
        return a8
    P, m, K = a8.shape
    return gather_rows(a8.contiguous().view(P * m, K), group).view(world, P, m, K).permute(1, 0, 2, 3).reshape(
        P, world * m, K).contiguous()


def gather_scaled_rows(a8, mant, e, group=None):
    """The input of an int8-mode linear for ALL ranks' rows from each rank's own: a8 int8 [2, n, K] limb planes, mant
    and e int64 [n] -> ([2, world n, K], [world n], [world n]) in rank order, with ONE all-gather: every row travels
    as limb 0 | limb 1 | mant | e (2 K + 16 bytes), because at decode sizes an exchange costs its launch, not its
    bytes."""
    world = dist.get_world_size(group)
    if world == 1:
        return a8, mant, e
    P, n, K = a8.shape
    row = torch.cat([a8.permute(1, 0, 2).reshape(n, P * K).view(torch.uint8), mant.contiguous().view(torch.uint8).view(n, 8),
                     e.contiguous().view(torch.uint8).view(n, 8)], 1)
    out = gather_rows(row, group)
    N = world * n
    planes = out[:, :P * K].view(torch.int8).view(N, P, K).permute(1, 0, 2).contiguous()
    tail = out[:, P * K:].contiguous().view(torch.int64).view(N, 2)
    return planes, tail[:, 0].contiguous(), tail[:, 1].contiguous()


def combine_argmax(best, idx, group=None):
    """Per-row (shard maximum, first global index) pairs of every rank -> the row's first argmax over all shards:
    the larger value wins, then the smaller index."""
    world = dist.get_world_size(group)
    if world == 1:
        return idx
    pair = torch.stack([best, idx], 1).contiguous()                       # [M, 2] int64
    allp = torch.empty((world * pair.shape[0], 2), dtype=pair.dtype, device=pair.device)
    with _span("all_gather_argmax_pairs", allp.numel() * 8):
        dist.all_gather_into_tensor(allp, pair, group=group)
    allp = allp.view(world, pair.shape[0], 2)
    b, i = allp[..., 0], allp[..., 1]                                     # [world, M]
    top = b.amax(0, keepdim=True)
    big = torch.iinfo(torch.int64).max
    return torch.where(b == top, i, torch.full_like(i, big)).amin(0)


def allreduce_max(x, group=None):
    """Integer maximum over the ranks, in place (exact: no arithmetic, only comparisons)."""
    if dist.get_world_size(group) > 1:
        with _span("all_reduce_max", x.numel() * x.element_size()):
            dist.all_reduce(x, op=dist.ReduceOp.MAX, group=group)
    return x


def allreduce_sum(x, group=None):
    """Integer sum over the ranks, in place (exact in any order while the total stays below 2^63)."""
    if dist.get_world_size(group) > 1:
        dist.all_reduce(x, op=dist.ReduceOp.SUM, group=group)
    return x


def sharded_logp_q(lg, v0, tok, lnt, fr=16, group=None):
    """Integer log p (int64 [M] at 2^-40, identical on every rank) of tok [M] from a COLUMN SHARD of the logits:
    lg int64 [M, V_local] holds vocabulary entries v0 .. v0 + V_local - 1 of every row. Three exchanges on [M]: the
    integer maximum of the shard maxima, the integer sum of the shards' e^(l - max) sums, and the target term from the
    one rank that holds the token. The bits are those of `vllm_plugin.rl.int_logp_q` on the gathered rows."""
    from . import _native as nv
    from .vllm_plugin.rl import pair_table
    M, Vl = lg.shape
    assert lg.dtype == torch.int64 and lg.stride(1) == 1
    lib, dev, st = nv.lib(), lg.device, nv.stream()
    tab = pair_table(dev)
    scratch = torch.empty(max(1, lib.bx_logp_scratch_bytes(M, Vl)), dtype=torch.uint8, device=dev)
    mx = torch.empty(M, dtype=torch.long, device=dev)
    nv.check(lib.bx_logp_rowmax(lg.data_ptr(), lg.stride(0), scratch.data_ptr(), mx.data_ptr(), M, Vl, st),
             "bx_logp_rowmax")
    allreduce_max(mx, group)
    S = torch.empty(M, dtype=torch.long, device=dev)
    nv.check(lib.bx_logp_rowsum(lg.data_ptr(), lg.stride(0), mx.data_ptr(), tab.data_ptr(), tab.shape[0],
                                scratch.data_ptr(), S.data_ptr(), M, Vl, fr, st), "bx_logp_rowsum")
    allreduce_sum(S, group)
    loc = tok.long() - v0
    mine = (loc >= 0) & (loc < Vl)
    zt = torch.where(mine, lg.gather(1, loc.clamp(0, Vl - 1)[:, None])[:, 0] - mx, torch.full_like(mx, -(1 << 63)))
    allreduce_max(zt, group)                                  # exactly one rank holds the token's column
    out = torch.empty(M, dtype=torch.long, device=dev)
    nv.check(lib.bx_logp_finish(S.data_ptr(), zt.data_ptr(), lnt.data_ptr(), out.data_ptr(), M, fr, st),
             "bx_logp_finish")
    return out


def shard_gate_up_constants(c, name, FF, f0, f1):
    """Constants of the fused gate / up linear `name` (weight rows [0, FF) = gate, [FF, 2 FF) = up) restricted to the
    intermediate columns [f0, f1): the rank's gate rows followed by its up rows."""
    a = shard_linear_constants(c, name, f0, f1)
    b = shard_linear_constants(c, name, FF + f0, FF + f1)
    n = f1 - f0
    return {"limbs": torch.cat([a["limbs"], b["limbs"]], 1).contiguous(), "g": torch.cat([a["g"], b["g"]]),
            "d": torch.cat([a["d"], b["d"]]), "rr": torch.cat([a["rr"], b["rr"] + n]),
            "rc": torch.cat([a["rc"], b["rc"]]), "rv": torch.cat([a["rv"], b["rv"]])}


class ShardedMLP:
    """Column-sharded MLP of one layer: rank r holds intermediate columns [f0, f1) of gate and up and output columns
    [d0, d1) of down. Two exchanges per call: the integer maximum of the SiLU row maxima (so that every shard
    quantises with the row exponent of the full row) with an all-gather of the quantised shard, and the all-gather
    of the down outputs. Nothing is summed across ranks, so every world size gives the bits of the single GPU."""

    def __init__(self, c, layer, FF, device, group=None):
        from .exact.model import Lin
        from .vllm_plugin.exact_gemm import FusedLin
        self.group, self.FF = group, FF
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.f0, self.f1 = column_bounds(FF, self.world, self.rank, 16)
        D = c[f"{layer}.wd.limbs"].shape[1]
        self.d0, self.d1 = column_bounds(D, self.world, self.rank)
        self.wgu = FusedLin(Lin(shard_gate_up_constants(c, f"{layer}.wgu", FF, self.f0, self.f1), None, device))
        self.wd = FusedLin(Lin(shard_linear_constants(c, f"{layer}.wd", self.d0, self.d1), None, device))

    def __call__(self, q, sh, lut, flag):
        """q int32 [M, D], sh int64 [M] (the normalised input, identical on every rank) -> the down projection's
        output y int64 [M, D] at 24 bits, identical on every rank."""
        from . import _native as nv
        lib = nv.lib()
        M = q.shape[0]
        FFl = self.f1 - self.f0
        dev = q.device
        y = self.wgu(q, sh, flag, False)                                   # [M, 2 FFl]
        P = torch.empty(M, FFl, dtype=torch.long, device=dev)
        rmax = torch.empty(M, dtype=torch.long, device=dev)
        nv.check(lib.bx_exact_silu_prod(y.data_ptr(), lut.data_ptr(), P.data_ptr(), rmax.data_ptr(), flag.data_ptr(), M,
                                        FFl, nv.stream()), "bx_exact_silu_prod")
        allreduce_max(rmax, self.group)
        ql = torch.empty(M, FFl, dtype=torch.int32, device=dev)
        shq = torch.empty(M, dtype=torch.long, device=dev)
        nv.check(lib.bx_exact_quant_rows(P.data_ptr(), rmax.data_ptr(), 48, ql.data_ptr(), FFl, shq.data_ptr(), None, 0,
                                         M, FFl, nv.stream()), "bx_exact_quant_rows")
        qf = gather_columns(ql, self.group)                               # [M, FF]: every rank needs all of K
        return gather_columns(self.wd(qf.contiguous(), shq, flag, True), self.group)


class ShardedHead:
    """Column-sharded LM head + sampler: rank r holds vocabulary rows [v0, v1) of the LM head; logits never leave
    the shard unless `full_logits` is called (test / hashing mode)."""

    def __init__(self, c, device, group=None):
        from .exact.model import Lin
        from .vllm_plugin.exact_gemm import FusedLin
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        V = c["lm.limbs"].shape[1]
        self.v0, self.v1 = column_bounds(V, self.world, self.rank)
        self.lin = FusedLin(Lin(shard_linear_constants(c, "lm", self.v0, self.v1), None, device))

    def local_logits(self, q, sh, flag):
        return self.lin(q, sh, flag, True)

    def full_logits(self, q, sh, flag):
        return gather_columns(self.local_logits(q, sh, flag), self.group)

    def sample(self, q, sh, flag, rows, lnt, fr=24):
        """rows int64 [M, 4] = (seed, t, tn, td) on the device -> tokens int64 [M] (identical on every rank)."""
        from . import _native as nv
        lg = self.local_logits(q, sh, flag)
        M, Vl = lg.shape
        lib = nv.lib()
        best = torch.empty(M, dtype=torch.long, device=lg.device)
        idx = torch.empty(M, dtype=torch.long, device=lg.device)
        scratch = torch.empty(max(1, lib.bx_sample_scratch_bytes(M, Vl)), dtype=torch.uint8, device=lg.device)
        rc = lib.bx_sample_shard(lg.data_ptr(), lg.stride(0), rows.data_ptr(), lnt.data_ptr(), scratch.data_ptr(),
                                 best.data_ptr(), idx.data_ptr(), M, Vl, self.v0, fr, nv.stream())
        nv.check(rc, "bx_sample_shard")
        return combine_argmax(best, idx, self.group)


class ShardedHeadInt8:
    """Column-sharded LM head + sampler of int8 mode: rank r holds rows [v0, v1) of the int8 LM-head weight and of its
    per-channel multipliers; logits (16 fractional bits) never leave the shard unless `full_logits` is called."""

    def __init__(self, c, device, group=None, nl=2):
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        V = c["lm"].shape[0]
        self.v0, self.v1 = column_bounds(V, self.world, self.rank)
        self.w = c["lm"][self.v0:self.v1].to(device).contiguous()
        self.m = c["lm.m"][self.v0:self.v1].to(device).contiguous()
        self.fmsh = int(c["lm.fm"]) + 8 * (nl - 1) - 24

    def local_logits(self, a8, mant, e, flag):
        from .int8.gemm_skinny import linear_post
        return linear_post(a8, self.w, self.m, self.fmsh, mant, e, flag, True)

    def full_logits(self, a8, mant, e, flag):
        return gather_columns(self.local_logits(a8, mant, e, flag), self.group)

    def sample(self, a8, mant, e, flag, rows, lnt):
        """rows int64 [M, 4] = (seed, t, tn, td) on the device -> tokens int64 [M] (identical on every rank)."""
        from . import _native as nv
        lg = self.local_logits(a8, mant, e, flag)
        M, Vl = lg.shape
        lib = nv.lib()
        best = torch.empty(M, dtype=torch.long, device=lg.device)
        idx = torch.empty(M, dtype=torch.long, device=lg.device)
        scratch = torch.empty(max(1, lib.bx_sample_scratch_bytes(M, Vl)), dtype=torch.uint8, device=lg.device)
        rc = lib.bx_sample_shard(lg.data_ptr(), lg.stride(0), rows.data_ptr(), lnt.data_ptr(), scratch.data_ptr(),
                                 best.data_ptr(), idx.data_ptr(), M, Vl, self.v0, 16, nv.stream())
        nv.check(rc, "bx_sample_shard")
        return combine_argmax(best, idx, self.group)


class ShardedMLPInt8:
    """Column-sharded MLP of one int8-mode layer: rank r holds intermediate columns [f0, f1) of gate and up (int8
    weight rows and their channel multipliers) and output columns [d0, d1) of down. As in exact mode, the SiLU
    product is quantised per FULL row: the shards' row maxima of |h| meet in an integer all-reduce MAX between
    `bx_int8_silu_prod` and `bx_int8_quant_rows` (the reference's one-kernel form: `tri_mlp.silu_quant`,
    src/bitexact/vllm_plugin/tri_mlp.py:153-183 = int8/segs.py:111-118), then two all-gathers rebuild the rows: the
    int8 limb planes of the quantised shard, and the int64 down outputs. Nothing is summed across ranks."""

    def __init__(self, c, layer, FF, device, group=None, nl=2):
        self.group, self.FF = group, FF
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.f0, self.f1 = column_bounds(FF, self.world, self.rank, 16)
        w, m = c[f"{layer}.wgu"], c[f"{layer}.wgu.m"]
        rows = torch.cat([torch.arange(self.f0, self.f1), torch.arange(FF + self.f0, FF + self.f1)])
        self.wgu = w[rows.to(w.device)].to(device).contiguous()
        self.mgu = m[rows.to(m.device)].to(device).contiguous()
        self.fm_gu = int(c[f"{layer}.wgu.fm"]) + 8 * (nl - 1) - 24
        wd = c[f"{layer}.wd"]
        self.d0, self.d1 = column_bounds(wd.shape[0], self.world, self.rank)
        self.wd = wd[self.d0:self.d1].to(device).contiguous()
        self.md = c[f"{layer}.wd.m"][self.d0:self.d1].to(device).contiguous()
        self.fm_d = int(c[f"{layer}.wd.fm"]) + 8 * (nl - 1) - 24

    def __call__(self, a8, mant, e, silu_t, flag, scr=None):
        """(a8 int8 [2 M, D] limb planes, mant, e [M]): the normalised input of ALL rows, identical on every rank ->
        the down projection's output y int64 [M, D] at 16 bits, identical on every rank. scr int64 [2]: receives the
        rank's maxima of |silu(gate)| and |up| (the caller takes their maximum over the ranks before `flag_end`)."""
        from . import _native as nv
        from .int8.gemm_skinny import linear_post
        lib, dev = nv.lib(), a8.device
        M = mant.shape[0]
        FFl = self.f1 - self.f0
        y = linear_post(a8, self.wgu, self.mgu, self.fm_gu, mant, e, flag, True)          # [M, 2 FFl]
        h = torch.empty(M, FFl, dtype=torch.long, device=dev)
        rmax = torch.empty(M, dtype=torch.long, device=dev)
        nv.check(lib.bx_int8_silu_prod(y.data_ptr(), silu_t.data_ptr(), h.data_ptr(), rmax.data_ptr(), nv.ptr(scr), M,
                                       FFl, nv.stream()), "bx_int8_silu_prod")
        allreduce_max(rmax, self.group)
        al = torch.empty(2, M, FFl, dtype=torch.int8, device=dev)
        mant2 = torch.empty(M, dtype=torch.long, device=dev)
        e2 = torch.empty(M, dtype=torch.long, device=dev)
        nv.check(lib.bx_int8_quant_rows(h.data_ptr(), rmax.data_ptr(), al.data_ptr(), mant2.data_ptr(), e2.data_ptr(), M,
                                        FFl, nv.stream()), "bx_int8_quant_rows")
        af = gather_columns(al.view(2 * M, FFl), self.group).contiguous()                   # [2 M, FF]: all of K
        return gather_columns(linear_post(af, self.wd, self.md, self.fm_d, mant2, e2, flag, True), self.group)


class ColumnShardedIntEngine:
    """int8 mode over `world` GPUs with BOTH shardings of the 8-GPU configuration: every rank owns a block of the
    sequences (its KV cache, attention, the attention-side linears and every row-local stage), while the MLP and the
    LM head + sampler run on ALL ranks' rows with the weights split by output column. Per layer: one all-gather of the
    normalised rows (int8 limb planes + row scales), the exchanges of `ShardedMLPInt8`, and each rank keeps its own
    rows of the result; per step one more row gather in front of the column-sharded head. Every rank must hold the
    same number of rows. Same integers as `IntEngine` on one GPU."""

    def __init__(self, c, dev, group=None):
        from .int8.engine import IntEngine
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.base = IntEngine(c, dev)
        b = self.base
        FF = c["0.wgu"].shape[0] // 2
        self.mlps = [ShardedMLPInt8(c, i, FF, dev, group) for i in range(b.L)]
        self.head = ShardedHeadInt8(c, dev, group)
        self.sharded = True          # False: every call runs on this rank alone (prompt processing: the ranks' row
        #                              counts differ from chunk to chunk, and the column exchange needs equal blocks)
        for a in ("dev", "D", "H", "HKV", "HD", "L", "FR", "ln", "fl", "emb", "V"):
            setattr(self, a, getattr(b, a))

    def check(self):
        self.base.check()

    def _rows(self, x):
        n = x.shape[0] // self.world
        return x[self.rank * n:(self.rank + 1) * n]

    def forward(self, kvs, ids, pos, slot, bt, rmap, tiles=None):
        """IntEngine.forward on this rank's rows, the MLP of every layer column-sharded over all ranks' rows
        (with `sharded` off, or for prompt tiles: the plain single-GPU forward with this rank's full weights)."""
        from .vllm_plugin import tri_fuse as fz
        from .vllm_plugin import tri_paged
        b = self.base
        if not self.sharded or tiles is not None:
            return b.forward(kvs, ids, pos, slot, bt, rmap, tiles=tiles)
        N, G = ids.shape[0], b.H // b.HKV
        pos = pos.long()
        slot = torch.where(slot < 0, torch.zeros_like(slot), slot).long()
        qpos = pos.view(-1, 1).expand(-1, G).contiguous()
        x, *pre = fz.embed_norm(b, ids, b.layers[0]["ga"])
        for i in range(b.L):
            ly = b.layers[i]
            q = fz.qkv(b, b._lin(pre, ly["wqkv"]), None, None, None, pos, slot, kvs[i], int32=True)
            num, den = tri_paged.attend(q, qpos, kvs[i], bt, b.ptab, rmap=rmap)
            x, a8, mant, e = fz.add_norm(b, b._lin(fz.attn_out(b, num, den), ly["wo"]), None, None, None, x, ly["gm"])
            A, Ma, Ea = gather_scaled_rows(a8.view(2, N, b.D), mant, e, self.group)
            y = self.mlps[i](A.view(2 * N * self.world, b.D), Ma, Ea, b.silu_t, b.fl, b.scr[i])
            nxt = b.layers[i + 1]["ga"] if i + 1 < b.L else None
            x, *pre = fz.add_norm(b, self._rows(y).contiguous(), None, None, None, x, nxt)
        allreduce_max(b.scr, self.group)                     # the product-bound maxima of every rank's columns
        fz.flag_end(b, b.scr)
        return x

    def sample(self, h, rows_all):
        """Final residual rows of this rank [n, D] and the sampler rows (seed, t, tn, td) of ALL ranks' rows
        [world n, 4] -> the tokens of this rank's rows (LM head and sampler column-sharded over all rows)."""
        from .vllm_plugin import tri_fuse as fz
        b = self.base
        a8, mant, e = fz.pre_norm(b, h, b.gf)
        n = h.shape[0]
        A, Ma, Ea = gather_scaled_rows(a8.view(2, n, b.D), mant, e, self.group)
        tok = self.head.sample(A.view(2 * n * self.world, b.D), Ma, Ea, b.fl, rows_all, b.ln)
        return self._rows(tok)

    def logits(self, h):
        """Full logits rows of this rank's rows (gathers the vocabulary shards: test / hashing mode)."""
        from .vllm_plugin import tri_fuse as fz
        b = self.base
        if not self.sharded:
            return b.logits(h)
        a8, mant, e = fz.pre_norm(b, h, b.gf)
        n = h.shape[0]
        A, Ma, Ea = gather_scaled_rows(a8.view(2, n, b.D), mant, e, self.group)
        return self._rows(self.head.full_logits(A.view(2 * n * self.world, b.D), Ma, Ea, b.fl))
