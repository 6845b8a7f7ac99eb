"""A minimal decode loop over `ExactEngine`: paged-cache bookkeeping, chunked prompt processing, greedy /
Gumbel-max sampling and per-position logits hashes (the reference's `generate` / `logits_sha`,
src/bitexact/generate.py:21-50, on a batch of sequences with one block-table row each)."""

import hashlib

import torch

from .vllm_plugin import sampler


def logits_sha(row):
    """SHA-256 (hex) of one int64 logits row: equal hashes <=> bit-identical logits."""
    return hashlib.sha256(row.contiguous().cpu().numpy().tobytes()).hexdigest()


class Session:
    """B sequences, each with a contiguous run of cache blocks (block 0 is the null block)."""

    def __init__(self, eng, B, max_len, bs=16, perm_seed=None):
        self.eng, self.B, self.bs = eng, B, bs
        self.nblk = (max_len + bs - 1) // bs
        nb = 1 + B * self.nblk
        dev = eng.dev
        self.kvs = [torch.zeros(nb, eng.HKV, bs, 8 * eng.HD, dtype=torch.int8, device=dev) for _ in range(eng.L)]
        blocks = torch.arange(1, nb, dtype=torch.int64)
        if perm_seed is not None:                                  # scattered pages
            g = torch.Generator().manual_seed(perm_seed)
            blocks = blocks[torch.randperm(nb - 1, generator=g)]
        self.bt = blocks.view(B, self.nblk).to(torch.int32).to(dev)
        self.lens = torch.zeros(B, dtype=torch.long, device=dev)
        self.rows = torch.arange(B, device=dev)

    def _slots(self, seq, pos):
        return self.bt[seq, pos // self.bs].long() * self.bs + pos % self.bs

    @torch.no_grad()
    def import_kv(self, seq, k, v, layers=None):
        """Loads keys / values of positions 0 .. n - 1 of sequence `seq` (int64 [n, HKV, HD] at 17 / 19 fractional
        bits, within three limbs) into the paged cache of the given layers (default: all) and sets the sequence's
        length to n: a prefix computed elsewhere, e.g. by another engine or an earlier session."""
        from .vllm_plugin import tri_paged
        dev = self.eng.dev
        k, v = k.to(dev).long().contiguous(), v.to(dev).long().contiguous()
        n = k.shape[0]
        pos = torch.arange(n, device=dev)
        slot = self._slots(torch.full_like(pos, int(seq)), pos)
        for i in (range(self.eng.L) if layers is None else layers):
            tri_paged.store(self.kvs[i], slot, k, v)
        self.lens[seq] = n

    @torch.no_grad()
    def prefill(self, prompts, lens=None, chunk_rows=4096, tiles=True):
        """prompts: int64 [B, P] right-padded, lens [B] the true lengths (default: all P). Token rows are processed
        in position chunks so that every row's keys are in the cache before it attends; with `tiles` the attention
        of a chunk runs on the prefill tile kernel (runs of 32 / G consecutive tokens share their K / V staging),
        else every token is a row of the decode kernel. Same integers either way. Returns the final residual row of
        each sequence [B, D]."""
        from .vllm_plugin import tri_prefill
        B, P = prompts.shape
        dev = self.eng.dev
        prompts = prompts.to(dev)
        lens_host = [P] * B if lens is None else [int(v) for v in lens.tolist()]
        lens = torch.full((B,), P, dtype=torch.long, device=dev) if lens is None else lens.to(dev).long()
        G = self.eng.H // self.eng.HKV
        # the tile kernel pays for itself once a tile walks a few key blocks (measured: 0.83 x the row kernel on
        # 128-token prompts, 1.7 x on 2048-token ones); short chunks at the start of a prompt stay on rows
        use_tiles = tiles and self.eng.HD == 64 and tri_prefill.BM % G == 0 and self.bs in (8, 16, 32, 64, 128)
        tile_from = 0 if tiles == "always" else 384
        step = max(1, chunk_rows // B)
        last = torch.zeros(B, self.eng.D, dtype=torch.long, device=dev)
        for p0 in range(0, P, step):
            p1 = min(P, p0 + step)
            grid = torch.arange(p0, p1, device=dev).expand(B, -1)
            live = grid < lens[:, None]
            if not bool(live.any()):
                break
            pos = grid[live]                                                      # sequence-major rows
            seq = self.rows[:, None].expand(-1, p1 - p0)[live]
            tt = None
            if use_tiles and p1 > tile_from:                                    # sequence-major rows: runs per sequence
                pre, row0 = [], 0
                for b in range(B):
                    n = max(0, min(p1, lens_host[b]) - p0)
                    if n:
                        pre.append((b, row0, n, p0 + n))
                    row0 += n
                tt = tri_prefill.tile_table(pre, G, tri_prefill.ROWS).to(dev)
            x = self.eng.forward(self.kvs, prompts[:, p0:p1][live], pos, self._slots(seq, pos), self.bt, seq, tiles=tt)
            fin = pos == lens[seq] - 1
            last[seq[fin]] = x[fin]
        self.lens += lens
        return last

    @torch.no_grad()
    def step(self, tokens, pos=None):
        """One decode step: tokens int64 [B] at positions `pos` (default: the lengths tracked on the device).
        Returns the residual rows [B, D]."""
        pos = self.lens.clone() if pos is None else pos
        x = self.eng.forward(self.kvs, tokens, pos, self._slots(self.rows, pos), self.bt, self.rows)
        self.lens += 1
        return x


class GraphDecoder:
    """The decode step (LM head, sampler, one forward over the batch) captured once in a CUDA graph and replayed:
    no Python or launch overhead per kernel. The step's state lives in static device tensors: the residual rows,
    the sampler rows (seed, t, tn, td) whose t advances on the device, the session's lengths."""

    def __init__(self, ses, rows, h, warmup=2):
        self.ses, self.eng = ses, ses.eng
        self.rows = rows
        self.h = h.clone()
        self.tok = torch.zeros(ses.B, dtype=torch.long, device=h.device)
        for _ in range(warmup):                     # configures every kernel and fills the caching allocator
            self._body()
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._body()

    def _body(self):
        lg = self.eng.logits(self.h)
        tok = sampler.sample_rows(lg, self.rows, self.eng.ln, self.eng.FR)
        self.h.copy_(self.ses.step(tok))
        self.rows[:, 1] += 1
        self.tok.copy_(tok)

    def step(self):
        """Runs one captured step; returns the sampled tokens (a static tensor, overwritten by the next step)."""
        self.graph.replay()
        return self.tok


class GraphHostStep:
    """One decode step driven from the host, captured in a CUDA graph: the caller copies this step's token ids,
    positions and sampler rows into the static input tensors (`tok_in`, `pos_in`, `rows_in`), replays, and reads
    the sampled tokens from `tok`. Forward, LM head and sampler run inside the graph."""

    def __init__(self, ses, rows):
        self.ses, self.eng = ses, ses.eng
        dev = rows.device
        self.tok_in = torch.zeros(ses.B, dtype=torch.long, device=dev)
        self.pos_in = ses.lens.clone()
        self.rows_in = rows.clone()
        self.tok = torch.zeros(ses.B, dtype=torch.long, device=dev)
        keep = ses.lens.clone()
        for _ in range(2):
            self._body()
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._body()
        ses.lens.copy_(keep)                         # warm-up and capture advanced the device-side lengths

    def _body(self):
        x = self.ses.step(self.tok_in, self.pos_in)
        lg = self.eng.logits(x)
        self.tok.copy_(sampler.sample_rows(lg, self.rows_in, self.eng.ln, self.eng.FR))

    def step(self):
        self.graph.replay()
        return self.tok


@torch.no_grad()
def generate(eng, prompts, max_new, tn=0, td=1, seeds=None, hashes=True, max_len=None, perm_seed=None, lens=None):
    """prompts int64 [B, P] (right-padded, true lengths `lens`); generated token t of sequence b uses the noise
    keyed (seeds[b], t). Returns (tokens [B, max_new] on the host, list of per-position hash lists or None)."""
    B, P = prompts.shape
    dev = eng.dev
    seeds = list(range(B)) if seeds is None else seeds
    ses = Session(eng, B, max_len or (P + max_new), perm_seed=perm_seed)
    h = ses.prefill(prompts, lens)
    rows = torch.zeros(B, 4, dtype=torch.long, device=dev)
    rows[:, 0] = torch.tensor(seeds, device=dev)
    rows[:, 2], rows[:, 3] = tn, td
    toks, shas = [], [[] for _ in range(B)]
    for t in range(max_new):
        lg = eng.logits(h)
        rows[:, 1] = t
        y = sampler.sample_rows(lg, rows, eng.ln, eng.FR)
        toks.append(y)
        if hashes:
            for b in range(B):
                shas[b].append(logits_sha(lg[b]))
        if t + 1 < max_new:
            h = ses.step(y)
    eng.check()
    return torch.stack(toks, 1).cpu(), (shas if hashes else None)
