"""Host-side batch layout of one forward call over vLLM's paged KV cache: drop-in for `Plan`, `PreGroup`,
`make_plan` and `kv_view` of `bitexact.vllm_plugin.paged` (src/bitexact/vllm_plugin/paged.py:32-113).

vLLM describes a step by `query_start_loc` [R + 1], `seq_lens` [R], `block_table` [R, max_blocks] and
`slot_mapping` [n]. The reference turns that into decode rows (one query token) and groups of prefill requests
padded to a common query count, and runs its attention kernel once per group. The kernels of this package take
token rows instead: every query token is a row with its own position and a block-table ROW INDEX (`rmap`), so a
mixed batch is one launch with no padding. `Plan.rmap` / `Plan.rows()` give that form; the reference's fields
(`dec_req`, `dec_tok`, `pre`, `groups()`) are kept with the same contents for callers written against them.
Why the result cannot depend on the layout: every rule is row-local and masked keys get weight 0 before any
reduction (paged.py:9-15 of the reference)."""

from dataclasses import dataclass

import torch

H, HD = 32, 64                                       # Llama-3.2-1B query heads and head size (llama.py of the reference)
GROUP_BYTES = 1 << 28                                # cap on the padded int64 query tensor of one prefill group


@dataclass
class PreGroup:
    req: torch.Tensor           # [n] request of each tile
    idx: torch.Tensor           # [n, Tm] token index of each query (padding: the tile's first token)
    pos: torch.Tensor           # [n, Tm] its position
    valid: torch.Tensor         # [n, Tm] bool
    dst: torch.Tensor           # [n_valid] token index of each valid query (row-major over valid)


@dataclass
class Plan:
    """Batch layout of one forward call (one device-to-host copy per call)."""
    n: int                      # real tokens (the rest is padding)
    slot: torch.Tensor          # [n] int64 slot of each token
    block_table: torch.Tensor   # [R, max_blocks] int64
    dec_req: torch.Tensor       # [Rd] requests with one query token
    dec_tok: torch.Tensor       # [Rd] their token index
    pre: list                   # [(req, tok0, qlen, seq_len)] requests with more than one query token
    positions: torch.Tensor = None   # [N] position of each token
    qdim: int = H * HD
    rmap: torch.Tensor = None   # [n] int64 request (block-table row) of each token: the token-row form
    _groups: list = None

    def groups(self):
        """Prefill requests as padded query tiles (PreGroup), built on first use."""
        if self._groups is None:
            self._groups = _pre_groups(self.pre, self.positions, self.block_table.device, self.qdim)
        return self._groups

    def rows(self, n_tokens=None):
        """(slot, block_table, rmap) for a token-row engine call over n_tokens rows (default: the real tokens).
        Rows beyond the real tokens are padding: slot -1 (no store) and request 0."""
        N = self.n if n_tokens is None else n_tokens
        slot, rmap = self.slot[:N], self.rmap[:N]
        if N > self.n:
            pad = N - self.n
            slot = torch.cat([slot, slot.new_full((pad,), -1)])
            rmap = torch.cat([rmap, rmap.new_zeros(pad)])
        return slot, self.block_table, rmap


def _pre_groups(pre, positions, dev, qdim=H * HD):
    """Prefill requests, shortest first, in groups padded to the group's longest query count; a group is closed
    when one more request would take its padded int64 query tensor past GROUP_BYTES."""
    out, members = [], []

    def close():
        if not members:
            return
        tm = max(q for _, _, q, _ in members)
        first = torch.tensor([t0 for _, t0, _, _ in members])
        qlen = torch.tensor([q for _, _, q, _ in members])
        step = torch.arange(tm)
        valid = step[None, :] < qlen[:, None]
        idx = first[:, None] + torch.where(valid, step[None, :].expand_as(valid), torch.zeros_like(valid, dtype=torch.long))
        idx_d = idx.to(dev, non_blocking=True)
        out.append(PreGroup(req=torch.tensor([r for r, _, _, _ in members]).to(dev, non_blocking=True), idx=idx_d,
                            pos=positions[idx_d].long(), valid=valid.to(dev, non_blocking=True),
                            dst=idx[valid].to(dev, non_blocking=True)))
        members.clear()

    for item in sorted(pre, key=lambda t: t[2]):
        if members and (len(members) + 1) * item[2] * qdim * 8 > GROUP_BYTES:
            close()
        members.append(item)
    close()
    return out


def make_plan(meta, n_tokens, positions, qdim=H * HD):
    """meta: an object with query_start_loc, seq_lens, block_table and slot_mapping tensors (vLLM's attention
    metadata); n_tokens: rows of the forward call; positions [N]."""
    starts = meta.query_start_loc.cpu().tolist()
    lens = meta.seq_lens.cpu().tolist()
    R = len(lens)
    n = starts[R]
    dev = meta.block_table.device
    dec_req, dec_tok, pre = [], [], []
    for r in range(R):
        q = starts[r + 1] - starts[r]
        if q == 1:
            dec_req.append(r)
            dec_tok.append(starts[r])
        elif q > 1:
            pre.append((r, starts[r], q, lens[r]))
    counts = torch.tensor([starts[r + 1] - starts[r] for r in range(R)], dtype=torch.long)
    rmap = torch.repeat_interleave(torch.arange(R, dtype=torch.long), counts).to(dev)
    mk = lambda xs: torch.tensor(xs, dtype=torch.long, device=dev)
    return Plan(n=min(n, n_tokens), slot=meta.slot_mapping[:n].long(), block_table=meta.block_table.long(),
                dec_req=mk(dec_req), dec_tok=mk(dec_tok), pre=pre, positions=positions, qdim=qdim, rmap=rmap)


def kv_view(kv):
    """vLLM's bf16 cache view [nb, HKV, bs, 2 * 2 * HD] -> int8 limb planes [nb, HKV, bs, 8 * HD]."""
    assert kv.dim() == 4 and kv.shape[3] % 4 == 0 and kv.stride(3) == 1, (kv.shape, kv.stride())
    return kv.view(torch.int8)
