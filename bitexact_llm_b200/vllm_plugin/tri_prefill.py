"""Prefill attention on the token-major layout: drop-in for `bitexact.vllm_plugin.tri_prefill`
(src/bitexact/vllm_plugin/tri_prefill.py:86-108) on the tile kernel of libbitexact_b200 (`bx_prefill_attention`).

One CTA handles a tile of consecutive query tokens of one request and one KV head: every K / V row is staged once
per tile, both sweeps run inside the CTA, the limb products run on tcgen05. Key s is visible to a query iff
s <= its position and every sum is an exact integer reduction, so the grouping of tokens into tiles cannot change a
bit. The same kernel serves exact mode (`attend_exact`: per-row exponents and the 2^-f table), which has no
multi-token attention kernel in the reference."""

import torch

from .. import _native as nv

BM = 32     # query rows per tile (BM // G tokens): the reference's default
BN = 64
ROWS = 32   # tile height the kernel runs by default: 32 query rows per CTA (16: two smaller CTAs per SM; measured
#             equal on 512-token prompts, 5 % slower on 2048-token ones)


def tile_table(pre, G, bm=BM):
    """[T, 3] int32 (request, first token, tokens) of the bm // G-token tiles of the prefill requests
    pre = [(req, tok0, qlen, seq_len)], on the host."""
    bt_ = max(1, min(bm, 32) // G)
    return torch.tensor([[r, t0 + s, min(bt_, ql - s)] for r, t0, ql, _ in pre for s in range(0, ql, bt_)],
                        dtype=torch.int32).reshape(-1, 3)


def _fit(tiles, G, rows):
    """Tiles taller than the kernel's `rows` query rows are cut into pieces of rows // G tokens (on the device)."""
    per = max(1, rows // G)
    if tiles.shape[0] == 0 or int(tiles[:, 2].max()) <= per:
        return tiles.contiguous()
    t = tiles.long()
    pieces = (t[:, 2] + per - 1) // per
    idx = torch.repeat_interleave(torch.arange(t.shape[0], device=t.device), pieces)
    first = torch.cumsum(pieces, 0) - pieces
    k = torch.arange(idx.shape[0], device=t.device) - first[idx]
    out = torch.stack([t[idx, 0], t[idx, 1] + k * per, torch.minimum(t[idx, 2] - k * per, torch.full_like(k, per))], 1)
    return out.to(torch.int32).contiguous()


def _run(q32, sh, pos, cache, bt, tiles, lut, l2e, ptab, num, den, rows=None):
    N, HKV, G, HD = q32.shape
    rows = ROWS if rows is None else rows
    assert rows in (16, 32) and G <= rows
    assert HD == 64 and BM % G == 0 and cache.shape[1] == HKV and cache.shape[3] == 8 * HD and cache.stride(3) == 1
    assert bt.shape[1] * cache.shape[2] < 43690 and bt.dtype in (torch.int32, torch.int64) and bt.stride(1) == 1
    assert num.is_contiguous() and den.is_contiguous() and q32.is_contiguous() and tiles.dtype == torch.int32
    tiles = _fit(tiles, G, rows)
    if tiles.shape[0] == 0:
        return
    rc = nv.lib().bx_prefill_attention(q32.data_ptr(), nv.ptr(sh), pos.data_ptr(), tiles.data_ptr(), tiles.shape[0],
                                       cache.data_ptr(), cache.shape[0], cache.stride(0), cache.stride(1),
                                       cache.stride(2), cache.shape[2], bt.data_ptr(), int(bt.dtype == torch.int64),
                                       bt.stride(0), bt.shape[1], nv.ptr(lut), int(l2e), nv.ptr(ptab), num.data_ptr(),
                                       den.data_ptr(), HKV, G, HD, rows, nv.stream())
    nv.check(rc, "bx_prefill_attention")


def attend(q, pos, cache, bt, ptab, tiles, num, den, bm=BM, bn=BN, warps=4):
    """q int64 (or int32) [N, HKV, G, HD], pos int64 [N], cache int8 limb planes, bt [R, *] block table, tiles
    (tile_table, on the device) -> the rows of the tiles' tokens of num int64 [N, HKV, G, HD] and den [N, HKV, G, 1]
    written in place. bm, bn and warps are tuning arguments of the reference: accepted, no effect on results."""
    _run(q.to(torch.int32).contiguous(), None, pos.long().contiguous(), cache, bt, tiles, None, 0, ptab, num, den)


def attend_exact(q, sh, pos, cache, bt, tiles, lut, l2e, num=None, den=None, rows=None):
    """Exact-mode prefill attention: q int32 [N, HKV, G, HD] (|q| <= 2^22), sh int64 [N, HKV, G], pos int64 [N];
    lut = 2^-f table, l2e = round(log2(e) 2^28). Returns (num int64 [N, HKV, G, HD], den [N, HKV, G, 1]); rows of
    tokens outside every tile (padding) come back as num = 0, den = 1."""
    N, HKV, G, HD = q.shape
    assert q.dtype == torch.int32
    if num is None:
        num = torch.zeros(N, HKV, G, HD, dtype=torch.long, device=q.device)
        den = torch.ones(N, HKV, G, 1, dtype=torch.long, device=q.device)
    _run(q.contiguous(), sh.contiguous(), pos.long().contiguous(), cache, bt, tiles, lut, l2e, None, num, den, rows)
    return num, den
