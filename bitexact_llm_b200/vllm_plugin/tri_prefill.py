"""int8-mode prefill attention on the token-major layout: drop-in for `bitexact.vllm_plugin.tri_prefill`
(src/bitexact/vllm_plugin/tri_prefill.py:86-108).

Key s is visible to a query iff s <= its position, and every sum is an exact integer reduction, so the grouping of
query tokens into tiles cannot change a bit: each token of a tile is one row (its G query heads share the position)
of the paged attention kernel, with the request's block-table row. Everything stays on the device."""

import torch

from . import tri_paged

BM = 32     # query rows per tile of the reference (BM // G tokens)
BN = 64


def tile_table(pre, G, bm=BM):
    """[T, 3] int32 (request, first token, tokens) of the bm // G-token tiles of the prefill requests
    pre = [(req, tok0, qlen, seq_len)], on the host."""
    bt_ = bm // G
    return torch.tensor([[r, t0 + s, min(bt_, ql - s)] for r, t0, ql, _ in pre for s in range(0, ql, bt_)],
                        dtype=torch.int32).reshape(-1, 3)


def attend(q, pos, cache, bt, ptab, tiles, num, den, bm=BM, bn=BN, warps=4):
    """q int64 [N, HKV, G, HD], pos int64 [N], cache int8 limb planes, bt [R, *] block table, tiles (tile_table, on
    the device) -> the rows of the tiles' tokens of num int64 [N, HKV, G, HD] and den [N, HKV, G, 1] written in place.
    bn and warps are tuning arguments of the reference, ignored."""
    N, HKV, G, HD = q.shape
    assert bm % G == 0 and num.is_contiguous() and den.is_contiguous() and q.is_contiguous()
    T = tiles.shape[0]
    if T == 0:
        return
    per = bm // G
    tl_ = tiles.long()
    s = torch.arange(per, device=q.device)[None, :]
    # padding slots of a short tile repeat its last token: the same integers are written twice
    tok = (tl_[:, 1:2] + torch.minimum(s, tl_[:, 2:3] - 1)).reshape(-1)
    req = tl_[:, 0:1].expand(T, per).reshape(-1)
    qpos = pos.long()[tok][:, None].expand(-1, G).contiguous()
    n_, d_ = tri_paged.attend(q[tok], qpos, cache, bt, ptab, rmap=req)
    num[tok] = n_
    den[tok] = d_
