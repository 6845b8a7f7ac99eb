"""Paged int8 limb-plane KV cache helpers: drop-in for `bitexact.vllm_plugin.tri_paged.store / to_limbs`
(src/bitexact/vllm_plugin/tri_paged.py:311-348).

Cache layout, per (block, KV head, slot) row of 8 HD bytes: K limbs 0, 1, 2 at bytes [0, 3 HD), V limbs at
[3 HD, 6 HD); the rest of the row is unused."""

import torch

from .. import _native as nv


def store(c, slot, k, v):
    """Write K / V (int64 [N, HKV, HD], |.| within 3 limbs) of the tokens at cache slots slot [N] into the
    limb-plane cache c (int8 [nb, HKV, bs, 8 HD]); slot < 0 is skipped."""
    N, hkv, hd = k.shape
    assert c.stride(3) == 1 and k.stride(2) == 1 and v.stride(2) == 1
    if N:
        rc = nv.lib().bx_kv_store(c.data_ptr(), c.stride(0), c.stride(1), c.stride(2), c.shape[2],
                                  slot.long().contiguous().data_ptr(), k.data_ptr(), k.stride(0), k.stride(1),
                                  v.data_ptr(), v.stride(0), v.stride(1), N, hkv, hd, nv.stream())
        nv.check(rc, "bx_kv_store")


def to_limbs(c):
    """int32 cache [nb, HKV, bs, 2 HD] (K | V) -> the int8 limb-plane layout (test / conversion helper)."""
    HD = c.shape[-1] // 2
    out = torch.zeros(*c.shape[:3], 8 * HD, dtype=torch.int8, device=c.device)
    for part, o in ((c[..., :HD], 0), (c[..., HD:], 3)):
        r = part.long()
        for i in range(3):
            lo = ((r + 128) & 255) - 128
            out[..., (o + i) * HD:(o + i + 1) * HD] = lo.to(torch.int8)
            r = (r - lo) >> 8
    return out


def weight_table(lut):
    """The attention weight table rsh(exp_lut, 30 - 20) as int32 (src/bitexact/vllm_plugin/tri_paged.py:351-356)."""
    t = (lut + (1 << 9)) >> 10
    return t.to(torch.int32).contiguous()


def attend(q, qpos, cache, bt, ptab, nsplit=None, bm=None, bn=None, warps=4, rmap=None, variant=0):
    """int8-mode paged attention, M <= 4 query rows per (request, KV head): q int64 (or int32) [R, HKV, M, HD] within
    3 limbs, qpos int64 [R, M], cache int8 limb planes [nb, HKV, bs, 8 HD], bt [R, *] block-table rows, ptab =
    weight_table(exp table). Returns num int64 [R, HKV, M, HD], den int64 [R, HKV, M, 1]
    (src/bitexact/vllm_plugin/tri_paged.py:363-430, decode form). nsplit maps to the cluster size; bm, bn, warps are
    accepted and ignored."""
    R, HKV, M, HD = q.shape
    assert M <= 4 and HD == 64 and cache.shape[1] == HKV and cache.shape[3] == 8 * HD and cache.stride(3) == 1
    assert bt.shape[1] * cache.shape[2] < 43690 and bt.dtype in (torch.int32, torch.int64) and bt.stride(1) == 1
    q32 = q.to(torch.int32).contiguous()
    qpos = qpos.contiguous()
    num = torch.empty(R, HKV, M, HD, dtype=torch.long, device=q.device)
    den = torch.empty(R, HKV, M, 1, dtype=torch.long, device=q.device)
    cs = 0
    if nsplit is not None:
        cs = 1
        while cs < min(int(nsplit), 8):
            cs *= 2
    from .tri_exact_attn import _scratch
    ws, ws_bytes = _scratch(q.device, R * HKV, bt.shape[1], cache.shape[2])
    rc = nv.lib().bx_int8_attention_ws(q32.data_ptr(), qpos.data_ptr(), cache.data_ptr(), cache.shape[0], cache.stride(0),
                                       cache.stride(1), cache.stride(2), cache.shape[2], bt.data_ptr(),
                                       int(bt.dtype == torch.int64), bt.stride(0), bt.shape[1],
                                       nv.ptr(rmap.long().contiguous() if rmap is not None else None), ptab.data_ptr(),
                                       num.data_ptr(), den.data_ptr(), R, HKV, M, HD, cs, variant, nv.ptr(ws), ws_bytes,
                                       nv.stream())
    nv.check(rc, "bx_int8_attention_ws")
    return num, den
