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
