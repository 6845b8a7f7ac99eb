"""Exact-mode paged attention: drop-in for `bitexact.vllm_plugin.tri_exact_attn.attend`
(src/bitexact/vllm_plugin/tri_exact_attn.py:138-165)."""

import torch

from .. import _native as nv


def _scratch(device, pairs, nblk, bs):
    """Scratch for the scores of contexts beyond the shared-memory buffer of the streaming kernel: only when the
    block table is wide enough to need it and there are enough (request, KV head) pairs for that kernel."""
    if nblk * bs <= 896 or pairs < 296:
        return None, 0
    n = nv.lib().bx_attention_scratch_bytes(nblk, bs)
    return torch.empty(n, dtype=torch.uint8, device=device), n


def attend(q, sh, qpos, cache, bt, rmap, lut, l2e, nsplit=None, bn=64, warps=4, variant=0):
    """q int32 [R, HKV, M, HD] (M <= 4, |q| <= 2^22), sh int64 [R, HKV, M], qpos int64 [R, M] (key s visible to
    query i iff s <= qpos[r, i]), cache int8 limb planes [nb, HKV, bs, 8 HD], bt [*, nblk] block table, rmap int64
    [R], lut = 2^-f table (int64), l2e = round(log2(e) 2^28). Returns num int64 [R, HKV, M, HD], den [R, HKV, M, 1].

    nsplit maps to the cluster size (keys split over the CTAs of a thread-block cluster; rounded to 1, 2, 4, 8);
    bn and warps are accepted and ignored. None of them can change a bit of the result."""
    R, HKV, M, HD = q.shape
    assert M <= 4 and cache.shape[1] == HKV and cache.shape[3] == 8 * HD and cache.stride(3) == 1
    assert bt.shape[1] * cache.shape[2] < 43690 and q.dtype == torch.int32
    assert bt.dtype in (torch.int32, torch.int64) and bt.stride(1) == 1
    q, sh, qpos = q.contiguous(), sh.contiguous(), qpos.contiguous()
    num = torch.empty(R, HKV, M, HD, dtype=torch.long, device=q.device)
    den = torch.empty(R, HKV, M, 1, dtype=torch.long, device=q.device)
    cs = 0
    if nsplit is not None:
        cs = 1
        while cs < min(int(nsplit), 8):
            cs *= 2
    ws, ws_bytes = _scratch(q.device, R * HKV, bt.shape[1], cache.shape[2])
    rc = nv.lib().bx_exact_attention_ws(q.data_ptr(), sh.data_ptr(), qpos.data_ptr(), cache.data_ptr(), cache.shape[0],
                                        cache.stride(0), cache.stride(1), cache.stride(2), cache.shape[2], bt.data_ptr(),
                                        int(bt.dtype == torch.int64), bt.stride(0), bt.shape[1],
                                        nv.ptr(rmap.long().contiguous() if rmap is not None else None), lut.data_ptr(),
                                        int(l2e), num.data_ptr(), den.data_ptr(), R, HKV, M, HD, cs, variant,
                                        nv.ptr(ws), ws_bytes, nv.stream())
    nv.check(rc, "bx_exact_attention_ws")
    return num, den
