"""Exact-mode element-wise stages: drop-in for `bitexact.vllm_plugin.exact_fuse`
(src/bitexact/vllm_plugin/exact_fuse.py:342-414), one sm_100a kernel per stage.

`m` is the model object of the reference's wrappers: it provides D, H, HKV, HD, emb (int32 [V, D]), cos / sin
(int64 [max_pos, HD / 2]) and dev. `fl` is the sticky int32 [1] bound flag."""

import torch

from .. import _native as nv


def attach_planes(q, planes):
    """Remembers the limb planes a stage kernel wrote next to q, together with q's version counter and address:
    `FusedLin` uses them only while q has not been written since (an in-place edit of q bumps the counter)."""
    q._bx_planes = (planes, q._version, q.data_ptr())


def planes_of(q, M, K):
    """The limb planes attached to q if they still describe it, else None."""
    rec = getattr(q, "_bx_planes", None)
    if rec is None:
        return None
    planes, version, addr = rec
    if version != q._version or addr != q.data_ptr() or planes.shape != (3, M, K) or not q.is_contiguous():
        return None
    return planes


def _norm(m, x, y, ids, gamma, fl, mode, norm, store):
    M, D = (ids.shape[0], m.D) if mode == 0 else x.shape
    assert D & (D - 1) == 0 and 32 <= D <= 4096
    dev = m.dev
    xin = m.emb if mode == 0 else x.contiguous()
    xo = torch.empty(M, D, dtype=torch.long, device=dev) if store else None
    q = torch.empty(M, D, dtype=torch.int32, device=dev) if norm else None
    sh = torch.empty(M, dtype=torch.long, device=dev) if norm else None
    gm, ge = gamma if gamma is not None else (None, None)
    planes = torch.empty(3, M, D, dtype=torch.int8, device=dev) if norm else None
    rc = nv.lib().bx_exact_norm(mode, xin.data_ptr(), nv.ptr(y.contiguous() if y is not None else None),
                                nv.ptr(ids.contiguous() if ids is not None else None), nv.ptr(gm), nv.ptr(ge),
                                nv.ptr(xo), nv.ptr(q), nv.ptr(sh), nv.ptr(planes), fl.data_ptr(), M, D, int(norm),
                                nv.stream())
    nv.check(rc, "bx_exact_norm")
    if norm:
        attach_planes(q, planes)                         # the next fused linear skips its limb-splitting pass
    return (xo if store else x), q, sh


def embed_norm(m, ids, gamma, fl):
    """x = emb[ids] (int64) and pre_norm(x, gamma) -> (x, q, sh)."""
    return _norm(m, None, None, ids, gamma, fl, 0, True, True)


def add_norm(m, y, x, gamma, fl):
    """x + y and, when gamma is given, pre_norm of it -> (x, q, sh); else (x, None, None) with the bound flag."""
    x, q, sh = _norm(m, x, y, None, gamma, fl, 1, gamma is not None, True)
    return (x, q, sh) if gamma is not None else (x, None, None)


def pre_norm(m, h, gamma, fl):
    """pre_norm of h -> (q, sh)."""
    return _norm(m, h, None, None, gamma, fl, 2, True, False)[1:]


def qkv(m, y, pos, slot, cache, fl):
    """qkv linear output y [N, (H + 2 HKV) HD] -> (q int32 [N, H HD], sh int64 [N, H]); K / V stored at slot in
    cache (int8 limb planes [nb, HKV, bs, 8 HD]; None: no store)."""
    N = y.shape[0]
    H, HKV, HD = m.H, m.HKV, m.HD
    q = torch.empty(N, H * HD, dtype=torch.int32, device=m.dev)
    sh = torch.empty(N, H, dtype=torch.long, device=m.dev)
    if cache is not None:
        assert cache.stride(3) == 1 and cache.dtype == torch.int8
        st, bs = cache.stride()[:3], cache.shape[2]
    else:
        st, bs = (0, 0, 0), 1
    rc = nv.lib().bx_exact_qkv(y.contiguous().data_ptr(), m.cos.data_ptr(), m.sin.data_ptr(),
                               pos.long().contiguous().data_ptr(),
                               nv.ptr(slot.long().contiguous() if slot is not None else None), nv.ptr(cache), *st, bs,
                               q.data_ptr(), sh.data_ptr(), fl.data_ptr(), N, H, HKV, HD, nv.stream())
    nv.check(rc, "bx_exact_qkv")
    return q, sh


def attn_out(m, num, den):
    """num [N, HKV, G, HD] (any shape with N rows of H HD), den likewise [.., 1] -> (q int32 [N, H HD], sh [N])."""
    N = num.shape[0]
    K2 = m.H * m.HD
    q = torch.empty(N, K2, dtype=torch.int32, device=m.dev)
    sh = torch.empty(N, dtype=torch.long, device=m.dev)
    planes = torch.empty(3, N, K2, dtype=torch.int8, device=m.dev)
    rc = nv.lib().bx_exact_attn_out(num.contiguous().data_ptr(), den.contiguous().data_ptr(), q.data_ptr(),
                                    sh.data_ptr(), planes.data_ptr(), N, K2, m.HD, nv.stream())
    nv.check(rc, "bx_exact_attn_out")
    attach_planes(q, planes)
    return q, sh


def silu_quant(m, y, lut, fl):
    """gate_up output y [N, 2 FF] -> (q int32 [N, FF], sh [N]) of quant(silu(g) u, -48)."""
    N, FF = y.shape[0], y.shape[1] // 2
    q = torch.empty(N, FF, dtype=torch.int32, device=m.dev)
    sh = torch.empty(N, dtype=torch.long, device=m.dev)
    planes = torch.empty(3, N, FF, dtype=torch.int8, device=m.dev)
    rc = nv.lib().bx_exact_silu_quant(y.contiguous().data_ptr(), lut.data_ptr(), q.data_ptr(), sh.data_ptr(),
                                      planes.data_ptr(), fl.data_ptr(), N, FF, nv.stream())
    nv.check(rc, "bx_exact_silu_quant")
    attach_planes(q, planes)
    return q, sh
