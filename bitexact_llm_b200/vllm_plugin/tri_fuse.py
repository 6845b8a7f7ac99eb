"""int8-mode element-wise stages: drop-in for `bitexact.vllm_plugin.tri_fuse` and `tri_mlp.silu_quant`
(src/bitexact/vllm_plugin/tri_fuse.py:82-265, vllm_plugin/tri_mlp.py:153-183).

A linear's input is (limbs, mant, e): int8 limb planes [2 M, K] (limb i of row m at row i M + m) and the row scale.
The reference's stages take the RAW int_mm output `c` and apply `post` themselves; here `post` is normally fused into
the GEMM (`int8.gemm_skinny.linear_post`), so every stage accepts either the raw `c` (int32, with `lin = (w, m,
fmsh)` and the producing rows' `mant, e`) or the finished output `y` (int64, `lin = None`).
`m` provides D, H, HKV, HD, emb, cos, sin, dev and the sticky flag tensor `m.fl` (int32 [1])."""

import torch

from .. import _native as nv


def _y(m, c, lin, mant, e):
    """post(c) when c is a raw int_mm output, c itself when it already is the int64 linear output."""
    if c.dtype == torch.int64:
        return c
    M = mant.shape[0]
    N = c.shape[1]
    y = torch.empty(M, N, dtype=torch.long, device=c.device)
    rc = nv.lib().bx_int8_post(c.data_ptr(), lin[1].data_ptr(), int(lin[2]), mant.data_ptr(), e.data_ptr(),
                               y.data_ptr(), m.fl.data_ptr(), M, N, 1, nv.stream())
    nv.check(rc, "bx_int8_post")
    return y


def _run(m, x, y, ids, gamma, mode, norm):
    M = ids.shape[0] if mode == 0 else x.shape[0]
    D = m.D
    dev = m.dev
    xo = torch.empty(M, D, dtype=torch.long, device=dev)
    q = torch.empty(2 * M, D, dtype=torch.int8, device=dev) if norm else None
    nm = torch.empty(M, dtype=torch.long, device=dev) if norm else None
    ne = torch.empty(M, dtype=torch.long, device=dev) if norm else None
    xin = m.emb if mode == 0 else x.contiguous()
    rc = nv.lib().bx_int8_norm(mode, xin.data_ptr(), nv.ptr(y), nv.ptr(ids), nv.ptr(gamma), xo.data_ptr(), nv.ptr(q),
                               nv.ptr(nm), nv.ptr(ne), m.fl.data_ptr(), M, D, int(norm), nv.stream())
    nv.check(rc, "bx_int8_norm")
    return xo, q, nm, ne


def embed_norm(m, ids, gamma):
    """x = emb[ids] and pre_norm(x, gamma) -> (x, limbs, mant, e)."""
    return _run(m, None, None, ids.long().contiguous(), gamma, 0, True)


def add_norm(m, c, lin, mant, e, x, gamma):
    """x + post(c) and, when gamma is given, pre_norm of it -> (x, limbs, mant, e); else (x, None, None, None) with
    the 2^42 bound flag of x."""
    return _run(m, x, _y(m, c, lin, mant, e).contiguous(), None, gamma, 1, gamma is not None)


def pre_norm(m, x, gamma):
    """pre_norm of x -> (limbs, mant, e)."""
    return _run(m, x, None, None, gamma, 2, True)[1:]


def qkv(m, c, lin, mant, e, pos, slot, cache, int32=False):
    """qkv linear output -> q int64 [N, HKV, G, HD]; K / V of the tokens are stored at slot in cache. int32=True: q as
    int32 (the same values, |q| within three limbs), the type the attention kernels read: saves their conversion."""
    y = _y(m, c, lin, mant, e).contiguous()
    N = pos.shape[0]
    H, HKV, HD = m.H, m.HKV, m.HD
    q = torch.empty(N, HKV, H // HKV, HD, dtype=torch.int32 if int32 else torch.long, device=m.dev)
    st, bs = (cache.stride()[:3], cache.shape[2]) if cache is not None else ((0, 0, 0), 1)
    rc = nv.lib().bx_int8_qkv(y.data_ptr(), m.cos.data_ptr(), m.sin.data_ptr(), pos.long().contiguous().data_ptr(),
                              nv.ptr(slot.long().contiguous() if slot is not None else None), nv.ptr(cache), *st, bs,
                              None if int32 else q.data_ptr(), q.data_ptr() if int32 else None, m.fl.data_ptr(), N, H,
                              HKV, HD, nv.stream())
    nv.check(rc, "bx_int8_qkv")
    return q


def attn_out(m, num, den):
    """num [N, HKV, G, HD], den [N, HKV, G, 1] -> (limbs, mant, e) of pre_plain(rdiv(num << 2, den))."""
    N = num.shape[0]
    K2 = num.shape[1] * num.shape[2] * num.shape[3]
    q = torch.empty(2 * N, K2, dtype=torch.int8, device=m.dev)
    mant = torch.empty(N, dtype=torch.long, device=m.dev)
    e = torch.empty(N, dtype=torch.long, device=m.dev)
    rc = nv.lib().bx_int8_attn_out(num.contiguous().data_ptr(), den.contiguous().data_ptr(), q.data_ptr(),
                                   mant.data_ptr(), e.data_ptr(), N, K2, num.shape[3], nv.stream())
    nv.check(rc, "bx_int8_attn_out")
    return q, mant, e


def silu_quant(m, c, lin, mant, e, lut, scr=None):
    """gate_up linear output -> (limbs, mant', e', flag) of silu_mul (table SiLU, h = rsh(sg u, 16), 2-limb rows).
    scr int64 [2] (zeroed): the maxima of |sg|, |u| go there (atomic maxima) and flag is None; without scr the
    product-bound flag is returned as a 0-d bool tensor."""
    y = _y(m, c, lin, mant, e).contiguous()
    N, FF = y.shape[0], y.shape[1] // 2
    q = torch.empty(2 * N, FF, dtype=torch.int8, device=m.dev)
    mant2 = torch.empty(N, dtype=torch.long, device=m.dev)
    e2 = torch.empty(N, dtype=torch.long, device=m.dev)
    own = scr is None
    if own:
        scr = torch.zeros(2, dtype=torch.long, device=m.dev)
    rc = nv.lib().bx_int8_silu_quant(y.data_ptr(), lut.data_ptr(), q.data_ptr(), mant2.data_ptr(), e2.data_ptr(),
                                     scr.data_ptr(), N, FF, nv.stream())
    nv.check(rc, "bx_int8_silu_quant")
    return q, mant2, e2, ((scr[0] * scr[1] >= 1 << 62) if own else None)


def scratch(m):
    """The model's per-layer maxima buffer int64 [L, 2] (created on first use, like the reference's `m._scr`)."""
    if getattr(m, "scr", None) is None:
        m.scr = torch.zeros(m.L, 2, dtype=torch.long, device=m.dev)
    return m.scr


def mlp_mid(m, ly, c, mant, e, layer):
    """`tri_mlp.silu_quant` on the raw gate / up GEMM output c of layer `layer`, the product-bound maxima into the
    model's scratch row -> (limbs, mant, e) (src/bitexact/vllm_plugin/tri_fuse.py:243-245). ly["wgu"] = (w, m, fmsh)."""
    from . import tri_mlp
    return tri_mlp.silu_quant(c, ly["wgu"][1], ly["wgu"][2], mant, e, m.silu_t, False, scr=scratch(m)[layer])[:3]


def flag_end(m, scr=None):
    """Multiply the per-layer maxima collected in the model's scratch (or the given scr [L, 2]) into the bound flag
    m.fl and clear them (src/bitexact/vllm_plugin/tri_fuse.py:248-265: `flag_end(m)`)."""
    scr = scratch(m) if scr is None else scr
    nv.check(nv.lib().bx_int8_flag_end(scr.data_ptr(), m.fl.data_ptr(), scr.shape[0], nv.stream()), "bx_int8_flag_end")
