"""The element-wise stages of the exact engine between its matrix products, with the reference's names and
signatures (src/bitexact/exact/segs.py:25-192): each stage is one kernel of libbitexact_b200. The serving path runs
the fused forms (`vllm_plugin.exact_fuse`); these are the same integers stage by stage, for code written against
`bitexact.exact.segs` (the standalone engine `ExactLlama._layer`, src/bitexact/exact/model.py:106-125).

`err` is the reference's sticky bool tensor; `flag` results are bool tensors."""

import torch

from .. import _native as nv
from . import ops
from .wmm import epilogue

FR, FT = 24, 30
FK, FV, FP = 17, 19, 22
LIM3 = 8355711


def lin_y(C, rs, d, g, sh, checked=False):
    """C int64 [M, N] (or [split, M, N]), rs = (B,) dense residual or (q, ec, ev) ELL lists, d, g int64 [N],
    sh int64 [M] -> y int64 [M, N], and the flag when `checked`."""
    T = C.sum(0) if C.dim() == 3 else C
    if len(rs) == 1:
        return epilogue(T, rs[0], d, g, sh, 24, checked)
    q, ec, ev = rs
    M, N = T.shape
    R = ec.shape[1]
    if R == 0:
        return epilogue(T, None, d, g, sh, 24, checked)
    y = torch.empty((M, N), dtype=torch.long, device=T.device)
    flag = torch.zeros(1, dtype=torch.int32, device=T.device)
    if M:
        q32 = q.to(torch.int32).contiguous()
        cnt = torch.full((N,), R, dtype=torch.int32, device=T.device)       # padded lists: zero values add nothing
        rc = nv.lib().bx_exact_epilogue(T.contiguous().data_ptr(), None, q32.data_ptr(), q32.stride(0), cnt.data_ptr(),
                                        ec.to(torch.int32).contiguous().data_ptr(), ev.contiguous().data_ptr(), R,
                                        d.contiguous().data_ptr(), g.contiguous().data_ptr(),
                                        sh.contiguous().data_ptr(), y.data_ptr(), flag.data_ptr(), M, N,
                                        int(bool(checked)), nv.stream())
        nv.check(rc, "bx_exact_epilogue")
    return (y, flag[0] != 0) if checked else y


def lin_add(C, rs, d, g, sh, x):
    y, flag = lin_y(C, rs, d, g, sh, checked=True)
    return x + y.view(x.shape), flag


def add_y(y, x):
    return x + y.view(x.shape)


def rms(x, err):
    r, er = ops.rms(x)
    return r, er, err | (x.abs().amax() >= 1 << 40)


def ndiv(x, gm, ge, r, er):
    """x gamma / rms at 40 bits (one rounding per element)."""
    M, D = x.shape
    P = torch.empty(M, D, dtype=torch.long, device=x.device)
    rc = nv.lib().bx_exact_ndiv(x.contiguous().data_ptr(), gm.contiguous().data_ptr(), ge.contiguous().data_ptr(),
                                r.contiguous().data_ptr(), er.contiguous().data_ptr(), P.data_ptr(), M, D, nv.stream())
    nv.check(rc, "bx_exact_ndiv")
    return P


def quant(P, eps):
    q, sh = ops.quant(P, eps)
    return q.to(torch.int32), sh


def norm_quant(x, gm, ge, err):
    """rms + ndiv + quant in one kernel (what Segs.norm_q runs as three stages)."""
    M, D = x.shape
    q = torch.empty(M, D, dtype=torch.int32, device=x.device)
    sh = torch.empty(M, dtype=torch.long, device=x.device)
    flag = torch.zeros(1, dtype=torch.int32, device=x.device)
    rc = nv.lib().bx_exact_norm(2, x.contiguous().data_ptr(), None, None, gm.contiguous().data_ptr(),
                                ge.contiguous().data_ptr(), None, q.data_ptr(), sh.data_ptr(), None, flag.data_ptr(), M, D,
                                1, nv.stream())
    nv.check(rc, "bx_exact_norm")
    return q, sh, err | (flag[0] != 0)


def rope_y(y, pos, cos, sin, B, T, dm):
    """The qkv linear's output y [B T, (H + 2 HKV) HD] at 24 bits -> q at 54 bits [B, T, H, HD], k at 17 bits,
    v at 19 bits [B, T, HKV, HD], and y (for the bound check)."""
    h, hkv, hd = dm
    N = B * T
    y2 = y.reshape(N, -1).contiguous()
    Pq = torch.empty(B, T, h, hd, dtype=torch.long, device=y.device)
    k = torch.empty(B, T, hkv, hd, dtype=torch.long, device=y.device)
    v = torch.empty(B, T, hkv, hd, dtype=torch.long, device=y.device)
    rc = nv.lib().bx_exact_rope(y2.data_ptr(), cos.contiguous().data_ptr(), sin.contiguous().data_ptr(),
                                pos.reshape(N).long().contiguous().data_ptr(), Pq.data_ptr(), k.data_ptr(), v.data_ptr(),
                                N, h, hkv, hd, nv.stream())
    nv.check(rc, "bx_exact_rope")
    return Pq, k, v, y.view(B, T, -1)


def lin_rope(C, rs, d, g, sh, pos, cos, sin, B, T, dm):
    return rope_y(lin_y(C, rs, d, g, sh), pos, cos, sin, B, T, dm)


def q_group(Pq, k, v, y, err):
    """Quantise q per (token, head) and group by KV head: [B HKV, g T, HD] int32 and exponents [.., 1]."""
    B, T, h, hd = Pq.shape
    hkv = k.shape[2]
    qi, shq = ops.quant(Pq, -(FR + FT))
    g = h // hkv
    qg = qi.view(B, T, hkv, g, hd).permute(0, 2, 3, 1, 4).reshape(B * hkv, g * T, hd).to(torch.int32)
    shg = shq.view(B, T, hkv, g).permute(0, 2, 3, 1).reshape(B * hkv, g * T, 1)
    err = err | (y.abs().amax() >= 1 << 31) | (k.abs().amax() > LIM3) | (v.abs().amax() > LIM3) \
        | (shq.amax() > FK + 3 - ops.FZ)
    return qg, shg, err


def softmax(raw, qpos, shg, lut, l2e):
    """raw int64 [Z, gT, S] exact scores, qpos [Z, gT, 1] (key s visible iff s <= qpos), shg [Z, gT, 1] ->
    p int32 [Z, gT, S], den int64 [Z, gT, 1]."""
    Z, gT, S = raw.shape
    R = Z * gT
    raw2 = raw.reshape(R, S).contiguous()
    p = torch.empty(R, S, dtype=torch.int32, device=raw.device)
    den = torch.empty(R, dtype=torch.long, device=raw.device)
    rc = nv.lib().bx_softmax_w(raw2.data_ptr(), None, torch.broadcast_to(qpos, (Z, gT, 1)).reshape(R).long().contiguous()
                               .data_ptr(), shg.reshape(R).contiguous().data_ptr(), lut.data_ptr(), int(l2e), None,
                               p.data_ptr(), den.data_ptr(), R, S, nv.stream())
    nv.check(rc, "bx_softmax_w")
    return p.view(Z, gT, S), den.view(Z, gT, 1)


def attn_div(num, den, T, hkv):
    """num [B HKV, g T, HD] at 41 bits, den [B HKV, g T, 1] -> o at 24 bits [B T, H HD] (one rounding)."""
    Z, gT, hd = num.shape
    B, g = Z // hkv, gT // T
    o = torch.empty(Z * gT, hd, dtype=torch.long, device=num.device)
    rc = nv.lib().bx_exact_attn_div(num.contiguous().data_ptr(), den.contiguous().data_ptr(), o.data_ptr(), Z * gT, hd,
                                    nv.stream())
    nv.check(rc, "bx_exact_attn_div")
    return o.view(B, hkv, g, T, hd).permute(0, 3, 1, 2, 4).reshape(B * T, hkv * g * hd)


def silu_y(gu, lut):
    ff = gu.shape[1] // 2
    P, _, ok = ops.silu_mul(gu[:, :ff], gu[:, ff:], lut)
    return P, ok


def lin_silu(C, rs, d, g, sh, lut):
    return silu_y(lin_y(C, rs, d, g, sh), lut)


def quant_silu(P, ok, err):
    q, sh = ops.quant(P, -2 * FR)
    return q.to(torch.int32), sh, err | ~ok


STAGES = ("lin_y", "lin_add", "rms", "ndiv", "quant", "lin_rope", "q_group", "softmax", "attn_div",
          "lin_silu", "quant_silu", "rope_y", "add_y", "silu_y", "norm_quant")


class Segs:
    """The stage set bound to a geometry dm = (H, HKV, HD), as `bitexact.exact.segs.Segs`
    (src/bitexact/exact/segs.py:134-192). `compiled` is accepted and ignored: the stages are kernels already."""

    def __init__(self, compiled=False, dm=(32, 8, 64), one_region=False):
        self.dm = dm
        self.one_region = one_region
        self.l2e = ops.L2E28_HD[dm[2]]                           # KeyError: unsupported head_dim
        self.s = type("S", (), {n: staticmethod(globals()[n]) for n in STAGES})

    def norm_q(self, x, gm, ge, err):
        if self.one_region:
            return self.s.norm_quant(x, gm, ge, err)
        r, er, err = self.s.rms(x, err)
        q, sh = self.s.quant(self.s.ndiv(x, gm, ge, r, er), -ops.FN)
        return q, sh, err

    def pre_norm(self, x, gm, ge):
        return self.norm_q(x, gm, ge, torch.zeros((), dtype=torch.bool, device=x.device))[:2]

    def lin_out(self, C, rs, d, g, sh):
        return self.s.lin_y(C, rs, d, g, sh, True)

    def add_norm(self, C, rs, d, g, sh, x, gm, ge, err):
        x, flag = self.s.lin_add(C, rs, d, g, sh, x)
        q, s, err = self.norm_q(x.view(-1, x.shape[-1]), gm, ge, err | flag)
        return x, q, s, err

    def qkv(self, C, rs, d, g, sh, pos, cos, sin, B, T, err):
        Pq, k, v, y = self.s.lin_rope(C, rs, d, g, sh, pos, cos, sin, B, T, self.dm)
        qg, shg, err = self.s.q_group(Pq, k, v, y, err)
        return qg, shg, k, v, err

    def qkv_y(self, y, pos, cos, sin, B, T, err):
        Pq, k, v, y = self.s.rope_y(y, pos, cos, sin, B, T, self.dm)
        qg, shg, err = self.s.q_group(Pq, k, v, y, err)
        return qg, shg, k, v, err

    def add_norm_y(self, y, x, gm, ge, err):
        x = self.s.add_y(y, x)
        q, s, err = self.norm_q(x.view(-1, x.shape[-1]), gm, ge, err)
        return x, q, s, err

    def gu_silu_y(self, y, lut, err):
        P, ok = self.s.silu_y(y, lut)
        return self.s.quant_silu(P, ok, err)

    def softmax(self, raw, qpos, shg, lut):
        return self.s.softmax(raw, qpos, shg, lut, self.l2e)

    def attn_out(self, num, den, T):
        return self.s.quant(self.s.attn_div(num, den, T, self.dm[1]), -FR)

    def gu_silu(self, C, rs, d, g, sh, lut, err):
        P, ok = self.s.lin_silu(C, rs, d, g, sh, lut)
        return self.s.quant_silu(P, ok, err)
