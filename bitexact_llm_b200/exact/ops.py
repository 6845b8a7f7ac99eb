"""Integer rules of exact mode as device functions with the reference's names (src/bitexact/exact/ops.py): the
pieces the serving path fuses, callable one by one. Every function takes and returns CUDA tensors and launches one
kernel of libbitexact_b200 (two for `quant`)."""

import torch

from .. import _native as nv

FR, FT, FN, FT2, FZ, QB = 24, 30, 40, 26, 26, 22
L2E28, L2E30 = 387270501, 1549082005
L2E28_HD = {64: L2E28, 128: 273841598}


def rms(x):
    """sqrt(mean(x^2) + 1e-5) of each row of x (int64 [M, D] at 24 bits, D a power of two <= 4096) as (r, er):
    r 2^er with 2^30 <= r < 2^31 (ops.py:92-105)."""
    M, D = x.shape
    x = x.contiguous()
    r = torch.empty(M, dtype=torch.long, device=x.device)
    er = torch.empty(M, dtype=torch.long, device=x.device)
    nv.check(nv.lib().bx_exact_rms(x.data_ptr(), r.data_ptr(), er.data_ptr(), None, M, D, nv.stream()), "bx_exact_rms")
    return r, er


def quant(P, eps):
    """Per-row power-of-two quantisation of the values P 2^eps (P int64 [..., K], eps an int <= 0): q int64 with
    |q| <= 2^22 and sh [...] (ops.py:82-89)."""
    assert isinstance(eps, int) and -62 <= eps <= 0
    shape = P.shape
    P2 = P.reshape(-1, shape[-1]).contiguous()
    M, K = P2.shape
    lib, st = nv.lib(), nv.stream()
    rowmax = torch.empty(M, dtype=torch.long, device=P.device)
    q = torch.empty(M, K, dtype=torch.int32, device=P.device)
    sh = torch.empty(M, dtype=torch.long, device=P.device)
    if M:
        nv.check(lib.bx_rowmax_abs(P2.data_ptr(), rowmax.data_ptr(), M, K, st), "bx_rowmax_abs")
        nv.check(lib.bx_exact_quant_rows(P2.data_ptr(), rowmax.data_ptr(), -eps, q.data_ptr(), K, sh.data_ptr(), None, 0,
                                         M, K, st), "bx_exact_quant_rows")
    return q.long().view(shape), sh.view(shape[:-1])


def softmax_w(raw, ok, sh, kbits, lut, fp, l2e=None):
    """Attention weights at 22 bits from exact scores raw int64 [..., S] (value raw 2^(sh - 17 - 3), sh [..., 1]);
    ok marks the visible keys. Returns p int64 (0 where masked) and the row sums [..., 1] (ops.py:133-143)."""
    assert kbits == 17 and fp == 22
    shape = raw.shape
    S = shape[-1]
    raw2 = raw.reshape(-1, S).contiguous()
    R = raw2.shape[0]
    okb = torch.broadcast_to(ok, shape).reshape(R, S).to(torch.uint8).contiguous()
    sh2 = torch.broadcast_to(sh, shape[:-1] + (1,)).reshape(R).contiguous()
    p = torch.empty(R, S, dtype=torch.int32, device=raw.device)
    den = torch.empty(R, dtype=torch.long, device=raw.device)
    rc = nv.lib().bx_softmax_w(raw2.data_ptr(), okb.data_ptr(), None, sh2.data_ptr(), lut.data_ptr(),
                               int(L2E28 if l2e is None else l2e), None, p.data_ptr(), den.data_ptr(), R, S, nv.stream())
    nv.check(rc, "bx_softmax_w")
    return p.long().view(shape), den.view(shape[:-1] + (1,))


def silu_mul(g, u, lut):
    """silu(g) u for g, u int64 [N, FF] at 24 bits -> (P, eps, ok): value P 2^eps; ok is False when the product bound
    of the reference was violated somewhere (ops.py:119-130)."""
    N, FF = g.shape
    y = torch.cat([g, u], 1).contiguous()
    P = torch.empty(N, FF, dtype=torch.long, device=g.device)
    rmax = torch.empty(N, dtype=torch.long, device=g.device)
    flag = torch.zeros(1, dtype=torch.int32, device=g.device)
    nv.check(nv.lib().bx_exact_silu_prod(y.data_ptr(), lut.data_ptr(), P.data_ptr(), rmax.data_ptr(), flag.data_ptr(), N,
                                         FF, nv.stream()), "bx_exact_silu_prod")
    return P, -2 * FR, flag[0] == 0
