"""`lin_y` of the reference's stage set (src/bitexact/exact/segs.py:25-32): the epilogue of a linear whose dense
product and residual were computed separately (`exact.model.Lin.__call__`)."""

import torch

from .. import _native as nv
from .wmm import epilogue


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
