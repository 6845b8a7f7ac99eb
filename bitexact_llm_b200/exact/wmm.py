"""Unfused pieces of the exact linear: the dense limb product, the sparse residual and the epilogue, with the
reference's names (src/bitexact/exact/wmm.py:31-150). The serving path uses `vllm_plugin.exact_gemm.FusedLin`,
which does all three in one kernel."""

import torch

from .. import _native as nv

_UNIT = {}


def _unit(N, M, dev):
    """d = 0, g = -24 per weight row and sh = 0 per activation row: with these the fused linear returns T itself."""
    key = (N, M, str(dev))
    if key not in _UNIT:
        _UNIT[key] = (torch.zeros(N, dtype=torch.long, device=dev), torch.full((N,), -24, dtype=torch.long, device=dev),
                      torch.zeros(M, dtype=torch.long, device=dev), torch.zeros(1, dtype=torch.int32, device=dev))
    return _UNIT[key]


def wmm(q, limbs, cfg=None, target=None):
    """T = q @ W^T exactly: q int32 / int64 [M, K] (|q| <= 2^22), limbs int8 [3, N, K] -> int64 [M, N]
    (the sum over the reference's split dimension; `cfg` = tile rows, `target` ignored)."""
    M, K = q.shape
    N = limbs.shape[1]
    q32 = q.to(torch.int32).contiguous()
    d, g, sh, flag = _unit(N, M, q.device)
    y = torch.empty((M, N), dtype=torch.long, device=q.device)
    if M == 0:
        return y
    scratch = torch.empty(3 * M * K, dtype=torch.int8, device=q.device)
    rc = nv.lib().bx_exact_linear(q32.data_ptr(), q32.stride(0), sh.data_ptr(), limbs.data_ptr(), d.data_ptr(),
                                  g.data_ptr(), None, None, None, 0, scratch.data_ptr(), y.data_ptr(), flag.data_ptr(),
                                  M, N, K, 0, cfg or 0, nv.stream())
    nv.check(rc, "bx_exact_linear")
    return y


wmm_triton = wmm          # the reference's name of the GPU product


def residual(q, rr, rc, rv, N):
    """B[m, n] = sum over the residual entries (rr = n, rc = column, rv = value) of q[m, rc] * rv
    (exact/wmm.py:124-129)."""
    B = torch.zeros((q.shape[0], N), dtype=torch.long, device=q.device)
    if rr.numel():
        B.index_add_(1, rr, q[:, rc].long() * rv)
    return B


def epilogue(T, B, d, g, sh, fr=24, checked=False):
    """y = round((T 2^d + B) 2^(sh + g - d + 24)) (exact/wmm.py:132-150); with `checked` also the lost-bit /
    range flag as a bool tensor."""
    assert fr == 24
    M, N = T.shape
    y = torch.empty((M, N), dtype=torch.long, device=T.device)
    flag = torch.zeros(1, dtype=torch.int32, device=T.device)
    if M:
        rc = nv.lib().bx_exact_epilogue(T.contiguous().data_ptr(), nv.ptr(B.contiguous() if B is not None else None),
                                        None, 0, None, None, None, 0, d.contiguous().data_ptr(),
                                        g.contiguous().data_ptr(), sh.contiguous().data_ptr(), y.data_ptr(),
                                        flag.data_ptr(), M, N, int(bool(checked)), nv.stream())
        nv.check(rc, "bx_exact_epilogue")
    return (y, flag[0] != 0) if checked else y
