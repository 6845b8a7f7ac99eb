"""int8-mode GEMM: drop-in for `bitexact.int8.gemm_skinny.int_mm` (src/bitexact/int8/gemm_skinny.py:80-97) and a
fused variant with the `post` epilogue (src/bitexact/int8/segs.py:62-67), both on the tcgen05 limb GEMM."""

import torch

from .. import _native as nv


def int_mm(a, w, M=None):
    """a int8 [R, K] (two activation limbs stacked along rows by stack_limbs, limb i of row m at row i M + m; rows
    beyond 2 M are padding), w int8 [N, K], both contiguous -> int32 [R, N] like torch._int_mm(a, w.t()).
    M defaults to R // 2 (no padding rows)."""
    R, K = a.shape
    N = w.shape[0]
    assert a.dtype == torch.int8 and w.dtype == torch.int8 and a.is_contiguous() and w.is_contiguous()
    M = R // 2 if M is None else M
    c = torch.empty(R, N, dtype=torch.int32, device=a.device)
    if R > 2 * M:
        c[2 * M:].zero_()                                    # products of the zero padding rows
    nv.check(nv.lib().bx_int8_mm(a.data_ptr(), w.data_ptr(), c.data_ptr(), M, N, K, 0, nv.stream()), "bx_int8_mm")
    return c


def linear_post(a, w, m, fmsh, mant, e, flag, check=True, M=None):
    """post(join_limbs(int_mm(a, w)), m, fmsh, mant, e) in one kernel: int64 [M, N] at 16 fractional bits.
    m int64 [N], fmsh int, mant / e int64 [M]; flag int32 [1] is set when check and some |t| >= 2^38."""
    R, K = a.shape
    N = w.shape[0]
    M = mant.shape[0] if M is None else M
    assert a.dtype == torch.int8 and w.dtype == torch.int8 and a.is_contiguous() and w.is_contiguous() and R >= 2 * M
    y = torch.empty(M, N, dtype=torch.long, device=a.device)
    rc = nv.lib().bx_int8_linear_post(a.data_ptr(), w.data_ptr(), m.data_ptr(), int(fmsh), mant.contiguous().data_ptr(),
                                      e.contiguous().data_ptr(), y.data_ptr(), flag.data_ptr(), M, N, K,
                                      int(bool(check)), 0, nv.stream())
    nv.check(rc, "bx_int8_linear_post")
    return y
