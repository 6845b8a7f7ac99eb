"""Exact batched integer product: drop-in for `bitexact.bmm.bmm` (src/bitexact/bmm.py:78-102)."""

import torch

from . import _native as nv


def bmm(a, b, na=3, nb=3):
    """Exact a @ b for [Z, M, K] x [Z, K, N] integer CUDA tensors (int32 or int64, any strides, operands of at most
    na / nb limbs) -> int64 [Z, M, N]. na and nb are accepted for the reference's signature; the kernel multiplies
    the integers themselves, which is the same number."""
    Z, M, K = a.shape
    assert b.shape[0] == Z and b.shape[1] == K and K < 43690 and a.is_cuda and b.is_cuda
    assert a.dtype in (torch.int32, torch.int64) and b.dtype in (torch.int32, torch.int64)
    N = b.shape[2]
    c = torch.empty((Z, M, N), dtype=torch.long, device=a.device)
    for z0 in range(0, Z, 65535):
        z1 = min(Z, z0 + 65535)
        az, bz, cz = a[z0:z1], b[z0:z1], c[z0:z1]
        rc = nv.lib().bx_bmm(az.data_ptr(), int(a.dtype == torch.int64), bz.data_ptr(), int(b.dtype == torch.int64),
                             cz.data_ptr(), z1 - z0, M, N, K, a.stride(0), a.stride(1), a.stride(2), b.stride(0),
                             b.stride(1), b.stride(2), nv.stream())
        nv.check(rc, "bx_bmm")
    return c
