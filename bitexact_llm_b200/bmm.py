"""Exact batched integer product: drop-in for `bitexact.bmm.bmm` (src/bitexact/bmm.py:78-102)."""

import torch

from . import _native as nv


def bmm(a, b, na=3, nb=3, path="tensor", tile_rows=0):
    """Exact a @ b for [Z, M, K] x [Z, K, N] integer CUDA tensors (int32 or int64, any strides, operands of at most
    na / nb <= 3 signed base-256 limbs: |x| <= 8355711) -> int64 [Z, M, N].

    path "tensor" (default): both operands are packed into int8 limb planes and multiplied on the tcgen05 int8 tensor
    pipe, five int32 accumulators (one per limb weight) joined to int64 at the end, the reference's own scheme
    (src/bitexact/bmm.py:27-75). path "cuda": a CUDA-core int64 tile kernel (no scratch memory). Both give the same
    integers; na and nb are accepted for the reference's signature (all three limbs are always multiplied)."""
    Z, M, K = a.shape
    assert b.shape[0] == Z and b.shape[1] == K and K < 43690 and a.is_cuda and b.is_cuda
    assert a.dtype in (torch.int32, torch.int64) and b.dtype in (torch.int32, torch.int64)
    assert path in ("tensor", "cuda")
    N = b.shape[2]
    c = torch.empty((Z, M, N), dtype=torch.long, device=a.device)
    lib = nv.lib()
    if path == "tensor":
        scratch = torch.empty(max(16, lib.bx_bmm_limb_scratch_bytes(Z, M, N, K)), dtype=torch.int8, device=a.device)
        rc = lib.bx_bmm_limb(a.data_ptr(), int(a.dtype == torch.int64), b.data_ptr(), int(b.dtype == torch.int64),
                             c.data_ptr(), Z, M, N, K, a.stride(0), a.stride(1), a.stride(2), b.stride(0),
                             b.stride(1), b.stride(2), scratch.data_ptr(), tile_rows, nv.stream())
        nv.check(rc, "bx_bmm_limb")
        return c
    for z0 in range(0, Z, 65535):
        z1 = min(Z, z0 + 65535)
        az, bz, cz = a[z0:z1], b[z0:z1], c[z0:z1]
        rc = lib.bx_bmm(az.data_ptr(), int(a.dtype == torch.int64), bz.data_ptr(), int(b.dtype == torch.int64),
                        cz.data_ptr(), z1 - z0, M, N, K, a.stride(0), a.stride(1), a.stride(2), b.stride(0),
                        b.stride(1), b.stride(2), nv.stream())
        nv.check(rc, "bx_bmm")
    return c
