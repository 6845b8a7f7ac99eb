"""int8-mode GEMM (raw limb products and fused post epilogue) on the GPU against the golden vectors of the
reference's CPU path and against the oracle. Modelled on the reference's tests/test_gemm_skinny.py and
tests/test_gemm_sm90.py (adversarial all-extreme rows, padded row counts)."""

import os

import numpy as np
import pytest
import torch

from oracle import int8 as o8

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def T(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_golden_int8_linear_raw_and_fused():
    from bitexact_llm_b200.int8.gemm_skinny import int_mm, linear_post
    z = np.load(os.path.join(GOLD, "int8_ops.npz"))
    M = z["q"].shape[0]
    a, w = T(z["stacked"]), T(z["wq"])
    c = int_mm(a, w, M=M).cpu().numpy().astype(np.int64)
    assert np.array_equal(c[:M] + (c[M:2 * M] << 8), z["acc"]) and not c[2 * M:].any()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    fmsh = int(z["fm"]) + 8 - 24
    y = linear_post(a, w, T(z["m"]), fmsh, T(z["mant"]), T(z["e"]), flag)
    assert np.array_equal(y.cpu().numpy(), z["y"]) and bool(flag.item()) == bool(z["flag"])


@pytest.mark.parametrize("M,N,K", [(1, 256, 2048), (24, 3072, 2048), (100, 512, 8192), (300, 1024, 2048), (129, 200, 272)])
def test_seeded_int8_shapes(M, N, K):
    from bitexact_llm_b200 import _native as nv
    from bitexact_llm_b200.int8.gemm_skinny import int_mm, linear_post
    rng = np.random.RandomState(M + N)
    w = rng.randint(-127, 128, (N, K)).astype(np.int8)
    w[0] = 127
    q = rng.randint(-32512, 32513, (M, K)).astype(np.int64)
    q[0] = 32512
    m = rng.randint(1, 1 << 24, N).astype(np.int64)
    mant = rng.randint(1 << 23, (1 << 24) + 1, M).astype(np.int64)
    e = rng.randint(-30, -5, M).astype(np.int64)
    fmsh = 20 if M != 24 else 17                             # 17: some |t| reach 2^38 (flag case)
    acc = o8.imm(q, w)
    want, wflag = o8.post(acc, m, fmsh, mant, e)
    a = T(o8.stack_limbs(q, 2))
    c = int_mm(a, T(w), M=M).cpu().numpy().astype(np.int64)
    assert np.array_equal(c[:M] + (c[M:2 * M] << 8), acc)
    lib = nv.lib()
    wd, md, mantd, ed = T(w), T(m), T(mant), T(e)              # keep the device buffers alive across the calls
    # negative: the persistent kernel; 200 + rows (10000 S + 200 + rows): K split over clusters of up to 8 (of S) CTAs
    for tile in (0, 16, 32, 64, 128, -16, -32, -64, -128, 216, 232, 264, 20216, 20264, 40232, 80264):
        flag = torch.zeros(1, dtype=torch.int32, device="cuda")
        y = torch.empty(M, N, dtype=torch.long, device="cuda")
        rc = lib.bx_int8_linear_post(a.data_ptr(), wd.data_ptr(), md.data_ptr(), fmsh, mantd.data_ptr(),
                                     ed.data_ptr(), y.data_ptr(), flag.data_ptr(), M, N, K, 1, tile, nv.stream())
        torch.cuda.synchronize()
        assert rc == 0 and np.array_equal(y.cpu().numpy(), want), (tile, int((y.cpu().numpy() != want).sum()))
        assert bool(flag.item()) == wflag
    assert nv.device_status() == 0


def test_post_shift_regimes():
    """The fused post epilogue takes two plain rounding shifts when both shifts lie in 1 .. 62 and the general rule
    otherwise: row exponents and layer shifts on both sides of every boundary (shift 0, negative = left shift, 62, 63,
    beyond 63), on the tile, persistent and split-K kernels."""
    from bitexact_llm_b200 import _native as nv
    rng = np.random.RandomState(8)
    M, N, K = 96, 256, 512
    w = rng.randint(-127, 128, (N, K)).astype(np.int8)
    q = rng.randint(-32512, 32513, (M, K)).astype(np.int64)
    m = rng.randint(1, 1 << 12, N).astype(np.int64)
    mant = rng.randint(1 << 3, 1 << 6, M).astype(np.int64)
    e = np.array([8, 7, 9, 20, -54, -55, -56, -70, -12, 0][:10] * 10)[:M].astype(np.int64)     # shifts 0, 1, -1, -12, 62, 63, 64, 78 ...
    acc = o8.imm(q, w)
    a = T(o8.stack_limbs(q, 2))
    lib = nv.lib()
    wd, md, mantd, ed = T(w), T(m), T(mant), T(e)
    for fmsh in (20, 1, 0, -2, 62, 63):
        want, wflag = o8.post(acc, m, fmsh, mant, e)
        for tile in (0, 32, -32, 216, 20232):
            flag = torch.zeros(1, dtype=torch.int32, device="cuda")
            y = torch.empty(M, N, dtype=torch.long, device="cuda")
            rc = lib.bx_int8_linear_post(a.data_ptr(), wd.data_ptr(), md.data_ptr(), fmsh, mantd.data_ptr(),
                                         ed.data_ptr(), y.data_ptr(), flag.data_ptr(), M, N, K, 1, tile, nv.stream())
            torch.cuda.synchronize()
            assert rc == 0 and np.array_equal(y.cpu().numpy(), want), (fmsh, tile, int((y.cpu().numpy() != want).sum()))
            assert bool(flag.item()) == wflag, (fmsh, tile)
