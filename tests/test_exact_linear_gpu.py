"""Exact-mode fused linear on the GPU (through the C ABI) against the CPU oracle and the golden vectors.
Modelled on the reference's tests/test_vllm_exact_gemm.py and tests/test_exact_ops.py:118-134."""

import os

import numpy as np
import pytest
import torch

from oracle import exact as ox

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _lin(dec, dev="cuda"):
    from bitexact_llm_b200.exact.model import Lin
    from bitexact_llm_b200.vllm_plugin.exact_gemm import FusedLin
    return FusedLin(Lin({k: torch.from_numpy(np.ascontiguousarray(v)) for k, v in dec.items()}, None, dev))


def _run(fl, q, sh, checked=True, tile=None):
    fl.cfg = tile
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = fl(torch.from_numpy(q.astype(np.int32)).cuda(), torch.from_numpy(sh.astype(np.int64)).cuda(), flag, checked)
    torch.cuda.synchronize()
    return y.cpu().numpy(), bool(flag.item())


def test_golden_linear_with_residual_and_extreme_shifts():
    from bitexact_llm_b200 import _native as nv
    z = np.load(os.path.join(GOLD, "exact_ops.npz"))
    dec = {k: z["lin_" + k] for k in ("limbs", "g", "d", "rr", "rc", "rv")}
    fl = _lin(dec)
    # negative: the persistent kernel; 200 + rows: split-K over a cluster of CTAs; 400 + rows: CTA pairs (cta_group::2);
    # 500 / 600 + weight rows: activation rows on the MMA M side (CTA pairs / one CTA)
    for tile in (None, 16, 32, 48, 64, 80, -16, -32, -48, 216, 232, 264, 416, 432, 448, 516, 532, 548, 564, 580,
                 616, 632, 648, 664, 680, 764, 20764, 40764, 20264):
        y, flag = _run(fl, z["lin_q"], z["lin_sh"], True, tile)
        assert np.array_equal(y, z["lin_y"]), tile
        assert flag == bool(z["lin_flag"])
    for m in range(len(z["lin_q"])):                      # row-local flag
        y, flag = _run(fl, z["lin_q"][m:m + 1], z["lin_sh"][m:m + 1])
        assert np.array_equal(y, z["lin_y"][m:m + 1]) and flag == bool(z["lin_rowflag"][m]), m
    y, flag = _run(fl, z["lin_q"], z["lin_sh"], False)
    assert not flag                                          # unchecked calls never touch the flag
    assert nv.device_status() == 0


@pytest.mark.parametrize("M,N,K", [(1, 256, 2048), (7, 3072, 2048), (37, 512, 8192), (300, 1024, 2048),
                                   (17, 200, 272), (81, 136, 128), (64, 2048, 8192), (5, 130, 1040)])
def test_seeded_shapes_against_oracle(M, N, K):
    rng = np.random.RandomState(M * 1000 + N)
    W = rng.randint(-8355711, 8355712, (N, K)).astype(np.int64)
    W[0, :] = 8355711                                        # adversarial: all extremes
    q = rng.randint(-(1 << 22), (1 << 22) + 1, (M, K)).astype(np.int64)
    q[0, :] = 1 << 22
    limbs = np.stack([l.astype(np.int8) for l in ox.split_limbs(W, 3)[0]])
    nres = max(1, N // 16)
    rr = np.sort(rng.randint(0, N, nres))
    dec = {"limbs": limbs, "g": rng.randint(-34, -24, N).astype(np.int64), "d": rng.randint(0, 31, N).astype(np.int64),
           "rr": rr.astype(np.int64), "rc": rng.randint(0, K, nres).astype(np.int64),
           "rv": rng.randint(-(1 << 20), 1 << 20, nres).astype(np.int64)}
    sh = rng.randint(-45, -8, M).astype(np.int64)
    want, wflag = ox.linear(q, sh, dec, checked=True)
    fl = _lin(dec)
    for tile in (None, 16, 80, -48, 216, 232, 264, 416, 432, 448, 648, 680, 764, 40764) if M > 16 else \
            (None, 64, -16, 216, 264, 416, 448, 516, 548, 580, 616, 664, 764):
        y, flag = _run(fl, q, sh, True, tile)
        assert np.array_equal(y, want), (tile, int((y != want).sum()))
        assert flag == wflag


def test_persistent_kernel_many_tiles_per_cta():
    """More tiles than SMs: every CTA of the persistent kernel walks several tiles through both TMEM buffers."""
    rng = np.random.RandomState(77)
    M, N, K = 100, 20480, 256
    W = rng.randint(-8355711, 8355712, (N, K)).astype(np.int64)
    q = rng.randint(-(1 << 22), (1 << 22) + 1, (M, K)).astype(np.int64)
    dec = {"limbs": np.stack([l.astype(np.int8) for l in ox.split_limbs(W, 3)[0]]),
           "g": rng.randint(-34, -24, N).astype(np.int64), "d": rng.randint(0, 31, N).astype(np.int64),
           "rr": np.arange(0, N, 97, dtype=np.int64), "rc": rng.randint(0, K, len(range(0, N, 97))).astype(np.int64),
           "rv": rng.randint(-(1 << 20), 1 << 20, len(range(0, N, 97))).astype(np.int64)}
    sh = rng.randint(-45, -8, M).astype(np.int64)
    want, wflag = ox.linear(q, sh, dec, checked=True)
    fl = _lin(dec)
    for tile in (-16, -32, -48, None, 416, 432, 448, 532, 548, 564, 580, 632, 648, 664, 680):
        y, flag = _run(fl, q, sh, True, tile)
        assert np.array_equal(y, want), (tile, int((y != want).sum()))
        assert flag == wflag


def test_rounding_rule_boundaries_of_the_short_form():
    """The epilogue takes a short form of the rounding rule when a whole warp shifts right by 1 .. 31 bits with
    k >= d and moderate T, B, and the two-word rule otherwise: shifts on both sides of every boundary (k = d, k = d - 1,
    k = 0, 1, 31, 32), residual terms below and above 2^60, extreme T; warps with all rows alike and mixed warps."""
    rng = np.random.RandomState(11)
    M, N, K = 70, 512, 384
    W = rng.randint(-8355711, 8355712, (N, K)).astype(np.int64)
    W[5, :] = 8355711
    W[6, :] = -8355711
    q = rng.randint(-(1 << 22), (1 << 22) + 1, (M, K)).astype(np.int64)
    q[3, :] = 1 << 22
    q[4, :] = -(1 << 22)
    limbs = np.stack([l.astype(np.int8) for l in ox.split_limbs(W, 3)[0]])
    n = np.arange(N)
    d = np.where(n < 256, n % 31, (n // 32) % 31).astype(np.int64)     # rows 256..: one d per warp
    for s0, off in ((-10, 0), (-25, 2), (-39, 14), (-41, -6)):
        e = -((n // 32) % 4) * 3 - off
        g = (-24 - s0 + e).astype(np.int64)                            # k - d = (s0 - sh) - e
        sh = (s0 + (np.arange(M) % 7) - 3).astype(np.int64)            # k - d in -3 .. 3 (+ 0, 3, 6, 9 by warp, + off)
        rr = np.arange(0, N, 9, dtype=np.int64)
        rv = rng.randint(-(1 << 20), 1 << 20, len(rr)).astype(np.int64)
        rv[::4] = (1 << 37) + 12345                                    # |B| up to 2^59
        rv[1::8] = -(1 << 40)                                          # |B| up to 2^62: outside the short form
        dec = {"limbs": limbs, "g": g, "d": d, "rr": rr, "rc": rng.randint(0, K, len(rr)).astype(np.int64), "rv": rv}
        want, wflag = ox.linear(q, sh, dec, checked=True)
        fl = _lin(dec)
        for tile in (None, 16, 32, 48, 64, 80, -48, 216, 448, 548, 648, 664, 680, 764):
            y, flag = _run(fl, q, sh, True, tile)
            assert np.array_equal(y, want), (s0, tile, int((y != want).sum()))
            assert flag == wflag, (s0, tile)


def test_long_tile_lists_at_128_rows_and_more():
    """Long tile lists of batches of 128 rows and more (several rounds of the persistent activation-major kernel, an
    under-filled last round, a ragged last tile): the automatic choice, the activation-major kernel and the
    weight-major persistent kernel give the oracle's integers."""
    rng = np.random.RandomState(31)
    for M, N, K in ((130, 10247, 1024), (256, 9480, 512), (128, 10240, 384)):
        W = rng.randint(-8355711, 8355712, (N, K)).astype(np.int64)
        q = rng.randint(-(1 << 22), (1 << 22) + 1, (M, K)).astype(np.int64)
        nres = N // 16
        dec = {"limbs": np.stack([l.astype(np.int8) for l in ox.split_limbs(W, 3)[0]]),
               "g": rng.randint(-34, -24, N).astype(np.int64), "d": rng.randint(0, 31, N).astype(np.int64),
               "rr": np.sort(rng.randint(0, N, nres)).astype(np.int64), "rc": rng.randint(0, K, nres).astype(np.int64),
               "rv": rng.randint(-(1 << 20), 1 << 20, nres).astype(np.int64)}
        sh = rng.randint(-30, -8, M).astype(np.int64)
        want, wflag = ox.linear(q, sh, dec, checked=True)
        fl = _lin(dec)
        for tile in (None, 664, -48):
            y, flag = _run(fl, q, sh, True, tile)
            assert np.array_equal(y, want), (M, N, K, tile, int((y != want).sum()))
            assert flag == wflag


def test_long_residual_lists_on_every_kernel_family():
    """Weight rows with 1 .. 6 residual entries (the kernels keep the first one or two in registers and read the rest
    from the ELL arrays), whole warps of listed rows and warps without any, on every kernel family."""
    rng = np.random.RandomState(21)
    M, N, K = 150, 640, 8192
    W = rng.randint(-8355711, 8355712, (N, K)).astype(np.int64)
    q = rng.randint(-(1 << 22), (1 << 22) + 1, (M, K)).astype(np.int64)
    limbs = np.stack([l.astype(np.int8) for l in ox.split_limbs(W, 3)[0]])
    rows = np.concatenate([np.repeat(np.arange(0, 64), 1 + np.arange(64) % 6),          # two full warps of listed rows
                           np.repeat(np.arange(200, 640, 37), 5), [639] * 6])
    rows.sort()
    dec = {"limbs": limbs, "g": rng.randint(-34, -24, N).astype(np.int64), "d": rng.randint(0, 31, N).astype(np.int64),
           "rr": rows.astype(np.int64), "rc": rng.randint(0, K, len(rows)).astype(np.int64),
           "rv": rng.randint(-(1 << 20), 1 << 20, len(rows)).astype(np.int64)}
    sh = rng.randint(-45, -8, M).astype(np.int64)
    want, wflag = ox.linear(q, sh, dec, checked=True)
    fl = _lin(dec)
    for tile in (None, 32, 48, 80, -48, 232, 20264, 448, 548, 580, 648, 664, 680, 764, 40764):
        y, flag = _run(fl, q, sh, True, tile)
        assert np.array_equal(y, want), (tile, int((y != want).sum()))
        assert flag == wflag


def test_random_shapes_on_random_kernels():
    """Sixty seeded shapes (row counts around the 48 / 128 / 256 boundaries, ragged N and K, 0 .. N residual entries,
    three ranges of row exponents), each on eight kernels drawn from all tile codes."""
    rng = np.random.RandomState(4)
    codes = [None, 16, 32, 48, 64, 80, -16, -32, -48, 216, 232, 264, 20264, 40232, 416, 448, 516, 548, 580, 616, 632,
             648, 664, 680, 764, 20764, 40764]
    for _ in range(60):
        M = int(rng.choice([1, 3, 17, 48, 49, 64, 100, 127, 128, 129, 200, 255, 256, 257, 300, 385]))
        N = int(rng.choice([8, 40, 63, 64, 65, 128, 130, 200, 512, 1000, 2050]))
        K = int(rng.choice([16, 48, 128, 144, 256, 272, 1024, 2048, 4112]))
        W = rng.randint(-8355711, 8355712, (N, K)).astype(np.int64)
        q = rng.randint(-(1 << 22), (1 << 22) + 1, (M, K)).astype(np.int64)
        nres = int(rng.choice([0, 1, max(1, N // 16), N]))
        dec = {"limbs": np.stack([l.astype(np.int8) for l in ox.split_limbs(W, 3)[0]]),
               "g": rng.randint(-34, -24, N).astype(np.int64), "d": rng.randint(0, 31, N).astype(np.int64),
               "rr": np.sort(rng.randint(0, N, nres)).astype(np.int64), "rc": rng.randint(0, K, nres).astype(np.int64),
               "rv": rng.randint(-(1 << 20), 1 << 20, nres).astype(np.int64)}
        lo = int(rng.choice([-45, -25, -12]))
        sh = rng.randint(lo, lo + 20, M).astype(np.int64)
        want, wflag = ox.linear(q, sh, dec, checked=True)
        fl = _lin(dec)
        for ci in rng.choice(len(codes), 8, replace=False):
            y, flag = _run(fl, q, sh, True, codes[ci])
            assert np.array_equal(y, want), (M, N, K, codes[ci], nres, int((y != want).sum()))
            assert flag == wflag, (M, N, K, codes[ci])


def test_bf16_weights_config_one_shape():
    """q_proj shape of Llama-3.2-1B, M = 64, seed-0 N(0, 0.02^2) bf16 weights, uniform |q| <= 2^22."""
    from bitexact_llm_b200.exact.consts import decompose
    g = torch.Generator().manual_seed(0)
    w = (torch.randn(2048, 2048, generator=g) * 0.02).to(torch.bfloat16)
    q = torch.randint(-(1 << 22), (1 << 22) + 1, (64, 2048), generator=g)
    sh = torch.randint(-20, -7, (64,), generator=g)
    dec = {k: v.numpy() for k, v in decompose(w).items()}
    assert len(dec["rr"]) > 0
    want, wflag = ox.linear(q.numpy(), sh.numpy(), dec, checked=True)
    y, flag = _run(_lin(dec), q.numpy(), sh.numpy())
    assert np.array_equal(y, want) and flag == wflag


def test_strided_rows_and_empty_batch():
    rng = np.random.RandomState(5)
    N, K = 128, 256
    W = rng.randint(-8355711, 8355712, (N, K)).astype(np.int64)
    dec = {"limbs": np.stack([l.astype(np.int8) for l in ox.split_limbs(W, 3)[0]]), "g": np.full(N, -30, np.int64),
           "d": np.zeros(N, np.int64), "rr": np.zeros(0, np.int64), "rc": np.zeros(0, np.int64), "rv": np.zeros(0, np.int64)}
    fl = _lin(dec)
    big = torch.from_numpy(rng.randint(-(1 << 22), 1 << 22, (5, 2 * K)).astype(np.int32)).cuda()
    q = big[:, :K]                                           # row stride 2K
    sh = torch.full((5,), -12, dtype=torch.long, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = fl(q, sh, flag)
    want = ox.linear(q.cpu().numpy(), sh.cpu().numpy(), dec, checked=False)
    assert np.array_equal(y.cpu().numpy(), want)
    assert fl(q[:0], sh[:0], flag).shape == (0, N)


def test_unfused_linear_api_and_bmm():
    """Lin.__call__ + segs.lin_y (dense product, residual and epilogue as separate calls), wmm, and the exact batched
    product bmm give the integers of the fused kernel / of int64 numpy."""
    from bitexact_llm_b200.bmm import bmm
    from bitexact_llm_b200.exact import segs, wmm
    z = np.load(os.path.join(GOLD, "exact_ops.npz"))
    dec = {k: z["lin_" + k] for k in ("limbs", "g", "d", "rr", "rc", "rv")}
    fl = _lin(dec)
    from bitexact_llm_b200.exact.model import Lin
    lin = Lin({k: torch.from_numpy(v) for k, v in dec.items()}, None, "cuda")
    q = torch.from_numpy(z["lin_q"].astype(np.int64)).cuda()
    sh = torch.from_numpy(z["lin_sh"].astype(np.int64)).cuda()
    C, rs, d, g = lin(q)
    assert np.array_equal(C.cpu().numpy(), ox.dense_product(z["lin_q"].astype(np.int64), dec["limbs"]))
    y, flag = segs.lin_y(C, rs, d, g, sh, True)
    assert np.array_equal(y.cpu().numpy(), z["lin_y"]) and bool(flag) == bool(z["lin_flag"])
    y2 = segs.lin_y(C, (q, fl.ec.long(), fl.ev), d, g, sh) if fl.has_res else y
    assert np.array_equal(y2.cpu().numpy(), z["lin_y"])
    assert wmm.wmm_triton is wmm.wmm
    rng = np.random.RandomState(5)
    for Z, M, K, N, da, db in [(3, 5, 64, 70, np.int64, np.int64), (16, 16, 64, 300, np.int32, np.int64),
                               (2, 130, 515, 64, np.int64, np.int32), (1, 1, 1, 1, np.int32, np.int32),
                               (5, 97, 130, 129, np.int32, np.int32), (2, 260, 2048, 40, np.int64, np.int64)]:
        a = rng.randint(-(1 << 22), (1 << 22) + 1, (Z, M, K)).astype(da)
        b = rng.randint(-8355711, 8355712, (Z, N, K)).astype(db)               # stored transposed: strided view
        a[0, 0, :] = 8355711                                                    # extremes of three limbs
        b[0, 0, :] = -8355711
        bt = torch.from_numpy(b).cuda().transpose(1, 2)
        want = np.einsum("zmk,znk->zmn", a.astype(np.int64), b.astype(np.int64))
        ad = torch.from_numpy(a).cuda()
        for path, tiles in (("cuda", (0,)), ("tensor", (0, 16, 32, 48, 64, 80))):
            for tile in tiles:
                c = bmm(ad, bt, path=path, tile_rows=tile)
                assert np.array_equal(c.cpu().numpy(), want), (Z, M, K, N, path, tile)
        # b stored [Z, K, N] contiguous (the p.V layout) and a strided view of a
        bkn = torch.from_numpy(np.ascontiguousarray(b.transpose(0, 2, 1))).cuda()
        a2 = torch.from_numpy(np.concatenate([a, a], 2)).cuda()[:, :, :K]
        assert np.array_equal(bmm(a2, bkn).cpu().numpy(), want), (Z, M, K, N, "contiguous b")
    assert bmm(torch.zeros(2, 3, 0, dtype=torch.long, device="cuda"), torch.zeros(2, 0, 4, dtype=torch.long, device="cuda")) \
        .abs().sum().item() == 0
