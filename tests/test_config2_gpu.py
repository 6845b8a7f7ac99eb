"""The limb GEMMs of one Llama-3.2-1B decoder layer and the LM head at M in {1, 16, 256, 4096}, exact and int8 mode,
on bf16 weights drawn from N(0, 0.02^2) and activations quantised from N(0, 1) float64 rows, against the CPU
oracle (float64 GEMM of the limbs, the reference's CPU path). The seven separate projections and the fused forms
the engines use (qkv N = 3072, gate / up N = 16384). Modelled on the reference's tests/test_vllm_exact_gemm.py:23-31
(row counts x value ranges incl. flag equality). The oracle is row- and column-local, so the largest products
(LM head, M = 4096) are checked on a seeded sample of rows over every column."""

import numpy as np
import pytest
import torch

from oracle import exact as ox
from oracle import int8 as o8

pytestmark = pytest.mark.gpu

SHAPES = {"q": (2048, 2048), "k": (512, 2048), "v": (512, 2048), "o": (2048, 2048), "gate": (8192, 2048),
          "up": (8192, 2048), "down": (2048, 8192), "wqkv": (3072, 2048), "wgu": (16384, 2048),
          "lm": (128256, 2048)}
MS = (1, 16, 256, 4096)
ORACLE_ROWS = 128                                            # rows checked when M * N * K is too large for the CPU


def _weights(name):
    N, K = SHAPES[name]
    g = torch.Generator().manual_seed(sum(map(ord, name)))
    return (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)


def _rows(M, K, seed):
    return np.random.RandomState(seed).standard_normal((M, K))


def _sample_rows(M, N, K, seed):
    if 3.0 * M * N * K <= 3.0 * 4096 * 16384 * 2048:
        return np.arange(M)
    return np.sort(np.random.RandomState(seed).choice(M, ORACLE_ROWS, replace=False))


@pytest.mark.parametrize("name", list(SHAPES))
def test_exact_projection_all_batch_sizes(name):
    from bitexact_llm_b200.exact.consts import decompose
    from bitexact_llm_b200.exact.model import Lin
    from bitexact_llm_b200.vllm_plugin.exact_gemm import FusedLin
    N, K = SHAPES[name]
    dec = decompose(_weights(name).cuda())
    fl = FusedLin(Lin(dec, None, "cuda"))
    dec_np = {k: v.cpu().numpy() for k, v in dec.items()}
    dec_np["keep_w64"] = True                                    # one float64 weight copy for the four batch sizes
    for M in MS:
        x = _rows(M, K, M + N)
        q, sh = ox.quant(np.rint(x * 2.0 ** 40).astype(np.int64), -40)
        sel = _sample_rows(M, N, K, M)
        want, wflag = ox.linear(q[sel], sh[sel], dec_np, checked=True)
        flag = torch.zeros(1, dtype=torch.int32, device="cuda")
        y = fl(torch.from_numpy(q.astype(np.int32)).cuda(), torch.from_numpy(sh).cuda(), flag, True)
        got = y[torch.from_numpy(sel).cuda()].cpu().numpy()
        assert np.array_equal(got, want), (name, M, int((got != want).sum()))
        assert not wflag and not bool(flag.item())
        del y
    from bitexact_llm_b200 import _native as nv
    assert nv.device_status() == 0


@pytest.mark.parametrize("name", list(SHAPES))
def test_int8_projection_all_batch_sizes(name):
    from bitexact_llm_b200.int8.consts import q_linear
    from bitexact_llm_b200.int8.gemm_skinny import int_mm, linear_post
    N, K = SHAPES[name]
    w8, mul, fm = q_linear(_weights(name).double())
    assert np.array_equal(w8.numpy(), o8.q_linear(_weights(name).double().numpy())[0])
    fmsh = fm + 8 - 24
    w_dev, mul_dev = w8.cuda(), mul.cuda()
    w_np, mul_np = w8.numpy(), mul.numpy()
    for M in MS:
        x = _rows(M, K, 7 * M + N)
        q, mant, e = o8.pre_plain(np.rint(x * 2.0 ** 16).astype(np.int64), 2)
        sel = _sample_rows(M, N, K, M)
        acc = o8.imm(q[sel], w_np)
        want, wflag = o8.post(acc, mul_np, fmsh, mant[sel], e[sel])
        a = torch.from_numpy(o8.stack_limbs(q, 2)).cuda()
        flag = torch.zeros(1, dtype=torch.int32, device="cuda")
        y = linear_post(a, w_dev, mul_dev, fmsh, torch.from_numpy(mant).cuda(), torch.from_numpy(e).cuda(), flag, M=M)
        seld = torch.from_numpy(sel).cuda()
        got = y[seld].cpu().numpy()
        assert np.array_equal(got, want), (name, M, int((got != want).sum()))
        assert bool(flag.item()) == wflag
        if N <= 16384:                                           # the raw two-step form: limb products as int_mm
            c = int_mm(a, w_dev, M=M)
            joined = (c[:M].long() + (c[M:2 * M].long() << 8))[seld].cpu().numpy()
            assert np.array_equal(joined, acc), (name, M)
        del y
