"""Weight preparation on the GPU (bx_decompose_rows / bx_decompose_residual through exact.consts.decompose) against
the reference's golden decomposition, the CPU oracle and the host form of the same function, on ordinary weights and
on rows built to hit the edges: all-zero rows, subnormals, single huge or tiny entries, every significand."""

import os

import numpy as np
import pytest
import torch

from oracle import exact as ox

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
KEYS = ("limbs", "g", "d", "rr", "rc", "rv")


def from_bits(bits):
    return torch.from_numpy(bits.astype(np.uint16).view(np.int16)).view(torch.bfloat16)


def check(bits):
    from bitexact_llm_b200.exact.consts import decompose
    w = from_bits(bits)
    dev = decompose(w.cuda())
    want = ox.decompose(bits)
    host = decompose(w)
    for k in KEYS:
        got = dev[k].cpu().numpy()
        assert got.dtype == host[k].numpy().dtype and np.array_equal(got, want[k]), k
        assert np.array_equal(got, host[k].numpy()), k
    return dev


def test_golden_decomposition():
    z = np.load(os.path.join(GOLD, "exact_ops.npz"))
    dev = check(z["lin_w"])
    for k in KEYS:
        assert np.array_equal(dev[k].cpu().numpy(), z["lin_" + k]), k
    assert dev["rr"].numel() > 0


@pytest.mark.parametrize("N,K,seed", [(1, 16, 0), (37, 200, 1), (300, 2048, 2), (5, 8192, 3)])
def test_random_weights(N, K, seed):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
    w[0, : min(K, 4)] = torch.tensor([1e-9, -3e-8, 0.0, 2.0][: min(K, 4)]).to(torch.bfloat16)   # forces residual entries
    check(w.view(torch.int16).numpy().astype(np.uint16))


def test_edge_rows():
    K = 300
    rows = []
    rows.append(np.zeros(K, np.uint16))                                       # all zero
    r = np.zeros(K, np.uint16); r[7] = 0x8000; rows.append(r)                 # only a negative zero
    r = np.zeros(K, np.uint16); r[::3] = 0x0001; r[1::3] = 0x807F; rows.append(r)   # subnormals only
    r = np.full(K, 0x3C23, np.uint16); r[5] = 0x4A7F; rows.append(r)           # one large entry: everything else truncated
    r = np.full(K, 0x3C23, np.uint16); r[5] = 0x2F81; rows.append(r)           # one tiny entry
    r = (0x3F80 | (np.arange(K) & 0x7F)).astype(np.uint16); r[1::2] |= 0x8000; rows.append(r)   # every significand, both signs
    r = (0x3F80 + 0x80 * (np.arange(K) % 9)).astype(np.uint16); r[0] = 0x4A7F; rows.append(r)   # nine exponents + a large one
    r = np.zeros(K, np.uint16); r[K - 1] = 0x3FFF; rows.append(r)             # a single entry in the last column
    check(np.stack(rows))


def test_bad_weights_raise():
    from bitexact_llm_b200.exact.consts import decompose
    w = torch.zeros(3, 64, dtype=torch.bfloat16)
    w[1, 5] = float("inf")
    with pytest.raises(ValueError):
        decompose(w.cuda())
    w = torch.full((2, 64), 1.0, dtype=torch.bfloat16)
    w[0, 0] = 3.0e38                                                          # the other entries fall 2^127 below the grid
    with pytest.raises(ValueError):
        decompose(w.cuda())
