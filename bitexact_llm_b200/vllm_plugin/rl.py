"""Integer log p of given tokens from int64 logits rows: drop-in for `int_logp` and `lse_table` of
`bitexact.vllm_plugin.rl` (src/bitexact/vllm_plugin/rl.py:32-65), two sm_100a passes over the rows.

The rest of that module (weight swaps inside a live vLLM engine, the scoring requests of its scheduler) is vLLM glue
and is not part of this package."""

import torch

from .. import _native as nv

LSE_FE, LSE_MIN = 44, -40
FL = 40
_LSE_TAB = {}
_INVALID = -(1 << 63)


def lse_table(device):
    """e^x at 44 bits for x in [-40, 0] at step 2^-12: float64 on the CPU, rounded once (rl.py:32-40)."""
    k = str(device)
    if k not in _LSE_TAB:
        xs = torch.arange(LSE_MIN << 12, 1, dtype=torch.float64) / 4096
        _LSE_TAB[k] = torch.round(torch.exp(xs) * 2.0 ** LSE_FE).long().to(device)
    return _LSE_TAB[k]


def pair_table(device):
    """The table in the layout the kernels gather from: int64 [n, 2] = (entry i, entry min(i + 1, n - 1))."""
    k = "pair:" + str(device)
    if k not in _LSE_TAB:
        tab = lse_table(device)
        t2 = torch.empty(tab.shape[0], 2, dtype=torch.long, device=device)
        nv.check(nv.lib().bx_logp_pair_table(tab.data_ptr(), tab.shape[0], t2.data_ptr(), nv.stream()),
                 "bx_logp_pair_table")
        _LSE_TAB[k] = t2
    return _LSE_TAB[k]


def to_float(q):
    """The integer at 2^-40 as float64 (the reference's conversion); rows whose token was out of range give NaN."""
    return torch.where(q == _INVALID, torch.full_like(q, 0, dtype=torch.float64).fill_(float("nan")),
                       q.double() / 2.0 ** FL)


def int_logp_q(lg, tok, lnt, fr=16):
    """lg int64 [n, V] (unit column stride) at fr bits, tok int64 [n] -> int64 [n]: log p at 2^-40. No host sync."""
    n, V = lg.shape
    assert lg.dtype == torch.int64 and lg.stride(1) == 1 and lg.is_cuda
    out = torch.empty(n, dtype=torch.long, device=lg.device)
    if n:
        lib = nv.lib()
        tab = pair_table(lg.device)
        scratch = torch.empty(max(1, lib.bx_logp_scratch_bytes(n, V)), dtype=torch.uint8, device=lg.device)
        rc = lib.bx_int_logp(lg.data_ptr(), lg.stride(0), tok.long().contiguous().data_ptr(), lnt.data_ptr(),
                             tab.data_ptr(), tab.shape[0], scratch.data_ptr(), out.data_ptr(), n, V, fr, nv.stream())
        nv.check(rc, "bx_int_logp")
    return out


def int_logp(lg, tok, lnt, fr=16):
    """Integer-defined log p of tok [n] from int64 logits rows lg [n, V] (T = 1): float64 of an integer at 2^-40, a
    pure function of the logits row (rl.py:43-65). fr: fractional bits of the logits (the reference's int8 mode: 16)."""
    return to_float(int_logp_q(lg, tok, lnt, fr))
