"""First argmax of int64 logits and the float rows vLLM's sampler reads: drop-in for
`bitexact.vllm_plugin.tri_logits` (src/bitexact/vllm_plugin/tri_logits.py:77-100)."""

import torch

from .sampler import first_argmax as _first_argmax

MODES = {"none": 0, "float": 1, "onehot": 2}


def _float_row(li, y, scale, mode):
    if mode == "float":
        return li.to(torch.float32) * scale                  # round to nearest even, then an exact power of two
    out = torch.full(li.shape, float("-inf"), dtype=torch.float32, device=li.device)
    out.scatter_(1, y[:, None], 0.0)
    return out


def argmax_float(li, scale=2.0 ** -16, mode="float", nch=None, block=1024):
    """li int64 [M, V] -> (float32 [M, V] or None, int64 [M] first argmax). mode 'float': li * scale; 'onehot': -inf
    with 0 at the argmax; 'none': no float row. nch and block are tuning arguments of the reference, ignored.
    No host sync."""
    assert mode in MODES
    li = li.contiguous()
    y = _first_argmax(li)
    return (None if mode == "none" else _float_row(li, y, scale, mode)), y


def first_argmax(v):
    """intops.first_argmax for int64 [M, V] on CUDA (same indices)."""
    return _first_argmax(v.contiguous())
