"""LM-head post-processing, greedy argmax and integer Gumbel sampling from the int8-mode LM-head GEMM output:
drop-in for `bitexact.vllm_plugin.tri_sample` (src/bitexact/vllm_plugin/tri_sample.py:296-394).

`Head` carries the raw int32 limb products of the LM-head GEMM (or the int64 logits when the fused linear already
applied `post`) with the constants of `segs.post`; `head` gives the first argmax and the float rows vLLM's sampler
reads; `noisy` the Gumbel-max token per row. The integers are those of `segs.post`, `sampling.gumbel` and
`sampling.sample`."""

import numpy as np
import torch

from .. import _native as nv
from . import tri_logits
from .sampler import sample_rows


class Head:
    """The LM-head GEMM output and the constants that turn it into logits (segs.post's arguments)."""

    def __init__(self, c, m, fmsh, mant, e, rows=None):
        self.c, self.m, self.mant, self.e = c, m, mant, e
        self.fmsh = int(fmsh)
        self.M, self.V = mant.shape[0], c.shape[1]
        self.R = self.M if rows is None else rows         # rows used: the first R of the M the GEMM computed

    def logits(self):
        """The int64 logits [R, V] at 16 fractional bits."""
        if self.c.dtype == torch.int64:
            return self.c[:self.R]
        y = torch.empty(self.M, self.V, dtype=torch.long, device=self.c.device)
        flag = torch.zeros(1, dtype=torch.int32, device=self.c.device)
        if self.M:
            rc = nv.lib().bx_int8_post(self.c.data_ptr(), self.m.data_ptr(), self.fmsh, self.mant.contiguous().data_ptr(),
                                       self.e.contiguous().data_ptr(), y.data_ptr(), flag.data_ptr(), self.M, self.V, 0,
                                       nv.stream())
            nv.check(rc, "bx_int8_post")
        return y[:self.R]


def head(h, mode, block=1024, gate=None):
    """mode 'float': (float32 logits * 2^-16, first argmax); 'onehot': (-inf row with 0 at the argmax, argmax);
    'none': (None, argmax). `gate` (a device scalar that switches the pass off inside a CUDA graph in the reference)
    is accepted; the pass always runs, a caller that gated it off ignores the result."""
    return tri_logits.argmax_float(h.logits(), 2.0 ** -16, mode)


def row_state(keys, temps):
    """[(seed, t)], [(tn, td)] -> int64 [n, 4]: seed, t, tn, td per row (the PCG state is derived on the device)."""
    st = torch.zeros(len(keys), 4, dtype=torch.long)
    for r, ((seed, t), (tn, td)) in enumerate(zip(keys, temps)):
        st[r, 0], st[r, 1], st[r, 2], st[r, 3] = int(seed), max(int(t), 0), int(tn), int(td)
    return st


def noisy(h, st, lnt, block=1024, out=None):
    """Gumbel-max token per row: st int64 [n, 4] = seed, t, tn, td (torch or numpy, host or device; tn = 0: greedy).
    Same tokens as sampling.sample(li, tn, td, gumbel(raw, ...)). out: vLLM's float logits [M, V]; if given it is left
    as -inf rows with 0 at the token."""
    dev = h.c.device
    st = torch.as_tensor(np.asarray(st) if not torch.is_tensor(st) else st)
    assert st.shape[1] == 4, "rows are (seed, t, tn, td)"
    st = st.to(dev, non_blocking=True).contiguous()
    y = sample_rows(h.logits().contiguous(), st[:h.R], lnt, 16)
    if out is not None and h.R:
        out[:h.R].fill_(float("-inf"))
        out[:h.R].scatter_(1, y[:, None], 0.0)
    return y
