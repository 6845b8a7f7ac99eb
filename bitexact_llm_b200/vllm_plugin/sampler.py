"""Integer sampler: drop-in for `bitexact.vllm_plugin.sampler.integer_sample` and
`bitexact.vllm_plugin.tri_logits.first_argmax` (src/bitexact/vllm_plugin/sampler.py:57-88,
vllm_plugin/tri_logits.py:97-100)."""

import torch

from .. import _native as nv

FR = 24


def sample_rows(li, rows, lnt, fr=FR):
    """li int64 [M, V] (unit column stride), rows int64 [M, 4] on the device = (seed, t, tn, td) per row
    (tn = 0: greedy) -> int64 [M] tokens. No host sync."""
    M, V = li.shape
    assert li.dtype == torch.int64 and li.stride(1) == 1
    tok = torch.empty(M, dtype=torch.long, device=li.device)
    if M:
        lib = nv.lib()
        scratch = torch.empty(max(1, lib.bx_sample_scratch_bytes(M, V)), dtype=torch.uint8, device=li.device)
        rc = lib.bx_sample(li.data_ptr(), li.stride(0), rows.data_ptr(), lnt.data_ptr(), scratch.data_ptr(),
                           tok.data_ptr(), M, V, fr, nv.stream())
        nv.check(rc, "bx_sample")
    return tok


def integer_sample(li, seeds, ts, temps, lnt, greedy=None, fr=FR):
    """li int64 [M, V]; per row seed, generated index t, (tn, td). Returns int64 [M] token ids."""
    rows = torch.tensor([[int(s), max(int(t), 0), int(tn), int(td)] for s, t, (tn, td) in zip(seeds, ts, temps)],
                        dtype=torch.long).reshape(-1, 4).to(li.device)
    return sample_rows(li, rows, lnt, fr)


def first_argmax(v):
    """Index of the first maximum of each row of int64 [M, V]."""
    rows = torch.zeros(v.shape[0], 4, dtype=torch.long, device=v.device)
    rows[:, 3] = 1
    return sample_rows(v, rows, rows, FR)
