"""numpy's PCG64 raw stream on the GPU: drop-in for `bitexact.vllm_plugin.gpu_pcg.raw_rows`
(src/bitexact/vllm_plugin/gpu_pcg.py:94-108).  Seeding (SeedSequence) runs on the device too."""

import torch

from .. import _native as nv

V = 128256


def raw_rows(keys, device, n_out=V):
    """[(seed, t)] -> int64 [n, n_out] raw words of np.random.default_rng([20261022, seed, t]) on `device`."""
    n = len(keys)
    out = torch.empty(n, n_out, dtype=torch.long, device=device)
    if n:
        k = torch.tensor([[int(s), int(t)] for s, t in keys], dtype=torch.long).to(device)
        nv.check(nv.lib().bx_pcg_raw(k.data_ptr(), out.data_ptr(), n, n_out, nv.stream()), "bx_pcg_raw")
    return out
