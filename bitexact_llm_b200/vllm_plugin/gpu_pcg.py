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


def seed_state(keys, device="cuda"):
    """[(seed, t)] -> int64 [n, 4] on the host: state hi, lo, increment hi, lo of PCG64 after numpy's SeedSequence
    seeding of [20261022, seed, t] (src/bitexact/vllm_plugin/gpu_pcg.py:44-52; computed by a kernel here)."""
    n = len(keys)
    st = torch.empty(n, 4, dtype=torch.long, device=device)
    if n:
        k = torch.tensor([[int(s), int(t)] for s, t in keys], dtype=torch.long).to(device)
        nv.check(nv.lib().bx_pcg_seed_state(k.data_ptr(), st.data_ptr(), n, nv.stream()), "bx_pcg_seed_state")
    return st.cpu()


def raw_from_state(st, device, n_out=V):
    """st int64 [n, 4] (seed_state) -> int64 [n, n_out] raw words on `device`
    (src/bitexact/vllm_plugin/gpu_pcg.py:94-104)."""
    st = st.to(device).contiguous()
    out = torch.empty(st.shape[0], n_out, dtype=torch.long, device=device)
    if st.shape[0]:
        nv.check(nv.lib().bx_pcg_raw_from_state(st.data_ptr(), out.data_ptr(), st.shape[0], n_out, nv.stream()),
                 "bx_pcg_raw_from_state")
    return out
