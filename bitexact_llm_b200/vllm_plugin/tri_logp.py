"""Integer log p of given tokens from the LM-head GEMM output: drop-in for `bitexact.vllm_plugin.tri_logp.logp`
(src/bitexact/vllm_plugin/tri_logp.py:70-91). The reference reads the GEMM's int32 limb products twice and applies
`segs.post` on the fly; here the fused linear has already written the int64 logits (`Head.logits`), and the same two
passes (row maximum, sum of e^(l - max)) read those."""

from . import rl


def logp(h, tok, lnt):
    """Integer log p of tok [M] under the logits rows of Head h: float64 at 2^-40, equal to
    rl.int_logp(h.logits(), tok, lnt)."""
    return rl.int_logp(h.logits().contiguous(), tok[:h.R], lnt, 16)
