"""Stages of the int8 engine with the reference's names (src/bitexact/int8/segs.py:62-99): `post` on a joined
accumulator and the dense-score `softmax`, one kernel of libbitexact_b200 each. The serving path fuses `post` into
the GEMM (`gemm_skinny.linear_post`) and the weights into the paged attention kernels."""

import torch

from .. import _native as nv

FR, FQ, FV, FP, FA, FE = 16, 14, 14, 20, 12, 30


def post(acc, m, fmsh, mant, e, check=True):
    """acc int64 [M, N] (the joined limb products), m int64 [N], fmsh an int (or 0-d tensor), mant / e int64 [M] ->
    (y int64 [M, N] at 16 bits, flag): t = rsh(acc m, fmsh), y = rsh(t mant, 8 - e); flag (|t| >= 2^38 somewhere) is
    None without `check`."""
    M, N = acc.shape
    y = torch.empty(M, N, dtype=torch.long, device=acc.device)
    flag = torch.zeros(1, dtype=torch.int32, device=acc.device)
    rc = nv.lib().bx_int8_post_acc(acc.contiguous().data_ptr(), m.contiguous().data_ptr(), int(fmsh),
                                   mant.contiguous().data_ptr(), e.contiguous().data_ptr(), y.data_ptr(), flag.data_ptr(), M,
                                   N, int(bool(check)), nv.stream())
    nv.check(rc, "bx_int8_post_acc")
    return y, ((flag[0] != 0) if check else None)


def softmax(raw, qpos, expt, hd=64):
    """raw int64 [B, HKV, gT, S] q.k at 28 bits, qpos [B, 1, gT, 1] (or broadcastable) -> weights p int64 at 20 bits
    (masked: 0) and their sums [B, HKV, gT, 1] (head_dim 64 rule)."""
    assert hd == 64
    from ..vllm_plugin.tri_paged import weight_table
    shape = raw.shape
    S = shape[-1]
    R = raw.numel() // S
    raw2 = raw.reshape(R, S).contiguous()
    qp = torch.broadcast_to(qpos, shape[:-1] + (1,)).reshape(R).long().contiguous()
    ptab = weight_table(expt)
    p = torch.empty(R, S, dtype=torch.int32, device=raw.device)
    den = torch.empty(R, dtype=torch.long, device=raw.device)
    rc = nv.lib().bx_softmax_w(raw2.data_ptr(), None, qp.data_ptr(), None, None, 0, ptab.data_ptr(), p.data_ptr(),
                               den.data_ptr(), R, S, nv.stream())
    nv.check(rc, "bx_softmax_w")
    return p.long().view(shape), den.view(shape[:-1] + (1,))
