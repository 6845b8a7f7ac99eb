"""`tri_mlp.silu_quant` of the reference (src/bitexact/vllm_plugin/tri_mlp.py:153-183) on libbitexact_b200: from the
raw gate / up GEMM output to the quantised SiLU product in the 2-limb row layout."""

import torch

from .. import _native as nv


def silu_quant(c, m, fmsh, mant, e, lut, check, block=512, scr=None):
    """c = int_mm(2-limb input, Wgu^T) (int32, >= 2 M rows), m / fmsh / mant / e as in segs.post ->
    (a8 int8 [2 M + pad, FF] limb rows padded like stack_limbs, mant', e', flag) = segs.silu_mul(segs.post(...)).
    scr (int64 [2], zeroed): the maxima of |silu(g)|, |u| go there as atomic maxima and flag is None (check must be
    False; the caller multiplies them, tri_fuse.flag_end). `block` is a tuning argument of the reference, ignored."""
    M, FF = mant.shape[0], c.shape[1] // 2
    dev = c.device
    lib, st = nv.lib(), nv.stream()
    y = torch.empty(M, 2 * FF, dtype=torch.long, device=dev)
    pflag = torch.zeros(1, dtype=torch.int32, device=dev)
    rows = 2 * M
    pad = max(24, (rows + 7) // 8 * 8) - rows
    q = torch.empty(rows + pad, FF, dtype=torch.int8, device=dev)
    q[rows:].zero_()
    mant2 = torch.empty(M, dtype=torch.long, device=dev)
    e2 = torch.empty_like(mant2)
    own = scr is None
    if own:
        scr = torch.zeros(2, dtype=torch.long, device=dev)
    else:
        assert not check
    if M:
        nv.check(lib.bx_int8_post(c.contiguous().data_ptr(), m.data_ptr(), int(fmsh), mant.data_ptr(), e.data_ptr(),
                                  y.data_ptr(), pflag.data_ptr(), M, 2 * FF, int(bool(check)), st), "bx_int8_post")
        nv.check(lib.bx_int8_silu_quant(y.data_ptr(), lut.data_ptr(), q.data_ptr(), mant2.data_ptr(), e2.data_ptr(),
                                        scr.data_ptr(), M, FF, st), "bx_int8_silu_quant")
    if not own:
        return q, mant2, e2, None
    flag = scr[0] * scr[1] >= 1 << 62
    if check:
        flag = flag | (pflag[0] != 0)
    return q, mant2, e2, flag
