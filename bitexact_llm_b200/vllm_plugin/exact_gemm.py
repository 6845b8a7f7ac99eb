"""Exact-mode fused linear: drop-in for `bitexact.vllm_plugin.exact_gemm.FusedLin`
(src/bitexact/vllm_plugin/exact_gemm.py:228-316) on libbitexact_b200's tcgen05 limb GEMM."""

import torch

from .. import _native as nv


class FusedLin:
    """The linear layer `lin` (an `exact.model.Lin`): q int32 [M, K], sh int64 [M] -> y int64 [M, N] at 24
    fractional bits; sets flag (int32 [1]) to 1 when `checked` and the epilogue lost bits or |y| >= 2^62."""

    def __init__(self, lin, cfg=None):
        self.limbs, self.d, self.g, self.N = lin.limbs, lin.d, lin.g, lin.N
        self.K = self.limbs.shape[2]
        dev = self.limbs.device
        rr = lin.rr
        self.has_res = rr.numel() > 0
        if self.has_res:                                         # padded per-row residual lists (ELL)
            cnt = torch.bincount(rr, minlength=self.N)
            self.R = int(cnt.max())
            start = torch.cumsum(cnt, 0) - cnt
            order = torch.argsort(rr, stable=True)
            rs = rr[order]
            j = torch.arange(rr.numel(), device=rr.device) - start[rs]
            ec = torch.zeros(self.N, self.R, dtype=torch.int32, device=rr.device)
            ev = torch.zeros(self.N, self.R, dtype=torch.long, device=rr.device)
            ec[rs, j], ev[rs, j] = lin.rc[order].to(torch.int32), lin.rv[order]
            self.cnt, self.ec, self.ev = cnt.to(torch.int32).to(dev), ec.to(dev), ev.to(dev)
        else:
            self.R, self.cnt, self.ec, self.ev = 0, None, None, None
        self.cfg = cfg                                           # tile rows (16..80) or None = automatic
        self.timer = None                                        # optional callable(M, N, K) -> context manager

    def __call__(self, q, sh, flag, checked=True):
        M, K = q.shape
        assert q.dtype == torch.int32 and q.stride(1) == 1 and K == self.K and sh.dtype == torch.int64
        sh = sh.contiguous()
        y = torch.empty((M, self.N), dtype=torch.long, device=q.device)
        if M == 0:
            return y
        if self.timer is not None:
            with self.timer(M, self.N, K):
                return self._run(q, sh, flag, checked, y, M, K)
        return self._run(q, sh, flag, checked, y, M, K)

    def _run(self, q, sh, flag, checked, y, M, K):
        from .exact_fuse import planes_of
        planes = planes_of(q, M, K)                      # limb planes written by the stage kernel that produced q
        if planes is not None:
            rc = nv.lib().bx_exact_linear_planes(planes.data_ptr(), q.data_ptr(), q.stride(0), sh.data_ptr(),
                                                 self.limbs.data_ptr(), self.d.data_ptr(), self.g.data_ptr(),
                                                 nv.ptr(self.cnt), nv.ptr(self.ec), nv.ptr(self.ev), self.R,
                                                 y.data_ptr(), flag.data_ptr(), M, self.N, K, int(bool(checked)),
                                                 self.cfg or 0, nv.stream())
            nv.check(rc, "bx_exact_linear_planes")
            return y
        scratch = torch.empty(3 * M * K, dtype=torch.int8, device=q.device)
        rc = nv.lib().bx_exact_linear(q.data_ptr(), q.stride(0), sh.data_ptr(), self.limbs.data_ptr(),
                                      self.d.data_ptr(), self.g.data_ptr(), nv.ptr(self.cnt), nv.ptr(self.ec),
                                      nv.ptr(self.ev), self.R, scratch.data_ptr(), y.data_ptr(), flag.data_ptr(),
                                      M, self.N, K, int(bool(checked)), self.cfg or 0, nv.stream())
        nv.check(rc, "bx_exact_linear")
        return y
