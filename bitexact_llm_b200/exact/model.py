"""Weight holders of exact mode, mirroring `bitexact.exact.model.Lin` (src/bitexact/exact/model.py:31-70)."""

import torch


class Lin:
    """One linear layer's constants on a device: limbs int8 [3, N, K], g, d int64 [N], COO residual rr, rc, rv.

    `c` is a constants dict with keys `{name}.limbs|g|d|rr|rc|rv` (the reference's layout) or the dict returned
    by `consts.decompose` when `name` is None."""

    def __init__(self, c, name=None, device="cuda", gemm="triton", ell=False, R=0, cpu_lazy=False):
        """`gemm`, `ell`, `R` and `cpu_lazy` are the reference's arguments (GEMM back end, padded residual lists,
        their common width, lazy float64 copies on CPU): accepted and ignored, there is one back end here; `ell`
        only selects the form `__call__` returns the residual in."""
        t = (lambda k: c[k]) if name is None else (lambda k: c[f"{name}.{k}"])
        self.ell, self._R = bool(ell), int(R)
        self.limbs = t("limbs").to(device).contiguous()
        self.N, self.K = self.limbs.shape[1], self.limbs.shape[2]
        self.g, self.d = t("g").to(device).contiguous(), t("d").to(device).contiguous()
        self.rr, self.rc, self.rv = t("rr").to(device), t("rc").to(device), t("rv").to(device)

    def __call__(self, q):
        """(C, rs, d, g): the exact dense product and the residual, the arguments of `segs.lin_y`
        (src/bitexact/exact/model.py:61-70)."""
        from .wmm import residual, wmm
        if self.ell:
            return wmm(q, self.limbs), (q,) + self._ell_lists(), self.d, self.g
        return wmm(q, self.limbs), (residual(q, self.rr, self.rc, self.rv, self.N),), self.d, self.g

    def _ell_lists(self):
        """(ec, ev): the residual as padded per-row lists int64 [N, R] (src/bitexact/exact/model.py:39-48)."""
        if not hasattr(self, "_ec"):
            rr = self.rr
            cnt = torch.bincount(rr, minlength=self.N)
            R = max(self._R, int(cnt.max()) if rr.numel() else 0)
            start = torch.cumsum(cnt, 0) - cnt
            order = torch.argsort(rr, stable=True)
            rs = rr[order]
            j = torch.arange(rr.numel(), device=rr.device) - start[rs]
            ec = torch.zeros(self.N, R, dtype=torch.long, device=rr.device)
            ev = torch.zeros(self.N, R, dtype=torch.long, device=rr.device)
            ec[rs, j], ev[rs, j] = self.rc[order], self.rv[order]
            self._ec, self._ev = ec, ev
        return self._ec, self._ev
