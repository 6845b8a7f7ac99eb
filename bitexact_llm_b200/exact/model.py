"""Weight holders of exact mode, mirroring `bitexact.exact.model.Lin` (src/bitexact/exact/model.py:31-70)."""

import torch


class Lin:
    """One linear layer's constants on a device: limbs int8 [3, N, K], g, d int64 [N], COO residual rr, rc, rv.

    `c` is a constants dict with keys `{name}.limbs|g|d|rr|rc|rv` (the reference's layout) or the dict returned
    by `consts.decompose` when `name` is None."""

    def __init__(self, c, name=None, device="cuda"):
        t = (lambda k: c[k]) if name is None else (lambda k: c[f"{name}.{k}"])
        self.limbs = t("limbs").to(device).contiguous()
        self.N, self.K = self.limbs.shape[1], self.limbs.shape[2]
        self.g, self.d = t("g").to(device).contiguous(), t("d").to(device).contiguous()
        self.rr, self.rc, self.rv = t("rr").to(device), t("rc").to(device), t("rv").to(device)

    def __call__(self, q):
        """(C, rs, d, g): the exact dense product and the residual, the arguments of `segs.lin_y`
        (src/bitexact/exact/model.py:61-70)."""
        from .wmm import residual, wmm
        return wmm(q, self.limbs), (residual(q, self.rr, self.rc, self.rv, self.N),), self.d, self.g
