"""Weight preparation of exact mode: bf16 weights -> 3 dense int8 limbs + sparse low-bit residual.

Mirrors the interface of the reference's `bitexact.exact.consts` (`bf16_parts`, `decompose`, constants;
src/bitexact/exact/consts.py:23-107) and produces the same tensors.  Written with torch ops so that it runs on
the device that holds the weights (it is a load-time step, not part of the decode path).
"""

import torch

FR, FT, FL = 24, 30, 40
EXP2_BITS, EXP2_ONE = 14, 60
MAX_POS = 4096
LIM3 = 8355711
NW = 3


def bf16_parts(w):
    """bf16 tensor -> (signed significand, exponent), w = sm * 2^ex exactly (consts.py:33-42)."""
    b = w.contiguous().view(torch.int16).long() & 0xFFFF
    e = (b >> 7) & 0xFF
    if bool((e == 255).any()):
        raise ValueError("inf/nan weight")
    frac = b & 0x7F
    mag = torch.where(e > 0, frac | 0x80, frac)
    ex = e.clamp(min=1) - 134
    return torch.where(b >= 0x8000, -mag, mag), ex


def _smax_table(device):
    """smax[mag] = largest s >= 0 with mag << s <= LIM3 (mag = 1..255); 0 for mag = 0."""
    t = [0] * 256
    for m in range(1, 256):
        s = 0
        while (m << (s + 1)) <= LIM3:
            s += 1
        t[m] = s
    return torch.tensor(t, dtype=torch.long, device=device)


def decompose(w, row_chunk=4096):
    """bf16 [N, K] -> {"limbs": int8 [3, N, K], "g", "d": int64 [N], "rr", "rc", "rv": COO residual}.

    Per output row: grid exponent g = the smallest exponent for which every |trunc(w / 2^g)| <= LIM3 (three signed
    base-256 digits); the bits a truncation drops are kept exactly as sparse integers on the finer grid g - d
    (consts.py:67-107)."""
    N, K = w.shape
    dev = w.device
    smax = _smax_table(dev)
    limbs = torch.empty(3, N, K, dtype=torch.int8, device=dev)
    gs, ds, rrs, rcs, rvs = [], [], [], [], []
    for r0 in range(0, N, row_chunk):
        sm, ex = bf16_parts(w[r0:r0 + row_chunk])
        mag = sm.abs()
        nz = mag > 0
        need = torch.where(nz, ex - smax[mag], torch.full_like(ex, -10 ** 6))
        g = need.amax(1)
        g = torch.where(g < -10 ** 5, torch.zeros_like(g), g)
        sh = ex - g[:, None]
        up = sh >= 0
        l = sh.clamp(0, 40)
        r = (-sh).clamp(0, 40)
        dense = torch.where(up, mag << l, mag >> r)
        lost = torch.where(up, torch.zeros_like(mag), mag - ((mag >> r) << r))
        W = torch.where(sm < 0, -dense, dense)
        has = lost > 0
        low = lost & -lost                                     # lowest set bit, a power of two < 2^9
        lowidx = torch.zeros_like(low)
        for i in range(1, 9):
            lowidx = torch.where(low == (1 << i), torch.full_like(low, i), lowidx)
        lowexp = torch.where(has, ex + lowidx, torch.full_like(ex, 10 ** 6))
        gf = torch.minimum(lowexp.amin(1), g)
        d = g - gf
        if int(d.max()) > 30:
            raise ValueError("residual grid too fine")
        rr, rc = has.nonzero(as_tuple=True)
        s_ = ex[rr, rc] - gf[rr]
        rv = lost[rr, rc] << s_.clamp(min=0)                     # s_ >= 0: gf <= every residual bit's exponent
        rv = torch.where(sm[rr, rc] < 0, -rv, rv)
        rem = W
        for i in range(3):
            lo = ((rem + 128) & 255) - 128
            limbs[i, r0:r0 + row_chunk] = lo.to(torch.int8)
            rem = (rem - lo) >> 8
        if bool(rem.any()):
            raise ValueError("limb split left a remainder")
        gs.append(g), ds.append(d), rrs.append(rr + r0), rcs.append(rc), rvs.append(rv)
    return {"limbs": limbs, "g": torch.cat(gs), "d": torch.cat(ds), "rr": torch.cat(rrs), "rc": torch.cat(rcs),
            "rv": torch.cat(rvs)}


def exp2_table(device="cpu"):
    """2^-f at 2^60, f = i / 2^14, i = 0..2^14 (consts.py:112-113)."""
    f = torch.arange((1 << EXP2_BITS) + 1, dtype=torch.float64) / (1 << EXP2_BITS)
    return torch.round(torch.pow(2.0, -f) * 2.0 ** EXP2_ONE).long().to(device)


def ln_table(bits=FL, device="cpu"):
    """ln(1 + i / 2^16) at `bits` fractional bits (src/bitexact/llama.py:72-75)."""
    i = torch.arange((1 << 16) + 1, dtype=torch.float64)
    return torch.round(torch.log1p(i / (1 << 16)) * 2.0 ** bits).long().to(device)
