"""Weight preparation of exact mode: bf16 weights -> 3 dense int8 limbs + sparse low-bit residual.

Mirrors the interface of the reference's `bitexact.exact.consts` (`bf16_parts`, `decompose`, constants;
src/bitexact/exact/consts.py:23-107) and produces the same tensors.  Weights that live on a GPU are decomposed by
two sm_100a kernels (`bx_decompose_rows`, `bx_decompose_residual`); the torch-op form below serves host tensors
(it is a load-time step, not part of the decode path).
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
    if w.is_cuda:
        return _decompose_device(w)
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
        lv = lost[rr, rc]                                        # exact either way: gf <= the lowest lost bit
        rv = torch.where(s_ >= 0, lv << s_.clamp(min=0), lv >> (-s_).clamp(min=0))
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


def _decompose_device(w):
    """`decompose` of a bf16 tensor that lives on a GPU: two row-parallel kernels (limbs, g, d, counts; then the
    coordinate list at the offsets of the counts' prefix sum). One host sync for the number of entries."""
    from .. import _native as nv
    N, K = w.shape
    assert w.dtype == torch.bfloat16
    w = w.contiguous()
    dev, lib, st = w.device, nv.lib(), nv.stream()
    limbs = torch.empty(3, N, K, dtype=torch.int8, device=dev)
    g = torch.empty(N, dtype=torch.long, device=dev)
    d = torch.empty(N, dtype=torch.long, device=dev)
    cnt = torch.empty(N, dtype=torch.int32, device=dev)
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    nv.check(lib.bx_decompose_rows(w.data_ptr(), w.stride(0), limbs.data_ptr(), g.data_ptr(), d.data_ptr(),
                                   cnt.data_ptr(), flag.data_ptr(), N, K, st), "bx_decompose_rows")
    incl = torch.cumsum(cnt.long(), 0)
    f = int(flag)
    if f & 1:
        raise ValueError("inf/nan weight")
    if f & 2:
        raise ValueError("residual grid too fine")
    if f & 4:
        raise ValueError("limb split left a remainder")
    total = int(incl[-1]) if N else 0
    rr = torch.empty(total, dtype=torch.long, device=dev)
    rc = torch.empty(total, dtype=torch.long, device=dev)
    rv = torch.empty(total, dtype=torch.long, device=dev)
    if total:
        start = (incl - cnt).contiguous()
        nv.check(lib.bx_decompose_residual(w.data_ptr(), w.stride(0), g.data_ptr(), d.data_ptr(), start.data_ptr(),
                                           rr.data_ptr(), rc.data_ptr(), rv.data_ptr(), N, K, st),
                 "bx_decompose_residual")
    return {"limbs": limbs, "g": g, "d": d, "rr": rr, "rc": rc, "rv": rv}


def exp2_table(device="cpu"):
    """2^-f at 2^60, f = i / 2^14, i = 0..2^14 (consts.py:112-113)."""
    f = torch.arange((1 << EXP2_BITS) + 1, dtype=torch.float64) / (1 << EXP2_BITS)
    return torch.round(torch.pow(2.0, -f) * 2.0 ** EXP2_ONE).long().to(device)


def ln_table(bits=FL, device="cpu"):
    """ln(1 + i / 2^16) at `bits` fractional bits (src/bitexact/llama.py:72-75)."""
    i = torch.arange((1 << 16) + 1, dtype=torch.float64)
    return torch.round(torch.log1p(i / (1 << 16)) * 2.0 ** bits).long().to(device)


# ---- whole-model constants (same keys as the reference's consts.build, src/bitexact/exact/consts.py:118-149) ----

LLAMA_1B = dict(vocab_size=128256, hidden_size=2048, intermediate_size=8192, num_hidden_layers=16,
                num_attention_heads=32, num_key_value_heads=8, head_dim=64, rope_theta=500000.0,
                rms_norm_eps=1e-5, tie_word_embeddings=True,
                rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                  original_max_position_embeddings=8192))


def rope_inv_freq(cfg):
    """Llama-3 scaled inverse frequencies, float32 arithmetic as transformers' "llama3" rule, returned as float64
    (what src/bitexact/llama.py:52-62 obtains from transformers)."""
    hd = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
    base = cfg["rope_theta"]
    inv = 1.0 / (base ** (torch.arange(0, hd, 2, dtype=torch.int64).to(torch.float) / hd))
    rs = cfg.get("rope_scaling")
    if rs:
        factor, lo, hi, old = rs["factor"], rs["low_freq_factor"], rs["high_freq_factor"], \
            rs["original_max_position_embeddings"]
        low_wl, high_wl = old / lo, old / hi
        wl = 2 * torch.pi / inv
        inv_l = torch.where(wl > low_wl, inv / factor, inv)
        smooth = (old / wl - lo) / (hi - lo)
        smoothed = (1 - smooth) * inv_l / factor + smooth * inv_l
        medium = ~(wl < high_wl) * ~(wl > low_wl)
        inv = torch.where(medium, smoothed, inv_l)
    return inv.double()


def rope_tables(cfg, n_pos=MAX_POS, bits=FT):
    """Integer cos / sin [n_pos, HD / 2] at `bits` fractional bits (float64, rounded once; llama.py:64-69)."""
    ang = torch.arange(n_pos, dtype=torch.float64)[:, None] * rope_inv_freq(cfg)[None, :]
    return torch.round(torch.cos(ang) * 2.0 ** bits).long(), torch.round(torch.sin(ang) * 2.0 ** bits).long()


def embedding_table(emb):
    """bf16 embedding -> int32 at 2^-24, each entry rounded once (consts.py:130-135)."""
    sm, ex = bf16_parts(emb)
    s = ex + FR
    e = torch.where(s >= 0, sm << s.clamp(min=0), (sm + (1 << (-s - 1).clamp(min=0, max=62))) >> (-s).clamp(max=63))
    if int(e.abs().max()) >= 1 << 31:
        raise ValueError("embedding out of int32 range")
    return e.to(torch.int32)


def build(cfg, sd, n_layers=None, tables=None, n_pos=MAX_POS):
    """Constants dict from a HF Llama config dict and state dict (bf16 tensors, any device).
    tables: optional dict with "cos" / "sin" to use instead of computing them."""
    L = cfg["num_hidden_layers"] if n_layers is None else n_layers
    c = {"n_layers": L, "cfg": dict(cfg)}

    def put(name, w):
        for k, v in decompose(w).items():
            c[f"{name}.{k}"] = v

    emb = sd["model.embed_tokens.weight"]
    c["emb"] = embedding_table(emb)
    for i in range(L):
        p = f"model.layers.{i}."
        cat = lambda *ks: torch.cat([sd[p + k] for k in ks])
        put(f"{i}.wqkv", cat("self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight"))
        put(f"{i}.wo", sd[p + "self_attn.o_proj.weight"])
        put(f"{i}.wgu", cat("mlp.gate_proj.weight", "mlp.up_proj.weight"))
        put(f"{i}.wd", sd[p + "mlp.down_proj.weight"])
        for n, k in (("ga", "input_layernorm.weight"), ("gm", "post_attention_layernorm.weight")):
            c[f"{i}.{n}.m"], c[f"{i}.{n}.e"] = bf16_parts(sd[p + k])
    c["gf.m"], c["gf.e"] = bf16_parts(sd["model.norm.weight"])
    put("lm", sd.get("lm_head.weight", emb))
    if tables is None:
        c["cos"], c["sin"] = rope_tables(cfg, n_pos)
    else:
        c["cos"], c["sin"] = tables["cos"], tables["sin"]
    dev = emb.device
    c["cos"], c["sin"] = c["cos"].to(dev), c["sin"].to(dev)
    c["exp2"], c["ln"] = exp2_table(dev), ln_table(FL, dev)
    return c


def digest(c, skip=("cfg", "stats", "sha256")):
    """SHA-256 over every tensor and scalar in key order: the model identity of src/bitexact/llama.py:77-92."""
    import hashlib
    h = hashlib.sha256()
    for k in sorted(c):
        if k in skip:
            continue
        v = c[k]
        h.update(k.encode())
        if torch.is_tensor(v):
            h.update(str(v.dtype).encode())
            h.update(v.contiguous().cpu().numpy().tobytes())
        else:
            h.update(repr(v).encode())
    return h.hexdigest()


def random_state_dict(cfg, seed=0, device="cpu", std=0.02, n_layers=None, gamma_jitter=0.0):
    """Random-init Llama weights as bf16 (N(0, std^2) matrices, gamma = 1 (+ jitter)), generated with numpy's
    legacy RandomState on the host when device == "cpu" (stable across machines) or torch's generator on a GPU."""
    import numpy as np
    D, FF, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    H, HKV = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    HD = cfg.get("head_dim") or D // H
    L = cfg["num_hidden_layers"] if n_layers is None else n_layers
    if str(device) == "cpu":
        rng = np.random.RandomState(seed)
        mat = lambda n, k: torch.from_numpy((rng.standard_normal((n, k)) * std).astype(np.float32)).to(torch.bfloat16)
        vec = lambda n: torch.from_numpy((1.0 + gamma_jitter * rng.standard_normal(n)).astype(np.float32)).to(torch.bfloat16)
    else:
        g = torch.Generator(device=device).manual_seed(seed)
        mat = lambda n, k: (torch.randn(n, k, generator=g, device=device) * std).to(torch.bfloat16)
        vec = lambda n: (1.0 + gamma_jitter * torch.randn(n, generator=g, device=device)).to(torch.bfloat16)
    sd = {"model.embed_tokens.weight": mat(V, D)}
    for i in range(L):
        p = f"model.layers.{i}."
        sd[p + "self_attn.q_proj.weight"] = mat(H * HD, D)
        sd[p + "self_attn.k_proj.weight"] = mat(HKV * HD, D)
        sd[p + "self_attn.v_proj.weight"] = mat(HKV * HD, D)
        sd[p + "self_attn.o_proj.weight"] = mat(D, H * HD)
        sd[p + "mlp.gate_proj.weight"] = mat(FF, D)
        sd[p + "mlp.up_proj.weight"] = mat(FF, D)
        sd[p + "mlp.down_proj.weight"] = mat(D, FF)
        sd[p + "input_layernorm.weight"] = vec(D)
        sd[p + "post_attention_layernorm.weight"] = vec(D)
    sd["model.norm.weight"] = vec(D)
    if not cfg.get("tie_word_embeddings", True):
        sd["lm_head.weight"] = mat(V, D)
    return sd
