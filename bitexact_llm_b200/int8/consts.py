"""Weight preparation of int8 mode: per-output-channel int8 weights with integer multipliers, integer tables.

Mirrors the reference's `bitexact.int8.consts` (src/bitexact/int8/consts.py:23-92): same keys, same tensors (checked
against the reference's constants SHA-256 in the tests). Build-time float64 math only; nothing float runs later.
"""

import math

import torch

from ..exact.consts import ln_table, rope_tables

FR, FG, FA, FE, FT, FL = 16, 12, 12, 30, 16, 40
SILU_LIM, EXP_MIN, MAX_POS, QMAX_BITS = 32, -32, 2048, 23


def q_linear(w):
    """float64 [N, K] -> (int8 [N, K], int64 multipliers [N], fm) (consts.py:38-47)."""
    amax = w.abs().amax(1).clamp_min(1e-30)
    s = amax / 127.0
    q = torch.round(w / s[:, None]).clamp(-127, 127)
    l1 = q.abs().sum(1)
    worst = float((l1 * s / 127.0).max()) * 2.0 ** QMAX_BITS * 127.0
    fm = min(60, int(math.floor(62 - math.log2(worst))) - 1)
    m = torch.round(s / 127.0 * 2.0 ** fm).long()
    return q.to(torch.int8), m, fm


def exp_table():
    xs = torch.arange(EXP_MIN << FA, 1, dtype=torch.float64) / (1 << FA)
    return torch.round(torch.exp(xs) * (1 << FE)).long()


def silu_table():
    xs = torch.arange(-SILU_LIM << FA, (SILU_LIM << FA) + 1, dtype=torch.float64) / (1 << FA)
    return torch.round(xs / (1.0 + torch.exp(-xs)) * (1 << FR)).long()


def weight_table(lut, fp=20):
    """Attention weight table rsh(exp table, FE - FP) as int32 (src/bitexact/vllm_plugin/tri_paged.py:351-356)."""
    return ((lut + (1 << (FE - fp - 1))) >> (FE - fp)).to(torch.int32).contiguous()


def build(cfg, sd, n_layers=None, tables=None, n_pos=MAX_POS):
    """Constants dict from a HF Llama config dict and state dict (consts.py:56-92)."""
    g = lambda k: sd[k].double()
    L = cfg["num_hidden_layers"] if n_layers is None else n_layers
    c = {"n_layers": L, "cfg": dict(cfg)}
    emb = g("model.embed_tokens.weight")
    if float(emb.abs().max()) >= 2 ** (31 - FR):
        raise ValueError("embedding out of range")
    c["emb"] = torch.round(emb * (1 << FR)).to(torch.int32)
    for i in range(L):
        p = f"model.layers.{i}."
        wqkv = torch.cat([g(p + f"self_attn.{n}_proj.weight") for n in "qkv"])
        wgu = torch.cat([g(p + "mlp.gate_proj.weight"), g(p + "mlp.up_proj.weight")])
        for name, w in [("wqkv", wqkv), ("wo", g(p + "self_attn.o_proj.weight")), ("wgu", wgu),
                        ("wd", g(p + "mlp.down_proj.weight"))]:
            c[f"{i}.{name}"], c[f"{i}.{name}.m"], c[f"{i}.{name}.fm"] = q_linear(w)
        c[f"{i}.ga"] = torch.round(g(p + "input_layernorm.weight") * (1 << FG)).long()
        c[f"{i}.gm"] = torch.round(g(p + "post_attention_layernorm.weight") * (1 << FG)).long()
    c["gf"] = torch.round(g("model.norm.weight") * (1 << FG)).long()
    c["lm"], c["lm.m"], c["lm.fm"] = q_linear(g("lm_head.weight") if "lm_head.weight" in sd else emb)
    c["exp"], c["silu"] = exp_table(), silu_table()
    if tables is None:
        c["cos"], c["sin"] = rope_tables(cfg, n_pos, FT)
    else:
        c["cos"], c["sin"] = tables["cos"], tables["sin"]
    c["ln"] = ln_table(FL)
    return c


def digest(c):
    """SHA-256 identity of an int8 constants dict: every tensor and scalar in key order, the config by name only
    (src/bitexact/int8/consts.py:95-97, src/bitexact/llama.py:77-92)."""
    import hashlib
    h = hashlib.sha256()
    for k in sorted(c):
        if k == "sha256":
            continue
        v = c[k]
        h.update(k.encode())
        if torch.is_tensor(v):
            h.update(str(v.dtype).encode())
            h.update(v.contiguous().cpu().numpy().tobytes())
        elif k != "cfg":
            h.update(repr(v).encode())
    return h.hexdigest()
