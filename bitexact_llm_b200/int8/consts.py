"""Weight preparation of int8 mode: int8 weights with one integer multiplier per output channel, integer tables.

Produces the constants dict of the reference's `bitexact.int8.consts.build` (src/bitexact/int8/consts.py:23-92) —
same keys, same tensors; `tests/golden/make_golden.py` compares them tensor for tensor with the reference's.
The float64 expressions are evaluated in the reference's order because the rounded integers must come out
identical; everything after this load-time step is integer arithmetic.
"""

import math

import torch

from ..exact.consts import ln_table, rope_tables

FR, FG, FA, FE, FT, FL = 16, 12, 12, 30, 16, 40      # residual, gamma, table argument, exp, cos / sin, ln (bits)
SILU_LIM, EXP_MIN, MAX_POS, QMAX_BITS = 32, -32, 2048, 23

# (key in the constants dict, the state-dict matrices stacked along the output dimension)
_LAYER_MATRICES = (("wqkv", ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj")),
                   ("wo", ("self_attn.o_proj",)),
                   ("wgu", ("mlp.gate_proj", "mlp.up_proj")),
                   ("wd", ("mlp.down_proj",)))
_LAYER_GAMMAS = (("ga", "input_layernorm"), ("gm", "post_attention_layernorm"))


def multiplier_bits(bound):
    """Fractional bits of the channel multipliers: the most (at most 60) that keep acc * m below 2^61 when the
    largest |acc| * scale over all channels, against activations of QMAX_BITS bits, is `bound`."""
    return min(60, int(math.floor(62 - math.log2(bound))) - 1)


def q_linear(w):
    """Per-channel symmetric quantisation of a float64 matrix [N, K] (consts.py:38-47): int8 weights
    round(w / step) with step = max |row| / 127, the multipliers round(step / 127 * 2^fm) as int64 [N], and fm."""
    peak = w.abs().amax(1).clamp_min(1e-30)
    step = peak / 127.0
    w8 = torch.round(w / step[:, None]).clamp(-127, 127)
    bound = float((w8.abs().sum(1) * step / 127.0).max()) * 2.0 ** QMAX_BITS * 127.0
    fm = multiplier_bits(bound)
    return w8.to(torch.int8), torch.round(step / 127.0 * 2.0 ** fm).long(), fm


def exp_table():
    """e^x at FE bits, x from EXP_MIN to 0 in steps of 2^-FA."""
    x = torch.arange(EXP_MIN << FA, 1, dtype=torch.float64) / (1 << FA)
    return torch.round(torch.exp(x) * (1 << FE)).long()


def silu_table():
    """x sigmoid(x) at FR bits, x from -SILU_LIM to SILU_LIM in steps of 2^-FA."""
    x = torch.arange(-SILU_LIM << FA, (SILU_LIM << FA) + 1, dtype=torch.float64) / (1 << FA)
    return torch.round(x / (1.0 + torch.exp(-x)) * (1 << FR)).long()


def weight_table(lut, fp=20):
    """Attention weight table rsh(exp table, FE - FP) as int32 (src/bitexact/vllm_plugin/tri_paged.py:351-356)."""
    return ((lut + (1 << (FE - fp - 1))) >> (FE - fp)).to(torch.int32).contiguous()


def _put_linear(c, key, w):
    c[key], c[f"{key}.m"], c[f"{key}.fm"] = q_linear(w)


def _gamma(v):
    return torch.round(v.double() * (1 << FG)).long()


def build(cfg, sd, n_layers=None, tables=None, n_pos=MAX_POS):
    """Constants dict from a HF Llama config dict and state dict (bf16 or float tensors, any device)."""
    L = cfg["num_hidden_layers"] if n_layers is None else n_layers
    emb = sd["model.embed_tokens.weight"].double()
    if float(emb.abs().max()) >= 2 ** (31 - FR):
        raise ValueError("embedding out of range")
    c = {"n_layers": L, "cfg": dict(cfg), "emb": torch.round(emb * (1 << FR)).to(torch.int32)}
    for i in range(L):
        prefix = f"model.layers.{i}."
        for key, parts in _LAYER_MATRICES:
            _put_linear(c, f"{i}.{key}", torch.cat([sd[f"{prefix}{p}.weight"].double() for p in parts]))
        for key, name in _LAYER_GAMMAS:
            c[f"{i}.{key}"] = _gamma(sd[f"{prefix}{name}.weight"])
    c["gf"] = _gamma(sd["model.norm.weight"])
    _put_linear(c, "lm", sd["lm_head.weight"].double() if "lm_head.weight" in sd else emb)
    c["exp"], c["silu"], c["ln"] = exp_table(), silu_table(), ln_table(FL)
    c["cos"], c["sin"] = rope_tables(cfg, n_pos, FT) if tables is None else (tables["cos"], tables["sin"])
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
