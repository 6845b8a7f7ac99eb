"""Exact-mode Llama forward on the CPU, composed from the oracle's stages.  Oracle: test infrastructure only.

Follows the reference's token-row engine (src/bitexact/vllm_plugin/exact_run.py:55-143), which computes the same
integers as the standalone model (src/bitexact/exact/model.py:106-150): every token is a row with its own keys.
Here the KV "cache" is a plain per-sequence list; weights come as a constants dict with numpy arrays under the
reference's keys (`{i}.wqkv.limbs`, ..., `emb`, `cos`, `sin`, `exp2`, `ln`).
"""

import hashlib

import numpy as np

from . import exact as ox
from . import sampler as osamp
from .intrules import I64, i64


def _lin(c, name):
    return {k: np.asarray(c[f"{name}.{k}"]) for k in ("limbs", "g", "d", "rr", "rc", "rv")}


class OracleModel:
    def __init__(self, c):
        cfg = c["cfg"]
        self.D, self.H, self.HKV = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
        self.HD = cfg.get("head_dim") or self.D // self.H
        self.L = c["n_layers"]
        self.c = {k: (np.asarray(v) if hasattr(v, "shape") else v) for k, v in c.items()}
        self.lin = {(i, n): _lin(self.c, f"{i}.{n}") for i in range(self.L) for n in ("wqkv", "wo", "wgu", "wd")}
        self.lm = _lin(self.c, "lm")
        self.flag = False

    def new_cache(self, B):
        return [[{"k": [], "v": []} for _ in range(self.L)] for _ in range(B)]

    def forward(self, cache, ids, pos, seq):
        """ids, pos, seq: per token row (token id, position, sequence index). Rows of one sequence must be in
        position order. Returns the residual stream int64 [N, D]."""
        c, H, HKV, HD = self.c, self.H, self.HKV, self.HD
        G = H // HKV
        N = len(ids)
        x = i64(c["emb"][np.asarray(ids)])
        q, sh, f = ox.norm_quant(x, c["0.ga.m"], c["0.ga.e"])
        self.flag |= f
        for i in range(self.L):
            y, _ = ox.linear(q, sh, self.lin[i, "wqkv"], checked=True)
            qq, shq, k, v, f = ox.rope_qkv(y, np.asarray(pos), c["cos"], c["sin"], H, HKV, HD)
            self.flag |= f
            num = np.zeros((N, H, HD), dtype=I64)
            den = np.zeros((N, H, 1), dtype=I64)
            for n in range(N):
                kv = cache[seq[n]][i]
                assert len(kv["k"]) == pos[n], "rows of a sequence must arrive in position order"
                kv["k"].append(k[n]), kv["v"].append(v[n])
                K = np.stack(kv["k"], 1)                                   # [HKV, S, HD]
                V = np.stack(kv["v"], 1)
                qg = qq[n].reshape(HKV, G, HD)
                raw = np.einsum("hgd,hsd->hgs", qg, K)
                p, dn = ox.softmax_w(raw, np.ones_like(raw, dtype=bool), shq[n].reshape(HKV, G, 1), c["exp2"],
                                     ox.L2E28_HD[HD])
                num[n] = np.einsum("hgs,hsd->hgd", p, V).reshape(H, HD)
                den[n] = dn.reshape(H, 1)
            qo, sho = ox.attn_out(num, den)
            y, f = ox.linear(qo, sho, self.lin[i, "wo"], checked=True)
            self.flag |= f
            x = x + y
            q, sh, f = ox.norm_quant(x, c[f"{i}.gm.m"], c[f"{i}.gm.e"])
            self.flag |= f
            y, _ = ox.linear(q, sh, self.lin[i, "wgu"], checked=True)
            q, sh, f = ox.silu_quant(y, c["exp2"])
            self.flag |= f
            y, f = ox.linear(q, sh, self.lin[i, "wd"], checked=True)
            self.flag |= f
            x = x + y
            if i + 1 < self.L:
                q, sh, f = ox.norm_quant(x, c[f"{i + 1}.ga.m"], c[f"{i + 1}.ga.e"])
                self.flag |= f
        return x

    def logits(self, h):
        q, sh, f = ox.norm_quant(h, self.c["gf.m"], self.c["gf.e"])
        y, f2 = ox.linear(q, sh, self.lm, checked=True)
        self.flag |= f | f2
        return y


def logits_sha(row):
    return hashlib.sha256(np.ascontiguousarray(row, dtype=I64).tobytes()).hexdigest()


def generate(model, prompt, max_new, tn=0, td=1, seed=0):
    """One prompt: prefill, then max_new tokens; generated token t uses noise keyed (seed, t)
    (src/bitexact/generate.py:34-50). Returns (tokens, logits hashes)."""
    cache = model.new_cache(1)
    P = len(prompt)
    h = model.forward(cache, list(prompt), list(range(P)), [0] * P)[-1:]
    toks, shas = [], []
    V = model.c["emb"].shape[0]
    for t in range(max_new):
        lg = model.logits(h)
        g = osamp.gumbel(osamp.raw_words(seed, t, V), model.c["ln"], getattr(model, "FR", ox.FR))[None] if tn else None
        y = int(osamp.sample(lg, tn, td, g)[0])
        toks.append(y)
        shas.append(logits_sha(lg[0]))
        if t + 1 < max_new:
            h = model.forward(cache, [y], [P + t], [0])
    return toks, shas


class OracleInt8Model:
    """int8-mode forward on the CPU from the oracle's int8 stages (src/bitexact/int8/model.py:69-124, in the
    token-row form of the plugin). Constants dict with numpy arrays under the reference's int8 keys."""

    FR = 16

    def __init__(self, c):
        from . import int8 as o8
        self.o8 = o8
        cfg = c["cfg"]
        self.D, self.H, self.HKV = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
        self.HD = cfg.get("head_dim") or self.D // self.H
        self.L = c["n_layers"]
        self.c = {k: (np.asarray(v) if hasattr(v, "shape") else v) for k, v in c.items()}
        self.flag = False

    def _lin(self, pre, name, x=None):
        o8, c = self.o8, self.c
        q, mant, e = pre
        y, f = o8.post(o8.imm(q, c[name]), c[f"{name}.m"], int(c[f"{name}.fm"]) + 8 - 24, mant, e)
        self.flag |= f
        return y if x is None else x + y

    def new_cache(self, B):
        return [[{"k": [], "v": []} for _ in range(self.L)] for _ in range(B)]

    def forward(self, cache, ids, pos, seq):
        o8, c, H, HKV, HD = self.o8, self.c, self.H, self.HKV, self.HD
        G = H // HKV
        N = len(ids)
        x = i64(c["emb"][np.asarray(ids)])
        for i in range(self.L):
            y = self._lin(o8.pre_norm(x, c[f"{i}.ga"]), f"{i}.wqkv")
            q, k, v, f = o8.rope_qkv(y, np.asarray(pos), c["cos"], c["sin"], H, HKV, HD)
            self.flag |= f
            num = np.zeros((N, H, HD), dtype=I64)
            den = np.zeros((N, H, 1), dtype=I64)
            for n in range(N):
                kv = cache[seq[n]][i]
                assert len(kv["k"]) == pos[n]
                kv["k"].append(k[n]), kv["v"].append(v[n])
                K, V = np.stack(kv["k"], 1), np.stack(kv["v"], 1)
                raw = np.einsum("hgd,hsd->hgs", q[n].reshape(HKV, G, HD), K)
                p, dn = o8.softmax(raw, np.ones_like(raw, dtype=bool), c["exp"])
                num[n] = np.einsum("hgs,hsd->hgd", p, V).reshape(H, HD)
                den[n] = dn.reshape(H, 1)
            x = self._lin(o8.attn_out(num, den), f"{i}.wo", x)
            gu = self._lin(o8.pre_norm(x, c[f"{i}.gm"]), f"{i}.wgu")
            a, mant, e, f = o8.silu_mul(gu, c["silu"])
            self.flag |= f
            x = self._lin((a, mant, e), f"{i}.wd", x)
        self.flag |= bool(np.abs(x).max(initial=0) >= 1 << 42)
        return x

    def logits(self, h):
        return self._lin(self.o8.pre_norm(h, self.c["gf"]), "lm")
