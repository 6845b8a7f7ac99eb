"""A seeded decode-step sample at full model geometry and its CPU result.  Oracle: test infrastructure only.

One decode step of `rows` independent sequences, each at its own context length near `ctx`, against a KV cache
holding seeded keys and values: the shape of the reference's batch verification
(src/bitexact/repro.py:190-212: the same rows alone and inside a batch must give the same bits). The GPU tests
and the benchmark's parity leg load the same sample into the paged cache and compare residual rows, logits and
tokens with what `run_oracle` returns.
"""

import numpy as np

from . import exact as ox
from . import sampler as osamp
from .intrules import I64


def make_sample(cfg, rows=64, ctx=640, seed=0, spread=40):
    """ids [rows], lens [rows] (keys already cached per row, ctx - spread .. ctx + spread), and per row the cached
    k (17 fractional bits) / v (19 bits) as int64 [len, HKV, HD]: rounded N(0, 1) values, clipped to three limbs."""
    rng = np.random.RandomState(seed)
    HKV = cfg["num_key_value_heads"]
    HD = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
    ids = rng.randint(0, cfg["vocab_size"], rows).astype(I64)
    lens = (ctx + rng.randint(-spread, spread + 1, rows)).astype(I64) if spread else np.full(rows, ctx, I64)
    lim = ox.LIM3
    ks = [np.clip(np.rint(rng.standard_normal((int(n), HKV, HD)) * (1 << ox.FK)), -lim, lim).astype(I64) for n in lens]
    vs = [np.clip(np.rint(rng.standard_normal((int(n), HKV, HD)) * (1 << ox.FV)), -lim, lim).astype(I64) for n in lens]
    return {"ids": ids, "lens": lens, "k": ks, "v": vs}


def fill_cache(model, sample, layer_share=True):
    """The oracle model's per-sequence cache holding the sample's keys and values in every layer."""
    cache = model.new_cache(len(sample["ids"]))
    for r in range(len(sample["ids"])):
        for kv in cache[r]:
            kv["k"] = list(sample["k"][r])
            kv["v"] = list(sample["v"][r])
    return cache


def run_oracle(model, sample, want_logits=True):
    """Residual rows int64 [rows, D] after the model's layers and, optionally, the logits [rows, V]."""
    rows = len(sample["ids"])
    x = model.forward(fill_cache(model, sample), sample["ids"].tolist(), [int(n) for n in sample["lens"]],
                      list(range(rows)))
    return (x, model.logits(x)) if want_logits else (x, None)


def oracle_tokens(model, logits, seeds, t, tn, td):
    """Greedy (tn == 0) or Gumbel-max tokens of the logits rows with noise keyed (seeds[r], t)."""
    if tn == 0:
        return osamp.sample(logits, 0, 1)
    V = logits.shape[1]
    g = np.stack([osamp.gumbel(osamp.raw_words(int(s), t, V), model.c["ln"], ox.FR) for s in seeds])
    return osamp.sample(logits, tn, td, g)
