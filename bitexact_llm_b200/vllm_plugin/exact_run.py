"""Exact mode on a flattened token batch and the paged limb-plane KV cache: drop-in for
`bitexact.vllm_plugin.exact_run.ExactEngine` (src/bitexact/vllm_plugin/exact_run.py:23-143).

Every token is a row: its K / V are stored into the paged cache and it attends its own keys through its
request's block table. Nine kernels per layer (linear, qkv, attention, attn_out, linear, add_norm, linear,
silu_quant, linear, add_norm), device tensors only, no host synchronisation inside a step."""

import torch

from .. import _native as nv
from ..exact.model import Lin
from . import exact_fuse, tri_exact_attn, tri_prefill
from .exact_gemm import FusedLin

L2E28_HD = {64: 387270501, 128: 273841598}        # src/bitexact/exact/ops.py:19-20


class ExactEngine:
    FR = 24

    def __init__(self, c, dev="cuda", n_layers=None):
        self.dev = torch.device(dev)
        cfg = c.get("cfg", {})
        self.D = cfg.get("hidden_size", 2048)
        self.H = cfg.get("num_attention_heads", 32)
        self.HKV = cfg.get("num_key_value_heads", 8)
        self.HD = cfg.get("head_dim") or self.D // self.H
        self.FF = cfg.get("intermediate_size", 8192)
        self.L = c["n_layers"] if n_layers is None else n_layers
        t = lambda k: c[k].to(self.dev).contiguous()
        self.emb = t("emb")
        self.V = self.emb.shape[0]
        assert self.emb.shape[1] == self.D
        self.layers = []
        for i in range(self.L):
            ly = {n: FusedLin(Lin(c, f"{i}.{n}", self.dev)) for n in ("wqkv", "wo", "wgu", "wd")}
            for n in ("ga", "gm"):
                ly[n] = (t(f"{i}.{n}.m"), t(f"{i}.{n}.e"))
            self.layers.append(ly)
        self.gf = (t("gf.m"), t("gf.e"))
        self.lm = FusedLin(Lin(c, "lm", self.dev))
        self.cos, self.sin, self.exp2, self.ln = t("cos"), t("sin"), t("exp2"), t("ln")
        self.l2e = L2E28_HD[self.HD]
        self.fl = torch.zeros(1, dtype=torch.int32, device=self.dev)     # sticky bound flag of every kernel

    @property
    def err(self):
        return self.fl != 0

    def check(self):
        """Raises OverflowError when any kernel flagged an integer bound (src/bitexact/exact/model.py:155-157).
        Also raises `_native.DeviceWaitError` when a bounded device-side wait gave up since the last clear: the
        kernels launched after that left their outputs unwritten. Synchronises with the device."""
        nv.check_device_status()
        if bool(self.fl.item()):
            raise OverflowError("integer bound violated (exact mode)")

    def forward(self, kvs, ids, pos, slot, bt, rmap, tiles=None):
        """ids, pos, slot [N]: the step's tokens (slot < 0: padding, written to the null block 0); kvs: list of the
        per-layer caches int8 [nb, HKV, bs, 8 HD]; bt [*, nblk] block table, rmap [N] the table row of each token.
        tiles (int32 [T, 3] on the device: block-table row, first token row, tokens; `tri_prefill.tile_table`):
        prompt processing, runs of consecutive tokens of one request attend through the tile kernel (same integers).
        Returns the residual stream int64 [N, D] at 24 bits."""
        fl, fz = self.fl, exact_fuse
        N, G = ids.shape[0], self.H // self.HKV
        pos = pos.long()
        slot = torch.where(slot < 0, torch.zeros_like(slot), slot).long()
        qpos = pos.view(-1, 1).expand(-1, G).contiguous()
        x, q, sh = fz.embed_norm(self, ids.long(), self.layers[0]["ga"], fl)
        for i in range(self.L):
            ly = self.layers[i]
            qq, shq = fz.qkv(self, ly["wqkv"](q, sh, fl, False), pos, slot, kvs[i], fl)
            if tiles is not None:
                num, den = tri_prefill.attend_exact(qq.view(N, self.HKV, G, self.HD), shq.view(N, self.HKV, G), pos,
                                                    kvs[i], bt, tiles, self.exp2, self.l2e)
            else:
                num, den = tri_exact_attn.attend(qq.view(N, self.HKV, G, self.HD), shq.view(N, self.HKV, G), qpos,
                                                 kvs[i], bt, rmap, self.exp2, self.l2e)
            qo, sho = fz.attn_out(self, num, den)
            x, q, sh = fz.add_norm(self, ly["wo"](qo, sho, fl, True), x, ly["gm"], fl)
            q, sh = fz.silu_quant(self, ly["wgu"](q, sh, fl, False), self.exp2, fl)
            nxt = self.layers[i + 1]["ga"] if i + 1 < self.L else None
            x, q, sh = fz.add_norm(self, ly["wd"](q, sh, fl, True), x, nxt, fl)
        return x

    def logits(self, h):
        """Final residual rows [M, D] -> int64 logits [M, V] at 24 bits."""
        q, sh = exact_fuse.pre_norm(self, h, self.gf, self.fl)
        return self.lm(q, sh, self.fl, True)
