"""int8 mode on a flattened token batch and the paged limb-plane KV cache: the decode / prefill-row path of the
reference's plugin (src/bitexact/vllm_plugin/graph.py:69-87 `_decode_fused`, vllm_plugin/paged.py) with the model
rules of `IntLlama` (src/bitexact/int8/model.py:25-133). Nine kernels per layer: fused int8 linear (GEMM + post),
qkv, attention, attn_out, linear, add_norm, linear, silu_quant, linear, add_norm."""

import torch

from .. import _native as nv
from ..vllm_plugin import tri_fuse, tri_paged, tri_prefill
from .gemm_skinny import linear_post


class IntEngine:
    FR = 16

    def __init__(self, c, dev="cuda", n_layers=None, nl=2):
        assert nl == 2
        self.dev = torch.device(dev)
        cfg = c.get("cfg", {})
        self.D = cfg.get("hidden_size", 2048)
        self.H = cfg.get("num_attention_heads", 32)
        self.HKV = cfg.get("num_key_value_heads", 8)
        self.HD = cfg.get("head_dim") or self.D // self.H
        self.L = c["n_layers"] if n_layers is None else n_layers
        t = lambda k: c[k].to(self.dev).contiguous()
        self.emb = t("emb")
        self.V = self.emb.shape[0]
        lin = lambda k: (t(k), t(f"{k}.m"), int(c[f"{k}.fm"]) + 8 * (nl - 1) - 24)
        self.layers = [{"ga": t(f"{i}.ga"), "gm": t(f"{i}.gm"), **{n: lin(f"{i}.{n}") for n in ("wqkv", "wo", "wgu", "wd")}}
                       for i in range(self.L)]
        self.gf, self.lm = t("gf"), lin("lm")
        self.silu_t, self.cos, self.sin, self.ln = t("silu"), t("cos"), t("sin"), t("ln")
        self.ptab = tri_paged.weight_table(t("exp"))
        self.fl = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.scr = torch.zeros(self.L, 2, dtype=torch.long, device=self.dev)
        self.timer = None                                    # optional callable(M, N, K) -> context manager

    def check(self):
        """OverflowError on a flagged integer bound; `_native.DeviceWaitError` when a device-side wait gave up."""
        nv.check_device_status()
        if bool(self.fl.item()):
            raise OverflowError("integer bound violated (int8 mode)")

    def _lin(self, pre, lin):
        if self.timer is not None:
            with self.timer(pre[1].shape[0], lin[0].shape[0], lin[0].shape[1]):
                return linear_post(pre[0], lin[0], lin[1], lin[2], pre[1], pre[2], self.fl, True)
        return linear_post(pre[0], lin[0], lin[1], lin[2], pre[1], pre[2], self.fl, True)

    def forward(self, kvs, ids, pos, slot, bt, rmap, tiles=None):
        """Same contract as ExactEngine.forward; returns the residual stream int64 [N, D] at 16 bits."""
        fz = tri_fuse
        N, G = ids.shape[0], self.H // self.HKV
        pos = pos.long()
        slot = torch.where(slot < 0, torch.zeros_like(slot), slot).long()
        qpos = pos.view(-1, 1).expand(-1, G).contiguous()
        x, *pre = fz.embed_norm(self, ids, self.layers[0]["ga"])
        for i in range(self.L):
            ly = self.layers[i]
            q = fz.qkv(self, self._lin(pre, ly["wqkv"]), None, None, None, pos, slot, kvs[i], int32=True)
            if tiles is not None:
                num = torch.zeros(N, self.HKV, G, self.HD, dtype=torch.long, device=self.dev)
                den = torch.ones(N, self.HKV, G, 1, dtype=torch.long, device=self.dev)    # padding rows: 0 / 1
                tri_prefill.attend(q, pos, kvs[i], bt, self.ptab, tiles, num, den)
            else:
                num, den = tri_paged.attend(q, qpos, kvs[i], bt, self.ptab, rmap=rmap)
            x, *pre = fz.add_norm(self, self._lin(fz.attn_out(self, num, den), ly["wo"]), None, None, None, x, ly["gm"])
            a8, mant, e, _ = fz.silu_quant(self, self._lin(pre, ly["wgu"]), None, None, None, self.silu_t, scr=self.scr[i])
            nxt = self.layers[i + 1]["ga"] if i + 1 < self.L else None
            x, *pre = fz.add_norm(self, self._lin((a8, mant, e), ly["wd"]), None, None, None, x, nxt)
        fz.flag_end(self, self.scr)
        return x

    def logits(self, h):
        """Final residual rows [M, D] -> int64 logits [M, V] at 16 bits."""
        return self._lin(tri_fuse.pre_norm(self, h, self.gf), self.lm)
