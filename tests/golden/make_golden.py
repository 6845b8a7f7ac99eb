"""Generate the golden vectors of tests/golden/ by running the reference implementation itself.

Run once, in a container that has the reference checked out:

    PYTHONPATH=<reference>/src python tests/golden/make_golden.py

It imports `bitexact` (pure Python, CPU paths only), feeds it small seeded inputs and stores inputs
and outputs as compressed .npz files.  The tests never import the reference; they read these files.
"""

import os

import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))       # this repository (weight preparation only)


def n(t):
    return t.detach().cpu().numpy()


def bf16_bits(w):
    return w.contiguous().view(torch.int16).numpy().astype(np.uint16)


def limb_planes(c32, HD):
    """int32 cache [nb, HKV, bs, 2 HD] (K | V) -> int8 limb planes [nb, HKV, bs, 8 HD]."""
    from bitexact.intops import split_limbs
    out = torch.zeros(*c32.shape[:3], 8 * HD, dtype=torch.int8)
    for part, o in ((c32[..., :HD], 0), (c32[..., HD:], 3)):
        for i, lo in enumerate(split_limbs(part, 3)[0]):
            out[..., (o + i) * HD:(o + i + 1) * HD] = lo.to(torch.int8)
    return out


def exact_ops():
    from bitexact.exact import ops, segs
    from bitexact.exact.consts import FR, bf16_parts, decompose
    from bitexact.exact.model import Lin
    from bitexact.exact.segs import lin_y

    out = {}
    g = torch.Generator().manual_seed(11)
    lut = torch.round(torch.pow(2.0, -torch.arange((1 << 14) + 1, dtype=torch.float64) / (1 << 14)) * 2.0 ** 60).long()

    # --- linear with forced residual, ordinary and adversarial shifts ---
    N, K, M = 80, 192, 9
    w = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
    w[0, :5] = torch.tensor([1e-9, -3e-8, 0.0, 2.0, -0.5]).to(torch.bfloat16)
    w[7, 3] = torch.tensor(3e-7).to(torch.bfloat16)
    w[33, :] = 0
    dec = decompose(w)
    c = {f"x.{k}": v for k, v in dec.items() if k != "stats"}
    q = torch.randint(-(1 << 22), (1 << 22) + 1, (M, K), generator=g)
    q[0, :] = 1 << 22
    q[1, :] = -(1 << 22)
    q[2, :] = 0
    sh = torch.tensor([-20, -8, -14, -40, -70, 0, 12, 40, -97])
    lin = Lin(c, "x", "cpu", "cpu", False)
    y, flag = lin_y(*lin(q), sh, True)
    rowflag = [bool(lin_y(*lin(q[m:m + 1]), sh[m:m + 1], True)[1]) for m in range(M)]
    out.update(lin_w=bf16_bits(w), lin_q=n(q), lin_sh=n(sh), lin_y=n(y), lin_flag=np.array(bool(flag)),
               lin_rowflag=np.array(rowflag), lin_limbs=n(dec["limbs"]), lin_g=n(dec["g"]), lin_d=n(dec["d"]),
               lin_rr=n(dec["rr"]), lin_rc=n(dec["rc"]), lin_rv=n(dec["rv"]))

    # --- rms norm + quant ---
    D = 512
    x = torch.randint(-(1 << 27), 1 << 27, (6, D), generator=g)
    x[1] = torch.randint(-3, 4, (D,), generator=g)
    x[2] = 0
    x[3] = torch.randint(-(1 << 38), 1 << 38, (D,), generator=g)
    x[4] = torch.randint(-(1 << 39), 1 << 39, (D,), generator=g)
    gam = (1 + 0.3 * torch.randn(D, generator=g)).to(torch.bfloat16)
    gm, ge = bf16_parts(gam)
    qn, shn, _ = segs.norm_quant(x, gm, ge, torch.zeros((), dtype=torch.bool))
    r, er = ops.rms(x)
    out.update(norm_x=n(x), norm_gm=n(gm), norm_ge=n(ge), norm_q=n(qn), norm_sh=n(shn), norm_r=n(r), norm_er=n(er))

    # --- rope + q quant + k / v ---
    H, HKV, HD = 4, 2, 64
    T = 5
    yq = torch.randint(-(1 << 28), 1 << 28, (T, (H + 2 * HKV) * HD), generator=g)
    yq[4] = torch.randint(-(1 << 10), 1 << 10, ((H + 2 * HKV) * HD,), generator=g)
    pos = torch.tensor([0, 3, 17, 100, 255])
    ang = torch.arange(256, dtype=torch.float64)[:, None] \
        * (500000.0 ** (-torch.arange(0, HD, 2, dtype=torch.float64) / HD))[None]
    cos, sin = torch.round(torch.cos(ang) * 2.0 ** 30).long(), torch.round(torch.sin(ang) * 2.0 ** 30).long()
    Pq, k, v, _ = segs.rope_y(yq, pos.view(T, 1), cos, sin, T, 1, (H, HKV, HD))
    qi, shq = ops.quant(Pq, -(FR + 30))
    out.update(rope_y=n(yq), rope_pos=n(pos), rope_cos=n(cos), rope_sin=n(sin), rope_q=n(qi.view(T, H, HD)),
               rope_sh=n(shq.view(T, H)), rope_k=n(k.view(T, HKV, HD)), rope_v=n(v.view(T, HKV, HD)))

    # --- silu * up + quant ---
    FF = 384
    gu = torch.randint(-(12 << FR), 12 << FR, (4, 2 * FF), generator=g)
    gu[1, :FF] = torch.randint(-(70 << FR), 70 << FR, (FF,), generator=g)
    gu[2] = torch.randint(-(1 << 12), 1 << 12, (2 * FF,), generator=g)
    P, ok = segs.silu_y(gu, lut)
    qs, shs, errs = segs.quant_silu(P, ok, torch.zeros((), dtype=torch.bool))
    out.update(silu_y=n(gu), silu_q=n(qs), silu_sh=n(shs), silu_err=np.array(bool(errs)))

    # --- paged attention (the reference's unfused form: exact products + softmax_w) and attn_out ---
    nb, bs, HKV, HD, G = 40, 16, 2, 64, 4
    c32 = torch.randint(-8355711, 8355712, (nb, HKV, bs, 2 * HD), generator=g).to(torch.int32)
    c32[5:20] = torch.randint(-(1 << 12), 1 << 12, (15, HKV, bs, 2 * HD), generator=g).to(torch.int32)
    R = 4
    bt = torch.stack([torch.randperm(nb - 1, generator=g)[:12] + 1 for _ in range(R)]).to(torch.int32)
    bt[:2, :6] = torch.randint(5, 20, (2, 6), generator=g).to(torch.int32)
    qpos = torch.tensor([[60, 60, 60, 60], [150, 150, 150, 150], [3, 0, 7, 5], [191, 100, 1, 64]])
    qa = torch.randint(-(1 << 22), (1 << 22) + 1, (R, HKV, G, HD), generator=g)
    sha = torch.randint(-40, -10, (R, HKV, G), generator=g)
    S = int(qpos.max()) + 1
    s = torch.arange(S)
    kv = c32[bt.long()[:, s // bs], :, (s % bs)[None].expand(R, -1)].long()
    Kk, Vv = kv[..., :HD].permute(0, 2, 1, 3), kv[..., HD:].permute(0, 2, 1, 3)
    raw = torch.einsum("rhmd,rhsd->rhms", qa, Kk)
    ok = torch.arange(S)[None, None, None] <= qpos[:, None, :, None]
    p, den = ops.softmax_w(raw, ok, sha[..., None], segs.FK, lut, segs.FP, ops.L2E28)
    num = torch.einsum("rhms,rhsd->rhmd", p, Vv)
    o = ops.div_round(num, FR - segs.FV, den)
    qo, sho = ops.quant(o.reshape(R, -1), -FR)
    out.update(attn_cache=n(limb_planes(c32, HD)), attn_bt=n(bt), attn_qpos=n(qpos), attn_q=n(qa), attn_sh=n(sha),
               attn_num=n(num), attn_den=n(den), attn_qo=n(qo), attn_sho=n(sho))
    np.savez_compressed(os.path.join(HERE, "exact_ops.npz"), **out)


def sampler():
    from bitexact import sampling
    from bitexact.llama import ln_table
    g = torch.Generator().manual_seed(5)
    lnt = ln_table(40)
    keys = [(0, 0), (1, 0), (7, 33), (123456, 255)]
    raw = sampling.raw_rows(keys)[:, :2048].contiguous()
    raw[0, :6] = torch.tensor([0, -1, 1 << 11, (1 << 63) - 1, -(1 << 63), 12345 << 11])
    gum = sampling.gumbel(raw, lnt, 24)
    logits = torch.randint(-(30 << 24), 30 << 24, (4, 2048), generator=g)
    logits[2, 100] = logits[2].max() + 5
    logits[2, 900] = logits[2, 100]
    tok_g = sampling.sample(logits, 0, 1)
    tok_t = sampling.sample(logits, 7, 10, gum)
    np.savez_compressed(os.path.join(HERE, "sampler.npz"), keys=np.array(keys), raw=n(raw), gumbel=n(gum),
                        logits=n(logits), tok_greedy=n(tok_g), tok_t07=n(tok_t))


def logp():
    """Integer log p (rl.int_logp) of seeded int64 logits rows at 16 bits: ordinary, peaked, flat and far-below rows."""
    import hashlib
    from bitexact.llama import ln_table
    from bitexact.vllm_plugin import rl
    g = torch.Generator().manual_seed(31)
    lnt = ln_table(40)
    V = 3001
    lg = torch.randint(-(12 << 16), 12 << 16, (7, V), generator=g)
    lg[1] = lg[1] >> 6                                          # a nearly flat row
    lg[2, 17] = 90 << 16                                        # a peaked row: everything else below the table's range
    lg[3] = 5 << 16                                             # all equal
    lg[4, ::3] = -(1 << 40)                                     # far below: the clamp of the table argument
    lg[5, 5] = -(1 << 58)                                       # the target's clamp at -2^36
    lg[6] = lg[6] * 37 + 11                                     # remainders of every size
    tok = torch.tensor([0, 3000, 17, 1234, 3, 5, 77])
    tab = rl.lse_table("cpu")
    lp = rl.int_logp(lg, tok, lnt)
    np.savez_compressed(os.path.join(HERE, "logp.npz"), logits=n(lg), tok=n(tok), logp=n(lp),
                        tab_sha=np.array(hashlib.sha256(n(tab).tobytes()).hexdigest()), tab_sample=n(tab[::997]))


def plan_meta():
    """The step description used for the batch-layout fixture: 7 requests (decodes, prefill chunks of several
    lengths, one request without query tokens), 3 padding rows."""
    from types import SimpleNamespace
    qlen = [1, 5, 1, 0, 17, 5, 1]
    seq = [9, 5, 40, 3, 30, 12, 1]
    qsl = [0]
    for q in qlen:
        qsl.append(qsl[-1] + q)
    n = qsl[-1]
    g = torch.Generator().manual_seed(77)
    bt = torch.randint(1, 50, (len(qlen), 4), generator=g, dtype=torch.int32)
    slot = torch.randint(16, 800, (n + 3,), generator=g)
    pos = torch.cat([torch.arange(s - q, s) for q, s in zip(qlen, seq)] + [torch.zeros(3, dtype=torch.long)])
    meta = SimpleNamespace(query_start_loc=torch.tensor(qsl, dtype=torch.int32), seq_lens=torch.tensor(seq, dtype=torch.int32),
                           block_table=bt, slot_mapping=slot)
    return meta, n + 3, pos


def plan():
    """paged.make_plan / Plan.groups of the reference on plan_meta(), with a small group cap so that the prefill
    requests split into two groups."""
    from bitexact.vllm_plugin import paged
    meta, N, pos = plan_meta()
    out = {}
    for tag, cap in (("a", paged.GROUP_BYTES), ("b", 2 * 17 * 2048 * 8 - 1)):
        paged.GROUP_BYTES = cap
        p = paged.make_plan(meta, N, pos)
        out.update({f"{tag}_n": np.array(p.n), f"{tag}_slot": n(p.slot), f"{tag}_bt": n(p.block_table),
                    f"{tag}_dec_req": n(p.dec_req), f"{tag}_dec_tok": n(p.dec_tok), f"{tag}_pre": np.array(p.pre),
                    f"{tag}_ngroups": np.array(len(p.groups()))})
        for i, gr in enumerate(p.groups()):
            out.update({f"{tag}_g{i}_req": n(gr.req), f"{tag}_g{i}_idx": n(gr.idx), f"{tag}_g{i}_pos": n(gr.pos),
                        f"{tag}_g{i}_valid": n(gr.valid), f"{tag}_g{i}_dst": n(gr.dst)})
    np.savez_compressed(os.path.join(HERE, "plan.npz"), **out)


def int8_ops():
    """int8-mode linear through the reference's CPU path: quant_rows -> imm -> post."""
    from bitexact.int8 import ops as iops
    from bitexact.int8 import segs as isegs
    from bitexact.int8.consts import _q_linear
    from bitexact.intops import stack_limbs
    g = torch.Generator().manual_seed(21)
    N, K, M = 200, 320, 13
    w = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16).double()
    wq, m, fm = _q_linear(w)
    x = torch.round(torch.randn(M, K, generator=g, dtype=torch.float64) * 2 ** 16).long()
    x[0] = 0
    x[1] = torch.randint(-3, 4, (K,), generator=g)
    x[2] = x[2] << 20
    q, mant, e = isegs.pre_plain(x, 2)
    fmsh = fm + 8 - 24
    acc = iops.imm(q, wq.double().t().contiguous())
    y, flag = isegs.post(acc, m, torch.tensor(fmsh), mant, e, True)
    out = dict(w=n(w), wq=n(wq), m=n(m), fm=np.array(fm), x=n(x), q=n(q), mant=n(mant), e=n(e), acc=n(acc), y=n(y),
               flag=np.array(bool(flag)), stacked=n(stack_limbs(q, 2)))
    np.savez_compressed(os.path.join(HERE, "int8_ops.npz"), **out)


TINY = dict(vocab_size=128256, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
            num_key_value_heads=1, head_dim=64, rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
            rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                              original_max_position_embeddings=8192))
TINY_PROMPTS = [[3, 500, 17, 128255, 9], list(range(100000, 100017)), [(7919 * i * i + 3) % 128256 for i in range(40)]]


def tiny_state_dict():
    """The tiny model's weights: numpy RandomState(0) (stable across machines), q / k scaled up so that the
    attention scores matter."""
    from bitexact_llm_b200.exact.consts import random_state_dict
    sd = random_state_dict(TINY, seed=0, std=0.05, gamma_jitter=0.2)
    for i in range(TINY["num_hidden_layers"]):
        for k in ("q_proj", "k_proj"):
            n_ = f"model.layers.{i}.self_attn.{k}.weight"
            sd[n_] = (sd[n_].float() * 4).to(torch.bfloat16)
    return sd


def tiny_model():
    """A 2-layer GQA Llama (head_dim 64, llama3 RoPE scaling) through the reference's constants build and CPU
    engine: tokens and logits hashes for three prompts, greedy and T = 0.7."""
    import tempfile

    from safetensors.torch import save_file
    from transformers import LlamaConfig

    from bitexact.exact.consts import build
    from bitexact.exact.model import ExactLlama
    from bitexact.generate import generate
    from bitexact_llm_b200.exact import consts as myc
    sd = tiny_state_dict()
    with tempfile.TemporaryDirectory() as d:
        LlamaConfig(max_position_embeddings=4096, **TINY).save_pretrained(d)
        save_file({k: v.contiguous() for k, v in sd.items()}, os.path.join(d, "model.safetensors"))
        c = build(d)
    mine = myc.build(TINY, sd)
    for k, v in c.items():                                    # this repo's weight preparation == the reference's
        if torch.is_tensor(v):
            assert torch.equal(v, mine[k]), k
    assert myc.digest(mine) == c["sha256"]
    m = ExactLlama(c, "cpu")
    out = {"sha256": np.array(c["sha256"]), "cos": n(c["cos"][:128]), "sin": n(c["sin"][:128])}
    for pi, prompt in enumerate(TINY_PROMPTS):
        for name, (tn, td) in (("greedy", (0, 1)), ("t07", (7, 10))):
            toks, hashes = generate(m, prompt, 8, tn, td, seed=pi)
            out[f"p{pi}_{name}_tok"] = np.array(toks)
            out[f"p{pi}_{name}_sha"] = np.array(hashes)
    np.savez_compressed(os.path.join(HERE, "tiny_model.npz"), **out)


def tiny_model_int8():
    """The same tiny model through the reference's int8 constants build and CPU engine (IntLlama)."""
    import tempfile

    from safetensors.torch import save_file
    from transformers import LlamaConfig

    from bitexact.generate import generate
    from bitexact.int8.consts import build
    from bitexact.int8.model import IntLlama
    sd = tiny_state_dict()
    with tempfile.TemporaryDirectory() as d:
        LlamaConfig(max_position_embeddings=4096, **TINY).save_pretrained(d)
        save_file({k: v.contiguous() for k, v in sd.items()}, os.path.join(d, "model.safetensors"))
        c = build(d)
    m = IntLlama(c, "cpu")
    out = {"sha256": np.array(c["sha256"]), "cos": n(c["cos"][:128]), "sin": n(c["sin"][:128]),
           "post_check": np.array(bool(m.post_check))}
    for pi, prompt in enumerate(TINY_PROMPTS):
        for name, (tn, td) in (("greedy", (0, 1)), ("t07", (7, 10))):
            toks, hashes = generate(m, prompt, 8, tn, td, seed=pi)
            out[f"p{pi}_{name}_tok"] = np.array(toks)
            out[f"p{pi}_{name}_sha"] = np.array(hashes)
    # a few constants for pinning this repository's int8 weight preparation
    out["wqkv0"] = n(c["0.wqkv"][:64]); out["wqkv0_m"] = n(c["0.wqkv.m"]); out["wqkv0_fm"] = np.array(c["0.wqkv.fm"])
    out["emb_head"] = n(c["emb"][:8]); out["ga0"] = n(c["0.ga"])
    np.savez_compressed(os.path.join(HERE, "tiny_model_int8.npz"), **out)


if __name__ == "__main__":
    exact_ops()
    sampler()
    logp()
    plan()
    int8_ops()
    tiny_model()
    tiny_model_int8()
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))
