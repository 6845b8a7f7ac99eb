"""Whole-model checks on the CPU: this repository's weight preparation reproduces the reference's constants
(SHA-256 recorded by tests/golden/make_golden.py), and the oracle's forward reproduces the tokens and logits
hashes the reference's CPU engine generated for the tiny model."""

import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def tiny_constants(use_golden_tables=True):
    from make_golden import TINY, tiny_state_dict
    from bitexact_llm_b200.exact import consts
    z = np.load(os.path.join(GOLD, "tiny_model.npz"))
    c = consts.build(TINY, tiny_state_dict())
    return c, z


def test_weight_preparation_reproduces_reference_constants():
    from bitexact_llm_b200.exact import consts
    c, z = tiny_constants()
    assert consts.digest(c) == str(z["sha256"])
    assert np.array_equal(c["cos"][:128].numpy(), z["cos"]) and np.array_equal(c["sin"][:128].numpy(), z["sin"])


def test_rope_rule_matches_transformers():
    from make_golden import TINY
    from transformers import LlamaConfig
    from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
    from bitexact_llm_b200.exact import consts
    for cfg in (TINY, consts.LLAMA_1B):
        hf = LlamaConfig(max_position_embeddings=131072, **cfg)
        try:
            inv, scale = ROPE_INIT_FUNCTIONS["llama3"](hf, "cpu")
        except TypeError:
            inv, scale = ROPE_INIT_FUNCTIONS["llama3"](hf, torch.device("cpu"), None)
        assert scale == 1.0 and torch.equal(inv.double(), consts.rope_inv_freq(cfg))


def test_oracle_model_reproduces_reference_generation():
    from make_golden import TINY_PROMPTS
    from oracle.model import OracleModel, generate
    c, z = tiny_constants()
    m = OracleModel({k: (v.numpy() if torch.is_tensor(v) else v) for k, v in c.items()})
    for pi in (0, 1):
        for name, (tn, td) in (("greedy", (0, 1)), ("t07", (7, 10))):
            toks, shas = generate(m, TINY_PROMPTS[pi], 4, tn, td, seed=pi)
            assert toks == z[f"p{pi}_{name}_tok"][:4].tolist(), (pi, name)
            assert shas == z[f"p{pi}_{name}_sha"][:4].tolist(), (pi, name)
    assert not m.flag


def test_int8_weight_preparation_and_oracle_model_reproduce_the_reference():
    from make_golden import TINY, TINY_PROMPTS, tiny_state_dict
    from bitexact_llm_b200.int8 import consts
    from oracle.model import OracleInt8Model, generate
    z = np.load(os.path.join(GOLD, "tiny_model_int8.npz"))
    c = consts.build(TINY, tiny_state_dict())
    assert consts.digest(c) == str(z["sha256"])
    m = OracleInt8Model({k: (v.numpy() if torch.is_tensor(v) else v) for k, v in c.items()})
    for pi in (0, 1):
        for name, (tn, td) in (("greedy", (0, 1)), ("t07", (7, 10))):
            toks, shas = generate(m, TINY_PROMPTS[pi], 3, tn, td, seed=pi)
            assert toks == z[f"p{pi}_{name}_tok"][:3].tolist(), (pi, name)
            assert shas == z[f"p{pi}_{name}_sha"][:3].tolist(), (pi, name)
    assert not m.flag
