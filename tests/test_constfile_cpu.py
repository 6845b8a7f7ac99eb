"""The pickle-free constants file: round trip of a built constants dict (tensors, config, scalars), detection of a
damaged data section and of malformed headers."""

import json
import os
import struct
import sys

import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))


def test_round_trip_and_checks(tmp_path):
    from make_golden import TINY, tiny_state_dict
    from bitexact_llm_b200 import constfile
    from bitexact_llm_b200.exact import consts
    tables = {"cos": torch.zeros(64, 32, dtype=torch.long), "sin": torch.ones(64, 32, dtype=torch.long)}
    c = consts.build(dict(TINY, vocab_size=512), {k: (v[:512] if v.shape[0] == 128256 else v)
                                                    for k, v in tiny_state_dict().items()}, tables=tables, n_pos=64)
    c["empty"] = torch.zeros(0, 3, dtype=torch.int32)
    c["scalar"] = torch.tensor(7)
    p = str(tmp_path / "c.bxc")
    constfile.save(c, p)
    d = constfile.load(p)
    assert set(d) == set(c)
    for k, v in c.items():
        if torch.is_tensor(v):
            assert d[k].dtype == v.dtype and d[k].shape == v.shape and torch.equal(d[k], v), k
        else:
            assert d[k] == json.loads(json.dumps(v)), k
    assert consts.digest(d) == consts.digest(c)
    raw = bytearray(open(p, "rb").read())
    assert b"pickle" not in raw[:16] and raw[:8] == constfile.MAGIC
    raw[-1] ^= 1                                                   # one flipped bit in the data section
    bad = str(tmp_path / "bad.bxc")
    open(bad, "wb").write(raw)
    with pytest.raises(ValueError):
        constfile.load(bad)
    open(bad, "wb").write(b"PK\x03\x04" + bytes(60))               # not this format
    with pytest.raises(ValueError):
        constfile.load(bad)
    (hl,) = struct.unpack("<Q", bytes(raw[8:16]))
    head = json.loads(bytes(raw[16:16 + hl]).decode())
    name = next(iter(head["tensors"]))
    head["tensors"][name]["offset"] = 1 << 40                      # an extent outside the file
    hb = json.dumps(head).encode()
    hb += b" " * ((-(16 + len(hb))) % 64)
    raw[-1] ^= 1
    open(bad, "wb").write(constfile.MAGIC + struct.pack("<Q", len(hb)) + hb + bytes(raw[16 + hl:]))
    with pytest.raises(ValueError):
        constfile.load(bad, verify=False)
