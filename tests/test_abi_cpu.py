"""The C-ABI library builds for sm_100a, loads without a GPU and exports every symbol include/bitexact_b200.h
declares; the ctypes table covers them; argument-contract errors are reported without any device call."""

import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared():
    with open(os.path.join(ROOT, "include", "bitexact_b200.h")) as f:
        return sorted(set(re.findall(r"\b(bx_[a-z0-9_]+)\s*\(", f.read())))


def test_library_exports_every_declared_symbol():
    from bitexact_llm_b200 import _native, build
    path = build.build()
    h = ctypes.CDLL(path)
    names = declared()
    assert len(names) >= 16
    for n in names:
        assert hasattr(h, n), n
    assert set(_native.exported_symbols()) == set(names)
    assert _native.lib().bx_version() >= 1


def test_argument_contracts_fail_before_touching_a_device():
    from bitexact_llm_b200 import _native as nv
    lib = nv.lib()
    assert lib.bx_exact_linear(None, 0, None, None, None, None, None, None, None, 0, None, None, None,
                               4, 128, 128, 1, 0, None) == nv.BX_EARG
    assert lib.bx_exact_attention(None, None, None, None, 1, 0, 0, 0, 16, None, 0, 0, 4, None, None, 0, None, None,
                                  1, 8, 4, 64, 0, 0, None) == nv.BX_EARG
    assert lib.bx_sample(None, 0, None, None, None, None, 1, 10, 24, None) == nv.BX_EARG
    assert lib.bx_exact_linear_scratch_bytes(3, 64) == 3 * 3 * 64


def test_no_product_module_imports_the_oracle():
    pkg = os.path.join(ROOT, "bitexact_llm_b200")
    for dp, _, files in os.walk(pkg):
        for f in files:
            if f.endswith(".py"):
                src = open(os.path.join(dp, f)).read()
                assert "import oracle" not in src and "from oracle" not in src, f
