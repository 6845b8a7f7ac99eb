"""CPU oracle for the bitexact integer hot path.  TEST INFRASTRUCTURE ONLY.

This package restates, in numpy int64 arithmetic, the integer rules of the reference
implementation (mynotwo/bitexact-llm, `src/bitexact/...`).  Each function cites the
reference file:line it follows.  It exists to check the CUDA kernels of
`bitexact_llm_b200`; it is never imported by the product package, only by `tests/`,
by `__graft_entry__.smoke()` and by the CPU-baseline / reference legs of `bench.py`.

Parity is pinned: `tests/test_oracle_pins.py` checks this oracle against
  * the reference's known-answer transcript hash (`tests/test_repro.py:126`),
  * Python-integer / Fraction restatements of the reference's unit tests,
  * golden vectors under `tests/golden/` produced by importing the reference itself
    (`tests/golden/make_golden.py`).
"""
