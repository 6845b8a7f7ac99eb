"""bitexact_llm_b200: the integer hot path of the bit-exact Llama engine as hand-written sm_100a CUDA kernels.

The package mirrors the reference's module names for the path it replaces (`exact`, `int8`, `vllm_plugin`)
and calls `libbitexact_b200.so` through its C ABI (`include/bitexact_b200.h`).  There is no CPU or PyTorch
fallback: importing a compute entry point without the built library raises.
"""

__version__ = "0.1.0"
