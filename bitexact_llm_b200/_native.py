"""ctypes binding of libbitexact_b200.so (C ABI in include/bitexact_b200.h).

The library is built in-tree by `bitexact_llm_b200.build` (nvcc, sm_100a).  Loading fails loudly when it is
missing: there is deliberately no fallback path.
"""

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_lib", "libbitexact_b200.so")

BX_OK, BX_EARG, BX_ELAUNCH, BX_EDEVICE, BX_ELIMIT = 0, -1, -2, -3, -4
_ERR = {BX_EARG: "argument contract violated (shape / alignment / null pointer)",
        BX_ELAUNCH: "CUDA launch or driver call failed", BX_EDEVICE: "a device-side wait timed out",
        BX_ELIMIT: "request exceeds the fixed capacity of this entry point"}

_lib = None

P, I, L, Z = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_size_t

_SIGNATURES = {
    "bx_version": (I, []),
    "bx_launch_count": (ctypes.c_longlong, []),
    "bx_device_status": (I, []),
    "bx_clear_device_status": (I, []),
    "bx_set_device_status": (I, [I]),
    "bx_i8_tensor_peak": (I, [I, I, P, P]),
    "bx_exact_linear_scratch_bytes": (Z, [I, I]),
    "bx_exact_linear": (I, [P, L, P, P, P, P, P, P, P, I, P, P, P, I, I, I, I, I, P]),
    "bx_exact_linear_planes": (I, [P, P, L, P, P, P, P, P, P, P, I, P, P, I, I, I, I, I, P]),
    "bx_exact_linear_static_max_bytes": (Z, []),
    "bx_exact_linear_static": (I, [P, L, P, P, P, P, P, P, P, I, P, P, I, I, I, I, I, P]),
    "bx_split_limbs": (I, [P, L, P, I, I, P]),
    "bx_int8_mm": (I, [P, P, P, I, I, I, I, P]),
    "bx_int8_linear_post": (I, [P, P, P, L, P, P, P, P, I, I, I, I, I, P]),
    "bx_exact_norm": (I, [I, P, P, P, P, P, P, P, P, P, P, I, I, I, P]),
    "bx_exact_qkv": (I, [P, P, P, P, P, P, L, L, L, I, P, P, P, I, I, I, I, P]),
    "bx_kv_store": (I, [P, L, L, L, I, P, P, L, L, P, L, L, I, I, I, P]),
    "bx_exact_attn_out": (I, [P, P, P, P, P, I, I, I, P]),
    "bx_exact_silu_quant": (I, [P, P, P, P, P, P, I, I, P]),
    "bx_attention_scratch_bytes": (Z, [I, I]),
    "bx_exact_attention_ws": (I, [P, P, P, P, L, L, L, L, I, P, I, L, I, P, P, L, P, P, I, I, I, I, I, I, P, Z, P]),
    "bx_int8_attention_ws": (I, [P, P, P, L, L, L, L, I, P, I, L, I, P, P, P, P, I, I, I, I, I, I, P, Z, P]),
    "bx_exact_attention": (I, [P, P, P, P, L, L, L, L, I, P, I, L, I, P, P, L, P, P, I, I, I, I, I, I, P]),
    "bx_int8_attention": (I, [P, P, P, L, L, L, L, I, P, I, L, I, P, P, P, P, I, I, I, I, I, I, P]),
    "bx_prefill_attention": (I, [P, P, P, P, I, P, L, L, L, L, I, P, I, L, I, P, L, P, P, P, I, I, I, I, P]),
    "bx_int8_norm": (I, [I, P, P, P, P, P, P, P, P, P, I, I, I, P]),
    "bx_int8_qkv": (I, [P, P, P, P, P, P, L, L, L, I, P, P, P, I, I, I, I, P]),
    "bx_int8_attn_out": (I, [P, P, P, P, P, I, I, I, P]),
    "bx_int8_silu_quant": (I, [P, P, P, P, P, P, I, I, P]),
    "bx_int8_flag_end": (I, [P, P, I, P]),
    "bx_int8_silu_prod": (I, [P, P, P, P, P, I, I, P]),
    "bx_int8_quant_rows": (I, [P, P, P, P, P, I, I, P]),
    "bx_int8_post": (I, [P, P, L, P, P, P, P, I, I, I, P]),
    "bx_pcg_raw": (I, [P, P, I, I, P]),
    "bx_pcg_seed_state": (I, [P, P, I, P]),
    "bx_pcg_raw_from_state": (I, [P, P, I, I, P]),
    "bx_exact_rms": (I, [P, P, P, P, I, I, P]),
    "bx_exact_ndiv": (I, [P, P, P, P, P, P, I, I, P]),
    "bx_rowmax_abs": (I, [P, P, I, I, P]),
    "bx_exact_rope": (I, [P, P, P, P, P, P, P, I, I, I, I, P]),
    "bx_softmax_w": (I, [P, P, P, P, P, L, P, P, P, I, I, P]),
    "bx_exact_attn_div": (I, [P, P, P, I, I, P]),
    "bx_int8_post_acc": (I, [P, P, L, P, P, P, P, I, I, I, P]),
    "bx_exact_silu_prod": (I, [P, P, P, P, P, I, I, P]),
    "bx_exact_quant_rows": (I, [P, P, I, P, L, P, P, L, I, I, P]),
    "bx_bmm": (I, [P, I, P, I, P, I, I, I, I, L, L, L, L, L, L, P]),
    "bx_bmm_limb_scratch_bytes": (Z, [I, I, I, I]),
    "bx_bmm_limb": (I, [P, I, P, I, P, I, I, I, I, L, L, L, L, L, L, P, I, P]),
    "bx_exact_epilogue": (I, [P, P, P, L, P, P, P, I, P, P, P, P, P, I, I, I, P]),
    "bx_sample_scratch_bytes": (Z, [I, I]),
    "bx_sample": (I, [P, L, P, P, P, P, I, I, I, P]),
    "bx_sample_shard": (I, [P, L, P, P, P, P, P, I, I, L, I, P]),
    "bx_decompose_rows": (I, [P, L, P, P, P, P, P, I, I, P]),
    "bx_decompose_residual": (I, [P, L, P, P, P, P, P, P, I, I, P]),
    "bx_logp_scratch_bytes": (Z, [I, I]),
    "bx_logp_pair_table": (I, [P, I, P, P]),
    "bx_int_logp": (I, [P, L, P, P, P, I, P, P, I, I, I, P]),
    "bx_logp_rowmax": (I, [P, L, P, P, I, I, P]),
    "bx_logp_rowsum": (I, [P, L, P, P, I, P, P, I, I, I, P]),
    "bx_logp_finish": (I, [P, P, P, P, I, I, P]),
}


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m bitexact_llm_b200.build` "
                               "(nvcc, sm_100a). There is no fallback path.")
        h = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(h, name)                       # AttributeError if the library is stale
            fn.restype, fn.argtypes = res, args
        _lib = h
    return _lib


def exported_symbols():
    return sorted(_SIGNATURES)


def check(rc, what):
    if rc != BX_OK:
        raise RuntimeError(f"{what}: {_ERR.get(rc, rc)}")


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()


def stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


def device_status():
    """Number of device-side waits that gave up since the last clear (synchronises the device)."""
    return lib().bx_device_status()


def clear_device_status():
    check(lib().bx_clear_device_status(), "bx_clear_device_status")


def i8_tensor_peak(iters=1 << 17, repeats=5):
    """(best, mean) int8 TOPS of a shared-memory-resident tcgen05 kind::i8 loop on the current device."""
    import torch
    out = (ctypes.c_double * 2)()
    check(lib().bx_i8_tensor_peak(iters, repeats, ctypes.cast(out, ctypes.c_void_p), stream()), "bx_i8_tensor_peak")
    torch.cuda.synchronize()
    return out[0], out[1]


class DeviceWaitError(RuntimeError):
    """A bounded device-side wait gave up: kernels launched since then may have left their outputs unwritten."""


def check_device_status():
    """Raises DeviceWaitError when the device status word is non-zero (the state stays set until
    `clear_device_status`)."""
    n = device_status()
    if n != 0:
        raise DeviceWaitError(f"{n} device-side wait(s) timed out: results since then are not valid; "
                              "call clear_device_status() and rerun the step")
