"""Error reporting of the engines: the sticky arithmetic-bound flag must surface as OverflowError from check()
(the reference's tests/vllm/test_overflow_check.py:19-48 and tests/test_tri_fuse.py:117-130), and the device status
word of the bounded waits must surface as DeviceWaitError / BX_EDEVICE. The status word is written from the host
(bx_set_device_status): no wait is made to run out on the device."""

import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def engines():
    from make_golden import TINY, tiny_state_dict
    from bitexact_llm_b200.exact import consts
    from bitexact_llm_b200.int8 import consts as consts8
    from bitexact_llm_b200.int8.engine import IntEngine
    from bitexact_llm_b200.vllm_plugin.exact_run import ExactEngine
    sd = tiny_state_dict()
    return ExactEngine(consts.build(TINY, sd, n_pos=64), "cuda"), IntEngine(consts8.build(TINY, sd, n_pos=64), "cuda")


def test_exact_engine_check_raises_after_a_kernel_set_the_flag(engines):
    eng, _ = engines
    eng.check()                                                   # clean engine: no error
    lin = eng.layers[0]["wqkv"]
    q = torch.full((2, lin.K), 1 << 22, dtype=torch.int32, device="cuda")
    sh = torch.tensor([-30, 60], device="cuda")                   # row 1: the rounding shift leaves the int64 range
    lin(q, sh, eng.fl, True)
    with pytest.raises(OverflowError):
        eng.check()
    eng.fl.zero_()
    eng.check()
    lin(q, sh, eng.fl, False)                                     # unchecked calls never touch the flag
    eng.check()


def test_int8_engine_check_raises_after_a_kernel_set_the_flag(engines):
    from bitexact_llm_b200.int8.gemm_skinny import linear_post
    _, eng = engines
    eng.check()
    w, mul, _ = eng.layers[0]["wqkv"]
    K = w.shape[1]
    a = torch.full((24, K), 127, dtype=torch.int8, device="cuda")
    mant = torch.full((2,), 1 << 23, device="cuda")
    e = torch.full((2,), -20, device="cuda")
    big = torch.full_like(mul, 1 << 20)
    linear_post(a, torch.full_like(w, 127), big, 0, mant, e, eng.fl, True, M=2)   # |t| >= 2^38
    with pytest.raises(OverflowError):
        eng.check()
    eng.fl.zero_()
    eng.check()


def test_device_status_word_stops_the_kernels_and_surfaces_on_the_host(engines):
    from bitexact_llm_b200 import _native as nv
    eng, eng8 = engines
    lin = eng.layers[0]["wqkv"]
    g = torch.Generator().manual_seed(3)
    q = torch.randint(-(1 << 22), (1 << 22) + 1, (5, lin.K), generator=g, dtype=torch.int32).cuda()
    sh = torch.full((5,), -30, device="cuda")
    want = lin(q, sh, eng.fl, True).clone()
    torch.cuda.synchronize()
    lib = nv.lib()
    assert nv.device_status() == 0
    try:
        assert lib.bx_set_device_status(1) == 0
        # the device word is set but the host has not read it yet: the launch goes out, every CTA leaves at once
        y = torch.full((5, lin.N), -12345, dtype=torch.long, device="cuda")
        scratch = torch.empty(3 * 5 * lin.K, dtype=torch.int8, device="cuda")
        rc = lib.bx_exact_linear(q.data_ptr(), q.stride(0), sh.data_ptr(), lin.limbs.data_ptr(), lin.d.data_ptr(),
                                 lin.g.data_ptr(), nv.ptr(lin.cnt), nv.ptr(lin.ec), nv.ptr(lin.ev), lin.R,
                                 scratch.data_ptr(), y.data_ptr(), eng.fl.data_ptr(), 5, lin.N, lin.K, 1, 0, nv.stream())
        torch.cuda.synchronize()
        assert rc == 0 and bool((y == -12345).all()), "a CTA wrote output although the status word was set"
        for e in (eng, eng8):
            with pytest.raises(nv.DeviceWaitError):
                e.check()
        # now the host knows: entry points refuse to launch
        n0 = lib.bx_launch_count()
        with pytest.raises(RuntimeError, match="device-side wait"):
            lin(q, sh, eng.fl, True)
        assert lib.bx_launch_count() == n0
    finally:
        nv.clear_device_status()
    assert nv.device_status() == 0
    assert torch.equal(lin(q, sh, eng.fl, True), want)
    eng.check()
    eng8.check()
