"""The allocation-free exact linear (`bx_exact_linear_static`): for hosts that may not allocate device memory
at call time (a plugin called while its application records a CUDA graph, a fixed-arena runtime, a service that
bans cudaMalloc after start-up), the activation limb planes live in a 6 MiB buffer inside the library image.

Checked here through the C ABI: two calls in a row give exactly the integers of the ordinary entry point (the
buffer keeps the previous call's bytes, so the second call runs on a dirty buffer), the capacity limit is
reported as BX_ELIMIT, and no torch allocation happens inside the calls."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(M, N, K, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randint(-(1 << 22), (1 << 22) + 1, (M, K), dtype=torch.int32, device="cuda", generator=g)
    sh = torch.randint(-40, -8, (M,), device="cuda", generator=g)
    limbs = torch.randint(-128, 128, (3, N, K), dtype=torch.int8, device="cuda", generator=g)
    d = torch.randint(0, 31, (N,), device="cuda", generator=g)
    gg = torch.randint(-34, -24, (N,), device="cuda", generator=g)
    cnt = torch.zeros(N, dtype=torch.int32, device="cuda")
    cnt[::7] = 1
    ec = torch.randint(0, K, (N, 1), device="cuda", generator=g).to(torch.int32)
    ev = torch.randint(-(1 << 20), 1 << 20, (N, 1), device="cuda", generator=g)
    return q, sh, limbs, d, gg, cnt, ec, ev


def test_static_scratch_entry_matches_the_ordinary_one_twice_in_a_row():
    from bitexact_llm_b200 import _native as nv
    lib = nv.lib()
    st = nv.stream()
    assert lib.bx_exact_linear_static_max_bytes() == 3 * 256 * 8192
    for M, N, K, seed in [(256, 384, 2048, 1), (7, 200, 272, 2)]:            # second case runs on a dirty buffer
        q, sh, limbs, d, g, cnt, ec, ev = _case(M, N, K, seed)
        y_ref = torch.empty(M, N, dtype=torch.long, device="cuda")
        y_new = torch.full((M, N), -1, dtype=torch.long, device="cuda")
        f_ref = torch.zeros(1, dtype=torch.int32, device="cuda")
        f_new = torch.zeros(1, dtype=torch.int32, device="cuda")
        scratch = torch.empty(3 * M * K, dtype=torch.int8, device="cuda")
        rc = lib.bx_exact_linear(q.data_ptr(), K, sh.data_ptr(), limbs.data_ptr(), d.data_ptr(), g.data_ptr(),
                                 cnt.data_ptr(), ec.data_ptr(), ev.data_ptr(), 1, scratch.data_ptr(), y_ref.data_ptr(),
                                 f_ref.data_ptr(), M, N, K, 1, 0, st)
        assert rc == 0
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        for _ in range(2):
            rc = lib.bx_exact_linear_static(q.data_ptr(), K, sh.data_ptr(), limbs.data_ptr(), d.data_ptr(),
                                            g.data_ptr(), cnt.data_ptr(), ec.data_ptr(), ev.data_ptr(), 1,
                                            y_new.data_ptr(), f_new.data_ptr(), M, N, K, 1, 0, st)
            assert rc == 0
            torch.cuda.synchronize()
            assert torch.equal(y_new, y_ref) and torch.equal(f_new, f_ref)
            y_new.fill_(-1)
        assert torch.cuda.memory_allocated() == before
    # beyond the buffer: refused, nothing launched
    n0 = lib.bx_launch_count()
    rc = lib.bx_exact_linear_static(q.data_ptr(), 8192, sh.data_ptr(), limbs.data_ptr(), d.data_ptr(), g.data_ptr(),
                                    None, None, None, 0, y_new.data_ptr(), f_new.data_ptr(), 257, 128, 8192, 1, 0, st)
    assert rc == nv.BX_ELIMIT and lib.bx_launch_count() == n0
    assert nv.device_status() == 0
