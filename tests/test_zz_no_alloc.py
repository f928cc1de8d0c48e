"""The allocation-free GEMV entry point against the regular one.

qw3_gemv_w4a16_noalloc serves hosts that cannot allocate device memory at call time (all memory
handed out at start-up, or a cudaMalloc that would stall the other streams of the process).  Its
scratch is one fixed array inside the library that every call on the GPU reuses, so the check is
made on two calls in a row, on shapes whose tiles are shared between CTAs (the scratch is really
used) and whose second call would see stale counters if the entry point did not clear them.  The
kernel and the summation order are the same as in qw3_gemv_w4a16, so the results must be bitwise
equal, not merely close.  This file sorts last so that a run stopping at the first failure has
already covered every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def _noalloc(ops, p, s, z, M, K, x, y):
    cabi = ops.cabi
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = cabi.lib().qw3_gemv_w4a16_noalloc(C.c_void_p(p.data_ptr()), C.c_void_p(s.data_ptr()), C.c_void_p(z.data_ptr()),
                                           s.numel(), M, K, 1, C.c_void_p(x.data_ptr()), C.c_void_p(y.data_ptr()), st)
    cabi.check(rc, "qw3_gemv_w4a16_noalloc")


def test_noalloc_gemv_equals_workspace_gemv_on_two_calls_in_a_row(ops, orc, cuda):
    ws = ops.Workspace()
    free_before = None
    for call, (M, K, seed) in enumerate([(4096, 4096, 31), (1536, 512, 32), (4096, 12288, 33)]):
        p, s, z = orc.gen_linear(seed, M, K)
        x = orc.gen_normal_f16(seed, orc.ACT, K)
        pd, sd, zd, xd = _dev(p, cuda), _dev(s, cuda), _dev(z, cuda), _dev(x, cuda)
        want = torch.zeros(M, dtype=torch.float16, device=cuda)
        w = ops.W4Linear(pd, sd, zd, M, K)
        ops.gemv_w4a16(w, ws, ops.gemv_args(xd, y=want))
        got = torch.full((M,), 3.0, dtype=torch.float16, device=cuda)
        torch.cuda.synchronize()
        if call > 0:   # the first call may set the device up; from the second on the entry point must not allocate
            free_before = torch.cuda.mem_get_info()[0]
        _noalloc(ops, pd, sd, zd, M, K, xd, got)
        torch.cuda.synchronize()
        if call > 0:
            assert torch.cuda.mem_get_info()[0] == free_before, "qw3_gemv_w4a16_noalloc changed the free device memory"
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"call {call}: {M}x{K}"
        # and the result is the oracle's, within the tolerance the GEMV tests use
        y32, _ = orc.gemm_w4a16(p, s, z, M, K, x)
        err = np.abs(got.cpu().numpy().astype(np.float32) - y32)
        assert (err <= 2e-2 * np.abs(y32) + 2e-2 * np.abs(y32).mean()).all()
    ws.check()
    # no bounded wait gave up in any of the calls: the scratch's error word is clean
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert ops.cabi.lib().qw3_gemv_w4a16_noalloc_status(st) == ops.cabi.QW3_OK


def test_noalloc_gemv_refuses_sizes_beyond_its_scratch(ops, cuda):
    cabi = ops.cabi
    t = torch.zeros(1024, dtype=torch.uint8, device=cuda)
    rc = cabi.lib().qw3_gemv_w4a16_noalloc(C.c_void_p(t.data_ptr()), C.c_void_p(t.data_ptr()), C.c_void_p(t.data_ptr()), 1,
                                           151936, 4096, 1, C.c_void_p(t.data_ptr()), C.c_void_p(t.data_ptr()), None)
    assert rc == cabi.QW3_ERR_ARG
    assert b"16384" in cabi.lib().qw3_last_error()
