"""GPU test of nvfp4_linear_decode_noalloc, the GEMV entry point for hosts that may not allocate
device memory (their memory is fully planned at start-up, e.g. an engine that hands all free HBM
to its KV-cache pool).  It is called through the C ABI, twice in a row, and each result is checked
against the handle-based nvfp4_linear on the same inputs.  The file sorts last on purpose: a run
that stops at the first failure has then already been through every other test."""
import ctypes

import numpy as np
import pytest

import nvfp4
import oracle_binding as ob
import util

pytestmark = pytest.mark.gpu
TOL = 1e-3


def _case(N, K, M, seed, with_residual):
    packed, scale = util.make_weight(N, K, seed=seed)
    A = util.make_bf16((M, K), seed=seed + 1)
    R = util.make_bf16((M, N), seed=seed + 2) if with_residual else None
    return packed, scale, A, R


def test_noalloc_matches_handle_entry_point_twice_in_a_row():
    import torch
    assert torch.cuda.is_available()
    lib = nvfp4.load()
    h = nvfp4.Handle(0, 64 << 20)
    stream = torch.cuda.current_stream().cuda_stream
    try:
        # first call: tiles split over CTAs (partials + flags in the fixed array); second call: other shape,
        # residual in place, more than 8 tokens (two launches sharing the array back to back)
        # third and fourth: a last row tile that is only partly inside N, and 16 tokens (two full launches) with the
        # residual aliasing the output
        first = True
        for (N, K, M, seed, res) in [(5120, 17408, 4, 7, False), (2048, 5120, 12, 9, True), (1000, 2048, 3, 11, False),
                                     (4200, 5120, 16, 13, True)]:
            packed, scale, A, R = _case(N, K, M, seed, res)
            dA, dp, ds = util.to_dev(A), util.to_dev(packed), util.to_dev(scale)
            want = util.to_dev(R) if res else torch.zeros(M, N, dtype=torch.int16, device="cuda")
            got = util.to_dev(R) if res else torch.zeros(M, N, dtype=torch.int16, device="cuda")
            h.linear(dA, M, dp, ds, 1.0, N, K, want, residual=want if res else None)
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
            st = lib.nvfp4_linear_decode_noalloc(dA.data_ptr(), M, dp.data_ptr(), ds.data_ptr(), 1.0, N, K,
                                                 got.data_ptr() if res else None, got.data_ptr(), stream)
            assert st == 0, lib.nvfp4_status_string(st).decode()
            torch.cuda.synchronize()
            # what the entry point is for: free device memory is the same before and after the call (the very
            # first call may still load the kernel's code, so it is left out)
            if not first:
                assert torch.cuda.mem_get_info()[0] == free_before
            first = False
            g, w = util.to_host_u16(got), util.to_host_u16(want)
            assert ob.rel_frobenius(g, w) <= TOL
            assert ob.rel_frobenius(g, ob.linear(A, packed, scale, 1.0, residual=R, mode=ob.GEMV, threads=8)) <= TOL
        # beyond the fixed maximum: clear refusals, nothing launched
        dummy = torch.zeros(64 * 1024, dtype=torch.int16, device="cuda")
        p = dummy.data_ptr()
        assert lib.nvfp4_linear_decode_noalloc(p, 17, p, p, 1.0, 64, 256, None, p + 65536, stream) == -10
        assert lib.nvfp4_linear_decode_noalloc(p, 1, p, p, 1.0, 64, 48, None, p + 65536, stream) == -10
        assert b"allocation-free" in lib.nvfp4_status_string(-10)
        torch.cuda.synchronize()
        # no device-side wait ran out in any of the calls above; the accessor refuses a null pointer
        word = ctypes.c_uint(1)
        assert lib.nvfp4_noalloc_status(ctypes.byref(word), 0) == 0 and word.value == 0
        assert lib.nvfp4_noalloc_status(None, 0) == -1
    finally:
        h.close()
