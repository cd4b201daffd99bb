"""gg_gemm_tc_static, the entry point for callers that cannot allocate (a plug-in under a host
program that owns device memory, a loop that may not touch the allocator): called through its
exported C symbol, twice in a row, and compared with the regular entry point gg_gemm_tc, which
gets its scratch from the caller.  The static scratch keeps the first call's contents when the
second call runs; the second call's result must not depend on them.

This file is collected last on purpose: if it fails, a run that stops at the first failure has
already run every other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rel(a, b):
    a, b = a.double(), b.double()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def test_static_scratch_entry_point_matches_the_regular_one():
    from gogguf_b200.csrc import build
    from gogguf_b200.csrc import tcgen05_gemm as tc

    lib = ctypes.CDLL(build.compile_module("gemm_tcgen05_static"))
    fn = lib.gg_gemm_tc_static            # the exported C symbol itself
    vp, i, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    fn.argtypes = [vp, vp, vp, i, i, i, i, ll, ll, vp, vp]
    fn.restype = i
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device=DEV).manual_seed(21)

    def both(M, N, K_, mode_dtype, accumulate):
        x = torch.randn(M, K_, device=DEV, generator=g).to(torch.bfloat16)
        w = torch.randn(N, K_, device=DEV, generator=g).to(torch.bfloat16)
        splits = tc.splits_for(M, N, K_)
        base = torch.randn(M, N, device=DEV, generator=g).to(mode_dtype)
        want_out = base.clone()
        scratch = torch.empty(max(1, splits * M * N), device=DEV)
        tc.gemm_tc(x, w, want_out, accumulate=accumulate, scratch=scratch)      # the existing entry point
        got = base.clone()
        mode = 0 if mode_dtype == torch.bfloat16 else (2 if accumulate else 1)
        rc = fn(x.data_ptr(), w.data_ptr(), got.data_ptr(), mode, M, N, K_, K_, N, status.data_ptr(), stream)
        assert rc == 0, rc
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        exact = x.double() @ w.double().T + (base.double() if accumulate else 0)
        tol = (2e-6 + 2e-7 * math.sqrt(K_)) if mode_dtype == torch.float32 else 5e-3
        assert rel(got, exact) < tol
        assert rel(got, want_out) < tol
        assert torch.equal(got, want_out)        # same kernels, same split: the same bits
        return splits

    # two calls in a row; both split K, so both go through the shared static array, and the second
    # is smaller, so most of what the first call left there is still in place while it runs
    s1 = both(64, 1024, 4096, torch.float32, accumulate=True)
    s2 = both(9, 384, 2048, torch.bfloat16, accumulate=False)
    assert s1 > 1 and s2 > 1
    # a product beyond the array's stated size is refused before anything runs
    M, N, K_ = 128, 24576, 4096
    assert tc.splits_for(M, N, K_) * M * N > 4 * 1024 * 1024
    rc = fn(0, 0, 0, 1, M, N, K_, K_, N, status.data_ptr(), stream)
    assert rc == -1
