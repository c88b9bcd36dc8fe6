"""The allocation-free forward entry point (``tritt_tdp_fwd_noalloc``).

Some callers cannot give the library a scratch buffer because they may not allocate device memory
where they call it (a plugin inside a host program's enqueue hook, code that must not trigger the
allocator's device synchronisation).  For them the library carries a fixed 8 MiB scratch array in
its own device image.  This test calls that entry point through the C ABI twice in a row - the
array keeps the previous call's contents, so the second call checks that nothing stale leaks - and
compares both results with the ordinary entry point, which gets a fresh workspace.  It also checks
that a problem too large for the built-in array is refused with a message instead of being run.

This file sorts last on purpose: a run that stops at the first failure has then already executed
every other test.  It does not depend on them and passes in a fresh process as well.
"""
import ctypes

import pytest
import torch

from flash_trittention import _native

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _inputs(B, N, T, D, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(B, N, T, D, generator=g) * 0.5).to(dtype).to(DEV) for _ in range(5)]


@pytest.mark.parametrize("shape,dtype", [((2, 2, 256, 64), torch.bfloat16), ((1, 3, 200, 128), torch.float16),
                                         ((1, 2, 48, 32), torch.float32)])
def test_noalloc_forward_matches_workspace_forward_twice(shape, dtype):
    B, N, T, D = shape
    alpha = 1.0 / D
    for call, seed in enumerate((101, 202)):  # two calls in a row, different data
        t = _inputs(B, N, T, D, dtype, seed)
        o_ref, lse_ref = torch.empty_like(t[0]), torch.empty(B, N, T, device=DEV)
        _native.tdp_fwd(*t, o_ref, lse_ref, alpha, True, None, None, None, None)
        o = torch.full_like(t[0], float("nan"))
        lse = torch.full((B, N, T), float("nan"), device=DEV)
        _native.tdp_fwd_noalloc(*t, o, lse, alpha, True, None, None, None, None)
        torch.cuda.synchronize()
        assert _native.read_status(torch.device(DEV)) == 0
        # same kernels on the same inputs.  The tensor-core forward has no atomics: identical results.  The CUDA-core
        # forward (the fp32 case) merges partial rows with fp32 atomic adds, whose order is not fixed: last-bit noise.
        if dtype == torch.float32:
            assert float((o - o_ref).abs().max()) <= 1e-6 * float(o_ref.abs().max()), f"call {call}"
            assert float((lse - lse_ref).abs().max()) <= 1e-6 * float(lse_ref.abs().max()), f"call {call}"
        else:
            assert torch.equal(o, o_ref), f"call {call}: max diff {float((o.float() - o_ref.float()).abs().max())}"
            assert torch.equal(lse, lse_ref), f"call {call}: max diff {float((lse - lse_ref).abs().max())}"


def test_noalloc_rejects_problems_beyond_the_builtin_scratch():
    lib = _native.lib()
    cap = lib.tritt_noalloc_scratch_bytes()
    assert cap == 8 << 20
    B, N, T, D = 1, 64, 2048, 128  # 16 Mi elements of bf16: four times the built-in scratch
    small = torch.zeros(1024, dtype=torch.bfloat16, device=DEV)  # never touched: the call is refused first
    lse = torch.zeros(16, device=DEV)
    p = small.data_ptr()
    rc = lib.tritt_tdp_fwd_noalloc(p, p, p, p, p, p, lse.data_ptr(), B, N, T, D, _native.BF16, 1.0 / D, 1, T, T, T, T,
                                   None, 0, torch.cuda.current_stream().cuda_stream)
    assert rc < 0
    assert b"maximum" in lib.tritt_last_error()
    with pytest.raises(ValueError, match="maximum"):
        _native._check(rc, "tritt_tdp_fwd_noalloc")
