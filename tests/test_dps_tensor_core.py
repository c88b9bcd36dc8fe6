"""Dot-product-sum trittention with its two soft-max attentions on the tcgen05 kernel (16-bit inputs, head dimension
64 or 128): forward against the oracle's factorised fp32 restatement and against the CUDA-core path, over ragged
sequence lengths, narrow and wide ``k_diff`` bands, causal and not, large logits; and the backward (a row-owner and
a column-owner tcgen05 kernel per attention) likewise.  Tolerances: max-abs and rms error 5e-3 (fp16) / 2e-2 (bf16), relative to
each tensor's own magnitude."""
import pytest
import torch

from _parity import assert_close
from flash_trittention import _native
from oracle import trittention_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.float16: 5e-3, torch.bfloat16: 2e-2}


def _fwd(t, scale, causal, k_diff, flags=0):
    o = torch.empty_like(t[0])
    m = torch.empty(t[0].shape[:3], dtype=torch.float32, device=DEV)
    _native.dps_fwd(*t, o, m, scale, causal, k_diff, flags=flags)
    torch.cuda.synchronize()
    assert _native.read_status(torch.device(DEV)) == 0
    return o, m


def test_path_selection():
    assert _native.dps_path(1024, 64, _native.F16, 1024) == _native.PATH_TCGEN05
    assert _native.dps_path(100, 128, _native.BF16, 0) == _native.PATH_TCGEN05
    assert _native.dps_path(100, 32, _native.BF16, 8) == _native.PATH_SIMT
    assert _native.dps_path(100, 64, _native.F32, 8) == _native.PATH_SIMT
    assert _native.dps_path(100, 64, _native.F16, 8, _native.FLAG_FORCE_SIMT) == _native.PATH_SIMT


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("T,D,causal,k_diff", [
    (33, 64, True, 33), (100, 64, True, 8), (128, 64, True, 0), (129, 128, True, 129), (300, 64, True, 130),
    (300, 128, True, 2), (512, 64, True, 512), (384, 128, True, 200), (100, 64, False, 100), (260, 128, False, 5),
])
def test_forward_matches_oracle(dtype, T, D, causal, k_diff):
    B, N, scale = 1, 2, 1 / 8
    q, k1, k2, v1, v2, _ = orc.make_inputs(B, N, T, D, seed=T + D, dtype=dtype)
    t = [x.to(DEV) for x in (q, k1, k2, v1, v2)]
    assert _native.dps_path(T, D, _native.dtype_code(dtype), k_diff) == _native.PATH_TCGEN05
    o, m = _fwd(t, scale, causal, k_diff)
    z_ref, lse_ref = orc.dps_forward_factorised(*[x.float() for x in (q, k1, k2, v1, v2)], scale, causal, k_diff)
    tol = TOL[dtype]
    assert_close("o", o.cpu(), z_ref, dtype)
    assert float((m.cpu() - lse_ref).abs().max()) <= tol
    # and against the CUDA-core kernels on the same inputs
    o2, m2 = _fwd(t, scale, causal, k_diff, flags=_native.FLAG_FORCE_SIMT)
    assert_close("o (against the CUDA-core path)", o, o2, dtype)
    assert float((m - m2).abs().max()) <= tol


def test_large_logits_stay_finite():
    """Keys scaled by 8 (the reference's overflow guard, tests/test_dot_product_sum.py:84-118): logits of several
    hundred, exponentials taken against the running row maximum."""
    B, N, T, D, scale = 1, 2, 200, 64, 1 / 8
    q, k1, k2, v1, v2, _ = orc.make_inputs(B, N, T, D, seed=5, dtype=torch.float16)
    k1, k2 = k1 * 8, k2 * 8
    t = [x.to(DEV) for x in (q, k1, k2, v1, v2)]
    o, m = _fwd(t, scale, True, T)
    assert torch.isfinite(o).all() and torch.isfinite(m).all()
    z_ref, lse_ref = orc.dps_forward_factorised(*[x.float() for x in (q, k1, k2, v1, v2)], scale, True, T)
    assert_close("o", o.cpu(), z_ref, torch.float16)
    assert_close("m", m.cpu(), lse_ref, torch.float16)


def _bwd(t, o, m, dz, scale, causal, k_diff, flags=0):
    g = [torch.empty_like(t[0]) for _ in range(5)]
    _native.dps_bwd(*t, o, dz, m, *g, scale, causal, k_diff, flags=flags)
    torch.cuda.synchronize()
    assert _native.read_status(torch.device(DEV)) == 0
    return g


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("T,D,causal,k_diff", [
    (33, 64, True, 33), (100, 64, True, 8), (128, 128, True, 0), (200, 64, True, 200), (300, 64, True, 130),
    (160, 128, True, 12), (384, 128, True, 384), (100, 64, False, 100), (260, 128, False, 5),
])
def test_backward_matches_oracle(dtype, T, D, causal, k_diff):
    B, N, scale = 1, 2, 1 / 8
    q, k1, k2, v1, v2, dz = orc.make_inputs(B, N, T, D, seed=2 * T + D, dtype=dtype)
    t = [x.to(DEV) for x in (q, k1, k2, v1, v2)]
    dzd = dz.to(DEV)
    o, m = _fwd(t, scale, causal, k_diff)
    grads = _bwd(t, o, m, dzd, scale, causal, k_diff)
    g_ref = orc.dps_backward(*[x.float() for x in (q, k1, k2, v1, v2, dz)], scale, causal, k_diff)
    simt = _bwd(t, o, m, dzd, scale, causal, k_diff, flags=_native.FLAG_FORCE_SIMT)
    for name, a, b, c in zip(("dq", "dk1", "dk2", "dv1", "dv2"), grads, g_ref, simt):
        assert_close(name, a.cpu(), b, dtype)
        assert_close(name + " (against the CUDA-core path)", a, c, dtype)


def test_backward_through_the_module():
    from flash_trittention import TrittentionTriton

    B, N, T, D, scale, k_diff = 1, 2, 200, 64, 1 / 8, 40
    q, k1, k2, v1, v2, dz = orc.make_inputs(B, N, T, D, seed=11, dtype=torch.float16)
    leaves = [x.to(DEV).requires_grad_(True) for x in (q, k1, k2, v1, v2)]
    out, _ = TrittentionTriton(causal=True, softmax_scale=scale, k_diff=k_diff)(*leaves)
    out.backward(dz.to(DEV))
    torch.cuda.synchronize()
    assert _native.read_status(torch.device(DEV)) == 0
    g_ref = orc.dps_backward(*[x.float() for x in (q, k1, k2, v1, v2, dz)], scale, True, k_diff)
    for name, leaf, ref in zip(("dq", "dk1", "dk2", "dv1", "dv2"), leaves, g_ref):
        assert_close(name, leaf.grad.cpu(), ref, torch.float16)


@pytest.mark.parametrize("N,T,D", [(1, 33, 64), (3, 129, 128), (1, 77, 128)])
def test_odd_number_of_rows(N, T, D):
    """B*N*T odd: the fp32 scratch vectors of length B*N*T sit between [B,N,T,D] buffers that the tensor-core kernels
    write with 16-byte stores, so every workspace segment has to start on a 16-byte boundary whatever the row count."""
    B, scale, dtype = 1, 1 / 8, torch.float16
    q, k1, k2, v1, v2, dz = orc.make_inputs(B, N, T, D, seed=3 * T + N, dtype=dtype)
    t = [x.to(DEV) for x in (q, k1, k2, v1, v2)]
    assert _native.dps_path(T, D, _native.dtype_code(dtype), T) == _native.PATH_TCGEN05
    o, m = _fwd(t, scale, True, T)
    z_ref, lse_ref = orc.dps_forward_factorised(*[x.float() for x in (q, k1, k2, v1, v2)], scale, True, T)
    assert_close("o", o.cpu(), z_ref, dtype)
    assert float((m.cpu() - lse_ref).abs().max()) <= TOL[dtype]
    grads = _bwd(t, o, m, dz.to(DEV), scale, True, T)
    g_ref = orc.dps_backward(*[x.float() for x in (q, k1, k2, v1, v2, dz)], scale, True, T)
    for name, a, b in zip(("dq", "dk1", "dk2", "dv1", "dv2"), grads, g_ref):
        assert_close(name, a.cpu(), b, dtype)


@pytest.mark.parametrize("dtype,T,D,k_diff", [(torch.float16, 300, 64, 130), (torch.bfloat16, 129, 128, 129),
                                              (torch.float32, 70, 32, 9)])
def test_backward_with_the_forward_workspace_equals_the_recomputing_backward(dtype, T, D, k_diff):
    """``tritt_dps_bwd_saved`` reads the inner attention's results from the forward call's workspace instead of
    computing them again: same kernels on the same data, so the gradients are identical."""
    B, N, scale = 1, 2, 1 / 8
    q, k1, k2, v1, v2, dz = orc.make_inputs(B, N, T, D, seed=T + 3, dtype=dtype)
    t = [x.to(DEV) for x in (q, k1, k2, v1, v2)]
    dzd = dz.to(DEV)
    o = torch.empty_like(t[0])
    m = torch.empty(B, N, T, dtype=torch.float32, device=DEV)
    fwd_ws = _native.dps_fwd(*t, o, m, scale, True, k_diff)
    a = [torch.empty_like(t[0]) for _ in range(5)]
    _native.dps_bwd(*t, o, dzd, m, *a, scale, True, k_diff, fwd_ws=fwd_ws)
    b = _bwd(t, o, m, dzd, scale, True, k_diff)
    torch.cuda.synchronize()
    assert _native.read_status(torch.device(DEV)) == 0
    for name, x, y in zip(("dq", "dk1", "dk2", "dv1", "dv2"), a, b):
        assert torch.equal(x, y), name
