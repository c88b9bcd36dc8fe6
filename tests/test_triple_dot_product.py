"""Parity of the triple-dot-product entry point with the CPU oracle and with the fixtures
generated from the reference, following the reference's own test-suite
(tests/test_triple_dot_product.py of the reference): fp32 forward + five gradients for
T in {33, 64, 100} x causal, narrow windows, a loose fp16 forward, and the ValueErrors."""
import os

import numpy as np
import pytest
import torch

from conftest import golden_cases
from oracle import trittention_oracle as orc
from flash_trittention import _native
from flash_trittention.triple_dot_product.flash_trittention import flash_trittention

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run(q, k1, k2, v1, v2, dz, **kw):
    leaves = [t.detach().to(DEV).requires_grad_(True) for t in (q, k1, k2, v1, v2)]
    out = flash_trittention(*leaves, **kw)
    out.backward(dz.to(DEV).to(out.dtype))
    torch.cuda.synchronize()
    assert _native.read_status(torch.device(DEV)) == 0
    return out.detach().cpu(), [t.grad.cpu() for t in leaves]


def _compare(out, grads, z_ref, grads_ref, fwd_tol, bwd_tol):
    torch.testing.assert_close(out.float(), z_ref, rtol=fwd_tol[0], atol=fwd_tol[1])
    for name, a, b in zip(("dq", "dk1", "dk2", "dv1", "dv2"), grads, grads_ref):
        torch.testing.assert_close(a.float(), b, rtol=bwd_tol[0], atol=bwd_tol[1], msg=lambda m, n=name: f"{n}: {m}")


@pytest.mark.parametrize("seq_len", [33, 64, 100])
@pytest.mark.parametrize("causal", [True, False])
def test_forward_and_backward_fp32(seq_len, causal):
    B, N, D, scale = 2, 2, 32, 1 / 8
    q, k1, k2, v1, v2, dz = orc.make_inputs(B, N, seq_len, D, seed=seq_len)
    kw = dict(softmax_scale=scale, k1_window=seq_len, k2_window=seq_len, kk_left=seq_len, kk_right=seq_len,
              causal=causal)
    out, grads = _run(q, k1, k2, v1, v2, dz, **kw)
    z_ref, _ = orc.tdp_forward(q, k1, k2, v1, v2, scale, causal)
    g_ref = orc.tdp_backward(q, k1, k2, v1, v2, dz, scale, causal)
    # the reference's own tolerances are rtol 2e-2 / atol 2e-3 (fwd) and 5e-3 (grads); the fp32 path is far tighter
    _compare(out, grads, z_ref, g_ref, (1e-4, 2e-5), (1e-3, 1e-4))


@pytest.mark.parametrize("seq_len", [64, 100])
@pytest.mark.parametrize("windows", [(8, 8, 4, 4), (16, 7, 3, 9), (1, 1, 1, 1)])
def test_narrow_windows_causal(seq_len, windows):
    B, N, D, scale = 2, 2, 32, 1 / 8
    k1w, k2w, kkl, kkr = windows
    q, k1, k2, v1, v2, dz = orc.make_inputs(B, N, seq_len, D, seed=7 + seq_len)
    out, grads = _run(q, k1, k2, v1, v2, dz, softmax_scale=scale, k1_window=k1w, k2_window=k2w, kk_left=kkl,
                      kk_right=kkr, causal=True)
    z_ref, _ = orc.tdp_forward(q, k1, k2, v1, v2, scale, True, k1w, k2w, kkl, kkr)
    g_ref = orc.tdp_backward(q, k1, k2, v1, v2, dz, scale, True, k1w, k2w, kkl, kkr)
    _compare(out, grads, z_ref, g_ref, (1e-4, 2e-5), (1e-3, 1e-4))


def test_default_windows_are_one():
    """The entry point's defaults (all windows = 1) are the reference's (flash_trittention.py:396-409)."""
    q, k1, k2, v1, v2, dz = orc.make_inputs(1, 2, 40, 16, seed=11)
    out, _ = _run(q, k1, k2, v1, v2, dz)
    z_ref, _ = orc.tdp_forward(q, k1, k2, v1, v2, 1 / 8, True, 1, 1, 1, 1)
    torch.testing.assert_close(out, z_ref, rtol=1e-4, atol=2e-5)


@pytest.mark.parametrize("path", golden_cases("tdp_"), ids=os.path.basename)
def test_against_reference_fixture(path):
    d = np.load(path)
    t = {k: torch.from_numpy(d[k]) for k in ("q", "k1", "k2", "v1", "v2", "dz", "z", "dq", "dk1", "dk2", "dv1", "dv2")}
    f = lambda v: None if int(v) < 0 else int(v)
    out, grads = _run(t["q"], t["k1"], t["k2"], t["v1"], t["v2"], t["dz"], softmax_scale=float(d["softmax_scale"]),
                      k1_window=f(d["k1_window"]), k2_window=f(d["k2_window"]), kk_left=f(d["kk_left"]),
                      kk_right=f(d["kk_right"]), causal=bool(d["causal"]))
    _compare(out, grads, t["z"], [t[n] for n in ("dq", "dk1", "dk2", "dv1", "dv2")], (1e-4, 2e-5), (1e-3, 1e-4))


@pytest.mark.parametrize("dtype,tol", [(torch.float16, 5e-3), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("force_simt", [True, False])
def test_16bit_forward_backward_small(dtype, tol, force_simt):
    """16-bit inputs: max-abs error against the fp32 oracle on the same (rounded) inputs stays within
    2e-2 (bf16) / 5e-3 (fp16)."""
    B, N, T, D, scale = 2, 2, 64, 32, 1 / 8
    ins = orc.make_inputs(B, N, T, D, seed=21, dtype=dtype)
    q, k1, k2, v1, v2, dz = ins
    out, grads = _run(q, k1, k2, v1, v2, dz, softmax_scale=scale, k1_window=T, k2_window=T, kk_left=T, kk_right=T,
                      causal=True, convert_to_float32=force_simt)
    z_ref, _ = orc.tdp_forward(*(x.float() for x in (q, k1, k2, v1, v2)), scale, True)
    g_ref = orc.tdp_backward(*(x.float() for x in (q, k1, k2, v1, v2, dz)), scale, True)
    assert (out.float() - z_ref).abs().max() <= tol * float(z_ref.abs().max())
    for name, a, b in zip(("dq", "dk1", "dk2", "dv1", "dv2"), grads, g_ref):
        # every gradient is bounded against its own magnitude
        assert (a.float() - b).abs().max() <= tol * float(b.abs().max()), name


def test_rejects_mismatched_shapes():
    q, k1, k2, v1, v2 = (torch.randn(2, 2, 32, 32, device=DEV) for _ in range(5))
    with pytest.raises(ValueError):
        flash_trittention(q, k1, k2, v1, v2[:, :, :16, :].contiguous())


def test_rejects_non_pow2_head_dim():
    q, k1, k2, v1, v2 = (torch.randn(2, 2, 32, 24, device=DEV) for _ in range(5))
    with pytest.raises(ValueError):
        flash_trittention(q, k1, k2, v1, v2)


def test_non_contiguous_inputs_and_query_sharding():
    """Transposed views are accepted; computing the rows in two interleaved shards gives the same rows."""
    B, N, T, D, scale = 1, 2, 48, 16, 1 / 8
    q, k1, k2, v1, v2, _ = orc.make_inputs(B, N, T, D, seed=31)
    z_ref, lse_ref = orc.tdp_forward(q, k1, k2, v1, v2, scale, True)
    k1_t = k1.transpose(1, 2).contiguous().transpose(1, 2).to(DEV)
    out = flash_trittention(q.to(DEV), k1_t, k2.to(DEV), v1.to(DEV), v2.to(DEV), scale, None, None, None, None, True)
    torch.testing.assert_close(out.cpu(), z_ref, rtol=1e-4, atol=2e-5)
    dq, dk1, dk2, dv1, dv2 = (x.to(DEV) for x in (q, k1, k2, v1, v2))
    o = torch.zeros_like(dq)
    lse = torch.zeros(B, N, T, device=DEV)
    for rem in range(2):
        _native.tdp_fwd(dq, dk1, dk2, dv1, dv2, o, lse, scale, True, None, None, None, None, q_mod=2, q_rem=rem)
    torch.testing.assert_close(o.cpu(), z_ref, rtol=1e-4, atol=2e-5)
    torch.testing.assert_close(lse.cpu(), lse_ref, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("D", [8, 16, 64, 128, 256])
def test_fp32_head_dims(D):
    """Head dimensions on both CUDA-core kernel families: 16..128 run the register-resident kernels (four lanes
    per pair row, eight at 128), the others the shared-memory kernel; windows included.  ``input_precision="ieee"``
    keeps head dimensions 64 and 128 on these exact-fp32 kernels (fp32 inputs otherwise take the tensor cores there)."""
    B, N, T, scale = 1, 2, 70, 1 / 8
    q, k1, k2, v1, v2, dz = orc.make_inputs(B, N, T, D, scale=0.7, seed=40 + D)
    for windows in ((T, T, T, T), (20, 33, 6, 11)):
        k1w, k2w, kkl, kkr = windows
        out, grads = _run(q, k1, k2, v1, v2, dz, softmax_scale=scale, k1_window=k1w, k2_window=k2w, kk_left=kkl,
                          kk_right=kkr, causal=True, input_precision="ieee")
        z_ref, _ = orc.tdp_forward(q, k1, k2, v1, v2, scale, True, k1w, k2w, kkl, kkr)
        g_ref = orc.tdp_backward(q, k1, k2, v1, v2, dz, scale, True, k1w, k2w, kkl, kkr)
        _compare(out, grads, z_ref, g_ref, (1e-4, 3e-5), (1e-3, 2e-4))
