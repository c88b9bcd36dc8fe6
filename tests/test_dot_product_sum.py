"""Parity of the dot-product-sum module with the CPU oracle and the reference fixtures,
following the reference's tests/test_dot_product_sum.py: fp32 forward + gradients for
T in {33, 64, 100} x causal, k_diff in {2, 8}, large logits stay finite, non-contiguous
inputs, ValueError on mismatched shapes, and the (out, m) return value."""
import os

import numpy as np
import pytest
import torch

from conftest import golden_cases
from oracle import trittention_oracle as orc
from flash_trittention import _native
from flash_trittention.dot_product_sum.trittention_triton import TrittentionTriton

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run(q, k1, k2, v1, v2, dz, causal, scale, k_diff, **kw):
    leaves = [t.detach().to(DEV).requires_grad_(True) for t in (q, k1, k2, v1, v2)]
    out, m = TrittentionTriton(causal=causal, softmax_scale=scale, k_diff=k_diff, **kw)(*leaves)
    assert not m.requires_grad and m.dtype == torch.float32
    out.backward(dz.to(DEV).to(out.dtype))
    torch.cuda.synchronize()
    assert _native.read_status(torch.device(DEV)) == 0
    return out.detach().cpu(), m.cpu(), [t.grad.cpu() for t in leaves]


def run_and_compare(seq_len, causal, k_diff, B=2, N=2, D=32, seed=0):
    scale = 1 / 8
    q, k1, k2, v1, v2, dz = orc.make_inputs(B, N, seq_len, D, seed=seed)
    out, m, grads = _run(q, k1, k2, v1, v2, dz, causal, scale, k_diff)
    z_ref, lse_ref = orc.dps_forward(q, k1, k2, v1, v2, scale, causal, k_diff)
    g_ref = orc.dps_backward(q, k1, k2, v1, v2, dz, scale, causal, k_diff)
    torch.testing.assert_close(out, z_ref, rtol=1e-4, atol=2e-5)
    torch.testing.assert_close(m, lse_ref, rtol=1e-5, atol=1e-4)
    for name, a, b in zip(("dq", "dk1", "dk2", "dv1", "dv2"), grads, g_ref):
        torch.testing.assert_close(a, b, rtol=1e-3, atol=1e-4, msg=lambda msg, n=name: f"{n}: {msg}")


@pytest.mark.parametrize("seq_len", [33, 64, 100])
@pytest.mark.parametrize("causal", [True, False])
def test_forward_and_backward_fp32(seq_len, causal):
    run_and_compare(seq_len, causal, k_diff=seq_len, seed=seq_len)


@pytest.mark.parametrize("k_diff", [2, 8])
def test_narrow_k_diff_causal(k_diff):
    run_and_compare(seq_len=64, causal=True, k_diff=k_diff, seed=k_diff)


def test_default_k_diff_larger_than_sequence():
    run_and_compare(seq_len=48, causal=True, k_diff=1024, seed=3)


def test_large_logits_no_overflow():
    seq_len, scale = 64, 1 / 8
    q, k1, k2, v1, v2, dz = orc.make_inputs(2, 2, seq_len, 32, seed=4)
    k1, k2 = k1 * 8, k2 * 8
    out, m, grads = _run(q, k1, k2, v1, v2, dz, True, scale, seq_len, input_precision="ieee")
    assert torch.isfinite(out).all()
    z_ref, _ = orc.dps_forward(q, k1, k2, v1, v2, scale, True, seq_len)
    torch.testing.assert_close(out, z_ref, rtol=2e-2, atol=2e-3)
    for name, g in zip(("dq", "dk1", "dk2", "dv1", "dv2"), grads):
        assert torch.isfinite(g).all(), f"{name} contains non-finite values"


def test_non_contiguous_inputs():
    seq_len = 64
    q, _, _, v1, v2, dz = orc.make_inputs(2, 4, seq_len, 32, seed=5)
    g = torch.Generator().manual_seed(6)
    k1 = torch.randn(2, seq_len, 4, 32, generator=g).transpose(1, 2)
    k2 = torch.randn(2, seq_len, 4, 32, generator=g).transpose(1, 2)
    out, m = TrittentionTriton(causal=True, softmax_scale=1 / 8, k_diff=seq_len)(
        q.to(DEV), k1.to(DEV), k2.to(DEV), v1.to(DEV), v2.to(DEV))
    z_ref, _ = orc.dps_forward(q, k1, k2, v1, v2, 1 / 8, True, seq_len)
    torch.testing.assert_close(out.cpu(), z_ref, rtol=1e-4, atol=2e-5)


def test_rejects_mismatched_shapes():
    q, k1, k2, v1, v2 = (torch.randn(2, 2, 32, 32, device=DEV) for _ in range(5))
    with pytest.raises(ValueError):
        TrittentionTriton()(q, k1, k2, v1, v2[:, :, :16, :].contiguous())


@pytest.mark.parametrize("path", golden_cases("dps_"), ids=os.path.basename)
def test_against_reference_fixture(path):
    d = np.load(path)
    t = {k: torch.from_numpy(d[k]) for k in ("q", "k1", "k2", "v1", "v2", "dz", "z", "dq", "dk1", "dk2", "dv1", "dv2")}
    out, m, grads = _run(t["q"], t["k1"], t["k2"], t["v1"], t["v2"], t["dz"], bool(d["causal"]),
                         float(d["softmax_scale"]), int(d["k_diff"]))
    big = "large_logits" in path
    torch.testing.assert_close(out, t["z"], rtol=1e-4, atol=1e-4 if big else 2e-5)
    for name, a in zip(("dq", "dk1", "dk2", "dv1", "dv2"), grads):
        torch.testing.assert_close(a, t[name], rtol=1e-3, atol=5e-3 if big else 1e-4,
                                   msg=lambda msg, n=name: f"{n}: {msg}")


@pytest.mark.parametrize("dtype,tol", [(torch.float16, 5e-3), (torch.bfloat16, 2e-2)])
def test_16bit_inputs(dtype, tol):
    B, N, T, D, scale = 2, 2, 96, 64, 1 / 8
    q, k1, k2, v1, v2, dz = orc.make_inputs(B, N, T, D, seed=9, dtype=dtype)
    out, m, grads = _run(q, k1, k2, v1, v2, dz, True, scale, T)
    f = lambda *xs: [x.float() for x in xs]
    z_ref, _ = orc.dps_forward(*f(q, k1, k2, v1, v2), scale, True, T)
    g_ref = orc.dps_backward(*f(q, k1, k2, v1, v2, dz), scale, True, T)
    assert (out.float() - z_ref).abs().max() <= tol * float(z_ref.abs().max())
    for name, a, b in zip(("dq", "dk1", "dk2", "dv1", "dv2"), grads, g_ref):
        assert (a.float() - b).abs().max() <= tol * float(b.abs().max()), name


@pytest.mark.parametrize("D", [8, 16, 128, 256])
def test_other_head_dims(D):
    """Head dimensions on both kernel families: 16..128 run the register-resident kernels, the rest the
    shared-memory ones."""
    run_and_compare(seq_len=40, causal=True, k_diff=40, B=1, N=2, D=D, seed=D)
