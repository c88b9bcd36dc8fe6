"""fp32 inputs (and ``convert_to_float32`` on bf16 inputs) on the tensor-core path.

The reference's own test for fp32 inputs (``tests/test_triple_dot_product.py:51-96`` there: N(0,1) inputs, alpha = 1/8,
sequence lengths 33 / 64 / 100, causal and not) compares its TF32 kernels with the dense fp32 module at
``rtol=2e-2, atol=2e-3`` (output) and ``rtol=2e-2, atol=5e-3`` (gradients).  The same cases run here through the public
entry point at head dimensions 64 and 128, where fp32 inputs take the tcgen05 kernels through fp16 operand copies (11
significant bits, as TF32), against the oracle, at those tolerances; plus the pieces that path adds: the power-of-two
scaling of a tiny upstream gradient, the status bit for inputs beyond fp16's range, and ``convert_to_float32``."""
import pytest
import torch

from _parity import assert_close
from oracle import trittention_oracle as orc
from flash_trittention import _native, flash_trittention

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run(ins, scale, causal, **kw):
    leaves = [x.to(DEV).requires_grad_(True) for x in ins[:5]]
    out = flash_trittention(*leaves, scale, None, None, None, None, causal, **kw)
    out.backward(ins[5].to(DEV))
    torch.cuda.synchronize()
    return out.detach().cpu(), [x.grad.cpu() for x in leaves]


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("T", [33, 64, 100])
@pytest.mark.parametrize("causal", [True, False])
def test_reference_fp32_cases_on_the_tensor_core_path(T, causal, D):
    B, N, scale = 2, 2, 1 / 8
    assert _native.tdp_path(_native.OP_TDP_FWD, T, D, _native.F32, causal, None, None, None, None) == _native.PATH_TCGEN05
    assert _native.tdp_path(_native.OP_TDP_BWD, T, D, _native.F32, causal, None, None, None, None) == _native.PATH_TCGEN05
    ins = orc.make_inputs(B, N, T, D, seed=7 + T, dtype=torch.float32)
    out, grads = _run(ins, scale, causal)
    assert out.dtype == torch.float32 and all(g.dtype == torch.float32 for g in grads)
    assert _native.read_status(torch.device(DEV)) == 0
    z_ref, _ = orc.tdp_forward(*ins[:5], scale, causal)
    g_ref = orc.tdp_backward(*ins, scale, causal)
    torch.testing.assert_close(out, z_ref, rtol=2e-2, atol=2e-3)
    for name, a, b in zip(("dq", "dk1", "dk2", "dv1", "dv2"), grads, g_ref):
        torch.testing.assert_close(a, b, rtol=2e-2, atol=5e-3, msg=lambda m, n=name: f"{n}: {m}")
        assert_close(name, a, b, torch.float16)  # and within the fp16 bounds against each tensor's own magnitude


def test_fp32_benchmark_shape_per_head_and_tiny_upstream_gradient():
    """T = 512, D = 64 (the shape of config 2) in fp32, with an upstream gradient of order 1e-7: without the
    power-of-two scaling its fp16 copy would be all subnormals or zero."""
    B, N, T, D, scale = 1, 2, 512, 64, 1 / 64
    ins = orc.make_inputs(B, N, T, D, scale=0.5, seed=3, dtype=torch.float32)
    ins[5] = ins[5] * 1e-7
    out, grads = _run(ins, scale, True)
    assert _native.read_status(torch.device(DEV)) == 0
    z_ref, _ = orc.tdp_forward(*ins[:5], scale, True)
    g_ref = orc.tdp_backward(*ins, scale, True)
    assert_close("o", out, z_ref, torch.float16)
    for name, a, b in zip(("dq", "dk1", "dk2", "dv1", "dv2"), grads, g_ref):
        assert_close(name, a, b, torch.float16)


def test_convert_to_float32_gives_bf16_inputs_wider_operands():
    """bf16 inputs with ``convert_to_float32=True``: operands of 11 significant bits.  The result must be closer to
    the fp32 oracle than the plain bf16 path's (and inside the fp16 bound, up to the bf16 rounding of the output)."""
    B, N, T, D, scale = 1, 2, 200, 64, 1 / 8
    ins = orc.make_inputs(B, N, T, D, seed=5, dtype=torch.bfloat16)
    f = [x.float() for x in ins]
    z_ref, _ = orc.tdp_forward(*f[:5], scale, True)
    g_ref = orc.tdp_backward(*f, scale, True)
    out_w, g_w = _run(ins, scale, True, convert_to_float32=True)
    out_n, g_n = _run(ins, scale, True)
    assert _native.read_status(torch.device(DEV)) == 0
    assert out_w.dtype == torch.bfloat16
    err = lambda a, b: float((a.float() - b).norm() / b.norm())
    assert err(out_w, z_ref) < err(out_n, z_ref)
    for name, a, n, b in zip(("dq", "dk1", "dk2", "dv1", "dv2"), g_w, g_n, g_ref):
        assert err(a, b) < err(n, b), name
        assert_close(name, a, b, torch.bfloat16, scale=0.5)


def test_input_beyond_the_fp16_range_sets_the_status_bit():
    B, N, T, D = 1, 1, 64, 64
    ins = orc.make_inputs(B, N, T, D, seed=9, dtype=torch.float32)
    ins[1][0, 0, 3, 5] = 1.0e6
    t = [x.to(DEV) for x in ins[:5]]
    o, lse = torch.empty_like(t[0]), torch.empty(B, N, T, device=DEV)
    _native.tdp_fwd(*t, o, lse, 1 / 8, True, None, None, None, None)
    assert _native.read_status(torch.device(DEV)) == 64
    # the exact-fp32 kernels take such data
    _native.tdp_fwd(*t, o, lse, 1 / 8, True, None, None, None, None, flags=_native.FLAG_FORCE_SIMT)
    assert _native.read_status(torch.device(DEV)) == 0
    assert torch.isfinite(o).all()
