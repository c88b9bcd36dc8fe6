"""The ``torch.library`` operators and the ``TrittentionTDP`` module.

Without a GPU: registration, schemas, shape propagation on the meta device (forward and through autograd) and the
``ValueError`` checks.  With a GPU: the operators give the results of the reference-style entry points (same library
calls: the forward bit for bit, the gradients up to the order of the fp32 reduce-adds), ``torch.library.opcheck`` passes, and a function compiled with ``fullgraph=True`` calls them
without a graph break."""
import pytest
import torch

from flash_trittention import ops, TrittentionTDP
from oracle import trittention_oracle as orc

DEV = "cuda:0"


def _same_grads(a, b):
    """Two runs of a backward agree up to the summation order of its fp32 atomic accumulation."""
    for x, y in zip(a, b):
        gx, gy = x.grad.float(), y.grad.float()
        assert float((gx - gy).abs().max()) <= 8e-3 * float(gx.abs().max())  # one bf16 ulp of the largest element


def _meta(shape=(2, 3, 64, 32), dtype=torch.bfloat16, grad=True):
    return [torch.empty(*shape, device="meta", dtype=dtype, requires_grad=grad) for _ in range(5)]


def test_operators_are_registered_with_schemas():
    ns = torch.ops.flash_trittention
    for name in ("tdp_fwd", "tdp_bwd", "dps_fwd", "dps_bwd"):
        assert hasattr(ns, name)
    schema = str(ns.tdp_fwd.default._schema)
    assert "? k1_window" in schema and "bool causal" in schema and "-> (Tensor, Tensor)" in schema
    assert str(ns.dps_bwd.default._schema).count("Tensor") >= 13


def test_shapes_propagate_on_the_meta_device():
    t = _meta()
    o, lse = ops.tdp_attention(*t, 0.1, True, None, 8, 4, None)
    assert o.shape == t[0].shape and o.dtype == torch.bfloat16
    assert lse.shape == t[0].shape[:3] and lse.dtype == torch.float32
    assert o.requires_grad and not lse.requires_grad
    o.sum().backward()
    assert all(x.grad is not None and x.grad.shape == x.shape and x.grad.dtype == x.dtype for x in t)
    t = _meta(dtype=torch.float16)
    o, m = ops.dps_attention(*t, 0.125, True, 16)
    assert o.shape == t[0].shape and m.shape == t[0].shape[:3] and not m.requires_grad
    o.sum().backward()
    assert all(x.grad is not None and x.grad.shape == x.shape for x in t)


def test_module_mirrors_the_dot_product_sum_module():
    mod = TrittentionTDP(causal=True, softmax_scale=0.2, k1_window=5, kk_right=0)
    assert "k1_window=5" in repr(mod)
    o, lse = mod(*_meta(grad=False))
    assert o.shape == (2, 3, 64, 32) and lse.shape == (2, 3, 64)


def test_mismatched_inputs_raise_value_error():
    t = _meta(grad=False)
    with pytest.raises(ValueError, match="does not match q shape"):
        ops.tdp_attention(t[0], t[1], t[2], t[3], torch.empty(2, 3, 64, 16, device="meta", dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="dtype"):
        ops.dps_attention(t[0], t[1].float(), t[2], t[3], t[4])
    with pytest.raises(ValueError, match="power of 2"):
        ops.tdp_attention(*[torch.empty(1, 1, 8, 24, device="meta") for _ in range(5)])
    with pytest.raises(ValueError, match="batch, heads, seq_len, head_dim"):
        ops.tdp_attention(*[torch.empty(8, 16, device="meta") for _ in range(5)])


def test_cpu_tensors_have_no_implementation():
    with pytest.raises(NotImplementedError):
        ops.tdp_attention(*[torch.zeros(1, 1, 8, 8) for _ in range(5)])


# ------------------------------------------------------------------ GPU

def _gpu_inputs(B, N, T, D, dtype, seed):
    q, k1, k2, v1, v2, dz = orc.make_inputs(B, N, T, D, seed=seed, dtype=dtype)
    return [x.to(DEV) for x in (q, k1, k2, v1, v2)], dz.to(DEV)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,D,win", [(torch.bfloat16, 64, (None, None, None, None)),
                                         (torch.float16, 128, (40, 200, 16, 8)),
                                         (torch.float32, 32, (None, 20, None, 3))])
def test_tdp_operator_equals_the_entry_point(dtype, D, win):
    from flash_trittention import flash_trittention

    t, dz = _gpu_inputs(1, 2, 192, D, dtype, 301)
    a = [x.clone().requires_grad_(True) for x in t]
    b = [x.clone().requires_grad_(True) for x in t]
    k1w, k2w, kkl, kkr = win
    out_a = flash_trittention(*a, softmax_scale=1 / D, kk_left=kkl, kk_right=kkr, k1_window=k1w, k2_window=k2w,
                              causal=True)
    out_b, lse = TrittentionTDP(True, 1 / D, k1w, k2w, kkl, kkr)(*b)
    out_a.backward(dz)
    out_b.backward(dz)
    if dtype == torch.float32:  # the CUDA-core kernels sum a query's partial results with shared-memory atomics
        assert float((out_a - out_b).abs().max()) <= 1e-5
    else:
        assert torch.equal(out_a, out_b)
    assert torch.isfinite(lse).all()
    _same_grads(a, b)
    # and against the oracle, at the tolerance of the other parity tests
    ref = orc.tdp_forward(*[x.float().cpu() for x in t], 1 / D, True, k1w, k2w, kkl, kkr)[0]
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert float((out_b.float().cpu() - ref).abs().max()) <= tol


@pytest.mark.gpu
def test_dps_operator_equals_the_module():
    from flash_trittention import TrittentionTriton

    t, dz = _gpu_inputs(1, 2, 128, 32, torch.float16, 303)
    a = [x.clone().requires_grad_(True) for x in t]
    b = [x.clone().requires_grad_(True) for x in t]
    out_a, m_a = TrittentionTriton(causal=True, softmax_scale=0.125, k_diff=48)(*a)
    out_b, m_b = ops.dps_attention(*b, 0.125, True, 48)
    out_a.backward(dz)
    out_b.backward(dz)
    assert torch.equal(out_a, out_b) and torch.equal(m_a, m_b)
    _same_grads(a, b)


@pytest.mark.gpu
def test_opcheck():
    t, _ = _gpu_inputs(1, 1, 64, 32, torch.float32, 305)
    t = [x.requires_grad_(True) for x in t]
    checks = ("test_schema", "test_faketensor", "test_autograd_registration")
    torch.library.opcheck(torch.ops.flash_trittention.tdp_fwd.default, (*t, 0.1, True, None, 16, 8, None, False),
                          test_utils=checks)
    torch.library.opcheck(torch.ops.flash_trittention.dps_fwd.default, (*t, 0.1, True, 16), test_utils=checks)


@pytest.mark.gpu
def test_compiled_function_has_no_graph_break():
    from flash_trittention import flash_trittention

    t, dz = _gpu_inputs(1, 2, 128, 64, torch.bfloat16, 307)

    def f(q, k1, k2, v1, v2):
        return flash_trittention(q * 1.0, k1, k2, v1, v2, softmax_scale=1 / 64, kk_left=None, kk_right=None,
                                 k1_window=None, k2_window=64, causal=True) + 0.0

    eager = [x.clone().requires_grad_(True) for x in t]
    comp = [x.clone().requires_grad_(True) for x in t]
    out_e = f(*eager)
    out_e.backward(dz)
    # the "aot_eager" backend traces forward and backward graphs through the operators without a code generator
    out_c = torch.compile(f, fullgraph=True, backend="aot_eager")(*comp)
    out_c.backward(dz)
    assert torch.equal(out_e, out_c)
    _same_grads(eager, comp)
