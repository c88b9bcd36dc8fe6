"""Parity at the sequence lengths and head dimensions of the benchmark configurations, where the dense oracle
cannot run on the host.  Triple-dot-product (T=2048, D=128 and T=4096, D=64, bf16, causal, alpha = 1/D): whole
heads (output, log-sum-exp, all five gradients) against the oracle evaluated in fp32 on the GPU, and
size-independent properties of the backward (linearity in the upstream gradient, query-row shards summing to the
full gradient).  Dot-product-sum (T=1024, D=64, fp16):
the whole result against the factorised fp32 formulation on the CPU."""
import pytest
import torch

from _parity import assert_close, fmt
from oracle import trittention_oracle as orc
from flash_trittention import _native

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("T,D,heads_checked,dtype", [(2048, 128, 2, torch.bfloat16), (4096, 64, 1, torch.bfloat16),
                                                    (2048, 64, 1, torch.float16)])
def test_whole_heads_at_benchmark_sizes(T, D, heads_checked, dtype):
    """Output, log-sum-exp and all five gradients of whole heads at the benchmark shapes (causal, full windows,
    inputs N(0,1)*0.5, alpha = 1/D) against the oracle evaluated in fp32 on the GPU (TF32 off).  Every tensor is
    bounded against its own magnitude; the normalised errors are printed (run pytest with -s).  The fp16 case
    is there for the probabilities of late rows (~1/q^2 = 2e-7 at q = 2048), which lie below fp16's normal range."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        B, N, alpha = 1, 2, 1.0 / D
        q, k1, k2, v1, v2, dz = orc.make_inputs(B, N, T, D, scale=0.5, seed=101, dtype=dtype)
        t = [x.to(DEV) for x in (q, k1, k2, v1, v2)]
        do = dz.to(DEV)
        o, lse = torch.empty_like(t[0]), torch.empty(B, N, T, device=DEV)
        _native.tdp_fwd(*t, o, lse, alpha, True, None, None, None, None)
        g = [torch.empty_like(t[0]) for _ in range(5)]
        _native.tdp_bwd(*t, o, do, lse, *g, alpha, True, None, None, None, None)
        torch.cuda.synchronize()
        assert _native.read_status(torch.device(DEV)) == 0
        chunk = max(1, (1 << 27) // (T * T))  # 512 MiB per [chunk, T, T] fp32 intermediate
        for h in range(heads_checked):
            f = [x[:, h:h + 1].float() for x in t]
            z_ref, lse_ref = orc.tdp_forward(*f, alpha, True, chunk=chunk, device=DEV)
            g_ref = orc.tdp_backward(*f, do[:, h:h + 1].float(), alpha, True, chunk=chunk, device=DEV)
            rep = {}
            try:
                assert_close("o", o[:, h:h + 1], z_ref, dtype, report=rep)
                # late rows are averages over ~T^2 terms and therefore tiny: check them on their own as well
                assert_close("o[T/2:]", o[:, h:h + 1, T // 2:], z_ref[:, :, T // 2:], dtype, report=rep)
                assert float((lse[:, h:h + 1] - lse_ref).abs().max()) <= 5e-3
                for name, got, ref in zip(("dq", "dk1", "dk2", "dv1", "dv2"), g, g_ref):
                    assert_close(name, got[:, h:h + 1], ref, dtype, report=rep)
            finally:
                print(f"\nT={T} D={D} {dtype} head {h}: {fmt(rep)}")
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def test_backward_is_linear_in_the_upstream_gradient_at_benchmark_size():
    B, N, T, D, alpha = 1, 2, 2048, 128, 1.0 / 128
    q, k1, k2, v1, v2, dz = orc.make_inputs(B, N, T, D, scale=0.5, seed=103, dtype=torch.bfloat16)
    t = [x.to(DEV) for x in (q, k1, k2, v1, v2)]
    o, lse = torch.empty_like(t[0]), torch.empty(B, N, T, device=DEV)
    _native.tdp_fwd(*t, o, lse, alpha, True, None, None, None, None)
    do_a = dz.to(DEV)
    do_b = torch.roll(do_a, shifts=7, dims=2).contiguous()

    def grads(do):
        g = [torch.empty_like(t[0]) for _ in range(5)]
        _native.tdp_bwd(*t, o, do, lse, *g, alpha, True, None, None, None, None)
        return [x.float() for x in g]

    ga, gb = grads(do_a), grads(do_b)
    # 2 a - b is exactly representable only up to bf16 rounding of the sum: the tolerance covers it
    gc = grads((2 * do_a.float() - do_b.float()).to(torch.bfloat16))
    torch.cuda.synchronize()
    assert _native.read_status(torch.device(DEV)) == 0
    for name, a, b, c in zip(("dq", "dk1", "dk2", "dv1", "dv2"), ga, gb, gc):
        # three bf16-rounded results and a bf16-rounded input combination enter: twice the single-result bound
        assert_close(name, c, 2 * a - b, torch.bfloat16, scale=2.0)


def test_query_shards_sum_to_the_full_gradient_at_benchmark_size():
    B, N, T, D, alpha = 1, 1, 2048, 128, 1.0 / 128
    q, k1, k2, v1, v2, dz = orc.make_inputs(B, N, T, D, scale=0.5, seed=107, dtype=torch.bfloat16)
    t = [x.to(DEV) for x in (q, k1, k2, v1, v2)]
    do = dz.to(DEV)
    o, lse = torch.empty_like(t[0]), torch.empty(B, N, T, device=DEV)
    _native.tdp_fwd(*t, o, lse, alpha, True, None, None, None, None)
    o2, lse2 = torch.zeros_like(o), torch.zeros_like(lse)
    for rem in range(8):
        _native.tdp_fwd(*t, o2, lse2, alpha, True, None, None, None, None, q_mod=8, q_rem=rem)
    assert_close("o (shards vs whole)", o2, o, torch.bfloat16)
    assert float((lse2 - lse).abs().max()) <= 1e-3
    full = [torch.empty_like(t[0]) for _ in range(5)]
    _native.tdp_bwd(*t, o, do, lse, *full, alpha, True, None, None, None, None)
    dq = torch.zeros_like(t[0])
    n = t[0].numel()
    acc = torch.zeros(4 * n, device=DEV)
    for rem in range(8):
        ws = _native.tdp_bwd(*t, o, do, lse, dq, None, None, None, None, alpha, True, None, None, None, None,
                             q_mod=8, q_rem=rem, flags=_native.FLAG_BWD_PARTIAL)
        acc += ws[: 16 * n].view(torch.float32)
    ws = _native.workspace(_native.OP_TDP_BWD, B, N, T, D, _native.BF16, DEV)
    ws[: 16 * n].view(torch.float32).copy_(acc)
    outs = [torch.empty_like(t[0]) for _ in range(4)]
    _native.tdp_bwd_finalize(t[3], *outs, ws)
    torch.cuda.synchronize()
    assert _native.read_status(torch.device(DEV)) == 0
    for name, a, b in zip(("dq", "dk1", "dk2", "dv1", "dv2"), [dq] + outs, full):
        assert_close(name + " (shards vs whole)", a, b, torch.bfloat16)


def _dps_factorised(q, k1, k2, v1, v2, a, k_diff):
    """Differentiable fp32 restatement of the dot-product-sum variant as two chained soft-max attentions
    (inner over s per K2 row t, outer over t per query; causal, t - s <= k_diff), as in the oracle's
    ``dps_forward_factorised``."""
    T = q.shape[-2]
    sv1 = torch.nn.functional.silu(v1)
    E = a * torch.matmul(k1, k2.transpose(-1, -2))
    s = torch.arange(T).view(-1, 1)
    t = torch.arange(T).view(1, -1)
    E = E.masked_fill(~((s <= t) & (t - s <= k_diff)), float("-inf"))
    lse_in = torch.logsumexp(E, dim=-2)
    Y = torch.matmul(torch.exp(E - lse_in[..., None, :]).transpose(-1, -2), sv1)
    Fq = a * torch.matmul(q, k2.transpose(-1, -2)) + lse_in[..., None, :]
    Fq = Fq.masked_fill(~(t <= s), float("-inf"))
    lse = torch.logsumexp(Fq, dim=-1)
    return torch.matmul(torch.exp(Fq - lse[..., None]), Y * v2), lse


def test_dot_product_sum_at_benchmark_size():
    """Config 3 shape per head (T=1024, D=64, fp16, alpha = 1/8, causal, k_diff = T), two heads."""
    from flash_trittention.dot_product_sum.trittention_triton import TrittentionTriton

    B, N, T, D, a = 1, 2, 1024, 64, 1 / 8
    q, k1, k2, v1, v2, dz = orc.make_inputs(B, N, T, D, seed=109, dtype=torch.float16)
    leaves = [x.to(DEV).requires_grad_(True) for x in (q, k1, k2, v1, v2)]
    out, m = TrittentionTriton(causal=True, softmax_scale=a, k_diff=T)(*leaves)
    out.backward(dz.to(DEV))
    torch.cuda.synchronize()
    assert _native.read_status(torch.device(DEV)) == 0
    ref_leaves = [x.float().requires_grad_(True) for x in (q, k1, k2, v1, v2)]
    z_ref, lse_ref = _dps_factorised(*ref_leaves, a, T)
    z_ref.backward(dz.float())
    assert_close("o", out.detach().cpu(), z_ref.detach(), torch.float16)
    assert float((m.cpu() - lse_ref.detach()).abs().max()) <= 5e-3
    for name, leaf, ref in zip(("dq", "dk1", "dk2", "dv1", "dv2"), leaves, ref_leaves):
        assert_close(name, leaf.grad.cpu(), ref.grad, torch.float16)
