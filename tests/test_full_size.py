"""Parity at the sequence lengths and head dimensions of the benchmark configurations, where the dense oracle
cannot run.  Triple-dot-product (T=2048, D=128 and T=4096, D=64, bf16, causal, alpha = 1/D): sampled query rows
against an fp32 per-row evaluation of the same formulas, and size-independent properties of the backward (linearity
in the upstream gradient, query-row shards summing to the full gradient).  Dot-product-sum (T=1024, D=64, fp16):
the whole result against the factorised fp32 formulation on the CPU."""
import pytest
import torch

from oracle import trittention_oracle as orc
from flash_trittention import _native

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 2e-2  # max-abs error of bf16 results against fp32, relative to max(1, magnitude)


def _row_reference(q, k1, k2, v1, v2, do, o, alpha, rows):
    """fp32 evaluation of a few query rows of one head (tensors [T, D] on the GPU, TF32 off): returns
    O[rows], lse[rows], dQ[rows].  Formulas: S = alpha (Q[q] * K1) K2^T over j, k <= q; P = softmax;
    O = sum_jk P SiLU(V1[j]) V2[k]; dP = (dO * SiLU(V1)) V2^T; dS = P (dP - sum_h dO O); dQ = alpha sum_jk dS K1[j] K2[k]."""
    sv1 = torch.nn.functional.silu(v1)
    outs, lses, dqs = [], [], []
    for r in rows:
        n = r + 1
        s = alpha * ((q[r] * k1[:n]) @ k2[:n].T)          # [j, k]
        m = s.max()
        e = torch.exp(s - m)
        l = e.sum()
        p = e / l
        o_r = ((p @ v2[:n]) * sv1[:n]).sum(0)             # sum_j SiLU(V1[j]) * sum_k P[j,k] V2[k]
        dp = (do[r] * sv1[:n]) @ v2[:n].T
        ds = p * (dp - (do[r] * o_r).sum())
        dq = alpha * ((ds @ k2[:n]) * k1[:n]).sum(0)
        outs.append(o_r)
        lses.append(m + torch.log(l))
        dqs.append(dq)
    return torch.stack(outs), torch.stack(lses), torch.stack(dqs)


@pytest.mark.parametrize("T,D", [(2048, 128), (4096, 64)])
def test_sampled_rows_at_benchmark_sizes(T, D):
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        B, N, alpha = 1, 2, 1.0 / D
        q, k1, k2, v1, v2, dz = orc.make_inputs(B, N, T, D, scale=0.5, seed=101, dtype=torch.bfloat16)
        t = [x.to(DEV) for x in (q, k1, k2, v1, v2)]
        do = dz.to(DEV)
        o, lse = torch.empty_like(t[0]), torch.empty(B, N, T, device=DEV)
        _native.tdp_fwd(*t, o, lse, alpha, True, None, None, None, None)
        g = [torch.empty_like(t[0]) for _ in range(5)]
        _native.tdp_bwd(*t, o, do, lse, *g, alpha, True, None, None, None, None)
        torch.cuda.synchronize()
        assert _native.read_status(torch.device(DEV)) == 0
        rows = [0, 1, 63, 64, 127, 128, 129, 255, 256, T // 2 - 1, T // 2, T - 129, T - 128, T - 2, T - 1]
        for h in range(N):
            f = [x[0, h].float() for x in t]
            o_ref, lse_ref, dq_ref = _row_reference(*f, do[0, h].float(), o[0, h].float(), alpha, rows)
            assert float((o[0, h, rows].float() - o_ref).abs().max()) <= TOL
            assert float((lse[0, h, rows] - lse_ref).abs().max()) <= TOL
            mag = max(1.0, float(dq_ref.abs().max()))
            assert float((g[0][0, h, rows].float() - dq_ref).abs().max()) <= TOL * mag
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
        ref = 2 * a - b
        mag = max(1.0, float(ref.abs().max()))
        assert float((c - ref).abs().max()) <= 3 * TOL * mag, name


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
    assert float((o2.float() - o.float()).abs().max()) <= 1e-2
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
        mag = max(1.0, float(b.float().abs().max()))
        assert float((a.float() - b.float()).abs().max()) <= TOL * mag, name


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
    assert float((out.detach().float().cpu() - z_ref.detach()).abs().max()) <= 5e-3
    assert float((m.cpu() - lse_ref.detach()).abs().max()) <= 5e-3
    for name, leaf, ref in zip(("dq", "dk1", "dk2", "dv1", "dv2"), leaves, ref_leaves):
        g, r = leaf.grad.float().cpu(), ref.grad
        assert float((g - r).abs().max()) <= 5e-3 * max(1.0, float(r.abs().max())), name
