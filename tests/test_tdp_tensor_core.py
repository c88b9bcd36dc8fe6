"""Parity of the tensor-core (tcgen05) triple-dot-product path with the fp32 CPU oracle on
the same 16-bit-rounded inputs.  Every result tensor (output and each of the five gradients) is bounded
against its own magnitude: max|err| <= 2e-2 max|ref| (bf16) / 5e-3 max|ref| (fp16), and the same two
figures for the relative rms error, so that an all-zero or mis-scaled tensor fails whatever its size."""
import pytest
import torch

from _parity import assert_close, fmt
from oracle import trittention_oracle as orc
from flash_trittention import _native
from flash_trittention.triple_dot_product.flash_trittention import flash_trittention

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.bfloat16: 2e-2, torch.float16: 5e-3}


def _fwd_case(B, N, T, D, dtype, causal, scale_in, alpha, seed, o_scale=1.0):
    q, k1, k2, v1, v2, _ = orc.make_inputs(B, N, T, D, scale=scale_in, seed=seed, dtype=dtype)
    code = _native.dtype_code(dtype)
    assert _native.tdp_path(_native.OP_TDP_FWD, T, D, code, causal, None, None, None, None) == _native.PATH_TCGEN05
    dq, dk1, dk2, dv1, dv2 = (t.to(DEV) for t in (q, k1, k2, v1, v2))
    o = torch.empty_like(dq)
    lse = torch.empty(B, N, T, device=DEV)
    _native.tdp_fwd(dq, dk1, dk2, dv1, dv2, o, lse, alpha, causal, None, None, None, None)
    torch.cuda.synchronize()
    assert _native.read_status(torch.device(DEV)) == 0, "a bounded barrier wait ran out"
    z_ref, lse_ref = orc.tdp_forward(*(t.float() for t in (q, k1, k2, v1, v2)), alpha, causal)
    rep = {}
    assert_close("o", o.cpu(), z_ref, dtype, scale=o_scale, report=rep)
    print(f"\nfwd T={T} D={D} {dtype} causal={causal}: {fmt(rep)}")
    lerr = float((lse.cpu() - lse_ref).abs().max())
    return lerr


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("windows", [(None, None, None, None), (100, 70, 40, 30)])
def test_forward_heads_with_small_and_large_logits_in_one_launch(D, dtype, windows):
    """The forward picks the soft-max warps' organisation per head from a head-wide score bound (column split with
    the row's bound as reference / one warpgroup per tile with row maxima).  Heads of both kinds alternate here, so
    every CTA changes organisation between consecutive work items and the same barriers serve both."""
    B, N, T, alpha = 1, 6, 300, 1 / 8
    q, k1, k2, v1, v2, _ = orc.make_inputs(B, N, T, D, scale=1.0, seed=41 + D, dtype=torch.float32)
    head_scale = torch.tensor([0.25, 1.5, 0.25, 1.5, 1.5, 0.25]).view(1, N, 1, 1)
    q, k1, k2 = ((t * head_scale).to(dtype) for t in (q, k1, k2))
    v1, v2 = v1.to(dtype), v2.to(dtype)
    dev = [t.to(DEV) for t in (q, k1, k2, v1, v2)]
    o = torch.empty_like(dev[0])
    lse = torch.empty(B, N, T, device=DEV)
    _native.tdp_fwd(*dev, o, lse, alpha, True, *windows)
    torch.cuda.synchronize()
    assert _native.read_status(torch.device(DEV)) == 0, "a bounded barrier wait ran out"
    z_ref, lse_ref = orc.tdp_forward(*(t.float() for t in (q, k1, k2, v1, v2)), alpha, True, *windows)
    for h in range(N):   # per head: the large-logit heads would otherwise hide the small ones
        assert_close(f"o[head {h}]", o[:, h].cpu(), z_ref[:, h], dtype)
    # The log-sum-exp carries the absolute rounding error of the row's largest logit (one 16-bit rounding of the
    # operand A: 2^-9 relative for bf16); the large-logit heads reach |logit| ~ 25, hence five times the usual bound.
    tol = 2e-2 if dtype == torch.bfloat16 else 5e-3
    lerr = (lse.cpu() - lse_ref).abs().amax(dim=(0, 2))
    for h in range(N):
        assert float(lerr[h]) <= tol * (5.0 if float(head_scale[0, h, 0, 0]) > 1 else 1.0), (h, float(lerr[h]))


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("T", [40, 64, 100, 129, 256, 333])
@pytest.mark.parametrize("causal", [True, False])
def test_forward_bf16_matches_oracle(T, D, causal):
    if not causal and T > 256:
        pytest.skip("dense oracle too slow")
    lerr = _fwd_case(1, 2, T, D, torch.bfloat16, causal, 0.5, 1.0 / D, seed=T + D)
    assert lerr <= 5e-3, lerr


@pytest.mark.parametrize("D", [64, 128])
def test_forward_fp16_matches_oracle(D):
    lerr = _fwd_case(2, 2, 200, D, torch.float16, True, 0.5, 1.0 / D, seed=3)
    assert lerr <= 1e-3, lerr


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_forward_reference_test_distribution(dtype, D, causal):
    """The reference tests' own setting (tests/test_triple_dot_product.py:51-96 there): N(0,1) inputs with
    alpha = 1/8.  Logits are of order 1-10, so the running maximum moves (accumulator rescaling) and the
    16-bit rounding of the pre-product Q*K2 shows in the scores."""
    lerr = _fwd_case(1, 2, 192 if causal else 96, D, dtype, causal, 1.0, 1 / 8, seed=17 + D)
    assert lerr <= (2e-2 if dtype == torch.bfloat16 else 5e-3), lerr


def test_forward_matches_cuda_core_path_and_query_shards():
    B, N, T, D = 1, 3, 300, 64
    q, k1, k2, v1, v2, _ = orc.make_inputs(B, N, T, D, scale=0.5, seed=5, dtype=torch.bfloat16)
    t = [x.to(DEV) for x in (q, k1, k2, v1, v2)]
    o_ref, lse_ref = torch.empty_like(t[0]), torch.empty(B, N, T, device=DEV)
    _native.tdp_fwd(*t, o_ref, lse_ref, 1 / D, True, None, None, None, None, flags=_native.FLAG_FORCE_SIMT)
    o, lse = torch.zeros_like(t[0]), torch.zeros(B, N, T, device=DEV)
    for rem in range(4):
        _native.tdp_fwd(*t, o, lse, 1 / D, True, None, None, None, None, q_mod=4, q_rem=rem)
    torch.cuda.synchronize()
    assert _native.read_status(torch.device(DEV)) == 0
    assert_close("o vs cuda-core path", o, o_ref, torch.bfloat16)
    assert float((lse - lse_ref).abs().max()) <= 5e-3


def test_autograd_entry_point_uses_tensor_core_forward():
    B, N, T, D = 1, 2, 128, 64
    q, k1, k2, v1, v2, dz = orc.make_inputs(B, N, T, D, scale=0.5, seed=8, dtype=torch.bfloat16)
    leaves = [x.to(DEV).requires_grad_(True) for x in (q, k1, k2, v1, v2)]
    out = flash_trittention(*leaves, 1 / D, None, None, None, None, True)
    out.backward(dz.to(DEV))
    torch.cuda.synchronize()
    f = [x.float() for x in (q, k1, k2, v1, v2)]
    z_ref, _ = orc.tdp_forward(*f, 1 / D, True)
    g_ref = orc.tdp_backward(*f, dz.float(), 1 / D, True)
    assert_close("o", out.cpu(), z_ref, torch.bfloat16)
    for name, leaf, ref in zip(("dq", "dk1", "dk2", "dv1", "dv2"), leaves, g_ref):
        assert_close(name, leaf.grad.cpu(), ref, torch.bfloat16)


def _bwd_case(B, N, T, D, dtype, causal, scale_in, alpha, seed):
    q, k1, k2, v1, v2, dz = orc.make_inputs(B, N, T, D, scale=scale_in, seed=seed, dtype=dtype)
    code = _native.dtype_code(dtype)
    assert _native.tdp_path(_native.OP_TDP_BWD, T, D, code, causal, None, None, None, None) == _native.PATH_TCGEN05
    leaves = [x.to(DEV).requires_grad_(True) for x in (q, k1, k2, v1, v2)]
    out = flash_trittention(*leaves, alpha, None, None, None, None, causal)
    out.backward(dz.to(DEV))
    torch.cuda.synchronize()
    assert _native.read_status(torch.device(DEV)) == 0, "a bounded barrier wait ran out"
    f = [x.float() for x in (q, k1, k2, v1, v2)]
    g_ref = orc.tdp_backward(*f, dz.float(), alpha, causal)
    rep = {}
    try:
        for name, leaf, ref in zip(("dq", "dk1", "dk2", "dv1", "dv2"), leaves, g_ref):
            assert_close(name, leaf.grad.cpu(), ref, dtype, report=rep)
    finally:
        print(f"\nbwd T={T} D={D} {dtype} causal={causal}: {fmt(rep)}")


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("T", [40, 64, 100, 129, 256])
@pytest.mark.parametrize("causal", [True, False])
def test_backward_bf16_matches_oracle(T, D, causal):
    _bwd_case(1, 2, T, D, torch.bfloat16, causal, 0.5, 1.0 / D, seed=2 * T + D)


@pytest.mark.parametrize("D", [64, 128])
def test_backward_fp16_matches_oracle(D):
    _bwd_case(2, 2, 200, D, torch.float16, True, 0.5, 1.0 / D, seed=4)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_backward_reference_test_distribution(dtype, D, causal):
    """All five gradients on the reference tests' distribution (N(0,1), alpha = 1/8), both 16-bit types, both
    head dimensions, causal and not."""
    _bwd_case(1, 2, 160 if causal else 96, D, dtype, causal, 1.0, 1 / 8, seed=19 + D)


@pytest.mark.parametrize("dtype,causal,T", [(torch.bfloat16, True, 384), (torch.float16, True, 200),
                                            (torch.bfloat16, False, 192)])
def test_backward_on_cta_pairs_matches_oracle_and_default_path(dtype, causal, T):
    """TRITT_FLAG_BWD_CTA_PAIRS: the backward kernel as clusters of two CTAs (cta_group::2 products over two queries
    that share every key / value tile).  Checked against the oracle with the usual bounds, and against the default
    one-CTA-per-item launch, from which it may differ only by the order of the fp32 reduce-adds."""
    B, N, D, alpha = 1, 3, 128, 1 / 128
    q, k1, k2, v1, v2, dz = orc.make_inputs(B, N, T, D, scale=0.5, seed=31 + T, dtype=dtype)
    t = [x.to(DEV) for x in (q, k1, k2, v1, v2)]
    do = dz.to(DEV)
    o, lse = torch.empty_like(t[0]), torch.empty(B, N, T, device=DEV)
    _native.tdp_fwd(*t, o, lse, alpha, causal, None, None, None, None)
    base = [torch.empty_like(t[0]) for _ in range(5)]
    _native.tdp_bwd(*t, o, do, lse, *base, alpha, causal, None, None, None, None)
    pair = [torch.full_like(t[0], float("nan")) for _ in range(5)]
    _native.tdp_bwd(*t, o, do, lse, *pair, alpha, causal, None, None, None, None, flags=_native.FLAG_BWD_CTA_PAIRS)
    torch.cuda.synchronize()
    assert _native.read_status(torch.device(DEV)) == 0
    ref = orc.tdp_backward(q.float(), k1.float(), k2.float(), v1.float(), v2.float(), dz.float(), alpha, causal)
    for name, got, want, same in zip(("dq", "dk1", "dk2", "dv1", "dv2"), pair, ref, base):
        assert_close(name + " (pairs)", got, want, dtype)
        assert_close(name + " (pairs vs default launch)", got, same, torch.float32, scale=100.0)


def test_backward_query_shards_sum_to_full_gradient():
    """Query-sharded backward: each shard writes its rows of dq and leaves fp32 partial key-side sums;
    their sum, finalised once, equals the unsharded gradients (the multi-device path does the sum with
    an all-reduce)."""
    B, N, T, D, alpha = 1, 2, 200, 64, 1 / 64
    q, k1, k2, v1, v2, dz = orc.make_inputs(B, N, T, D, scale=0.5, seed=23, dtype=torch.bfloat16)
    t = [x.to(DEV) for x in (q, k1, k2, v1, v2)]
    do = dz.to(DEV)
    o, lse = torch.empty_like(t[0]), torch.empty(B, N, T, device=DEV)
    _native.tdp_fwd(*t, o, lse, alpha, True, None, None, None, None)
    full = [torch.empty_like(t[0]) for _ in range(5)]
    _native.tdp_bwd(*t, o, do, lse, *full, alpha, True, None, None, None, None)
    dq = torch.zeros_like(t[0])
    n = t[0].numel()
    acc = torch.zeros(4 * n, device=DEV)
    for rem in range(4):
        ws = _native.tdp_bwd(*t, o, do, lse, dq, None, None, None, None, alpha, True, None, None, None, None,
                             q_mod=4, q_rem=rem, flags=_native.FLAG_BWD_PARTIAL)
        acc += ws[: 16 * n].view(torch.float32)
    ws = _native.workspace(_native.OP_TDP_BWD, B, N, T, D, _native.BF16, DEV)
    ws[: 16 * n].view(torch.float32).copy_(acc)
    outs = [torch.empty_like(t[0]) for _ in range(4)]
    _native.tdp_bwd_finalize(t[3], *outs, ws)
    torch.cuda.synchronize()
    assert _native.read_status(torch.device(DEV)) == 0
    for name, a, b in zip(("dq", "dk1", "dk2", "dv1", "dv2"), [dq] + outs, full):
        assert_close(name + " (shards vs whole)", a, b, torch.bfloat16)


WINDOWS = [
    (8, 8, 4, 4),          # the reference tests' narrow band (tests/test_triple_dot_product.py)
    (128, 128, 32, 32),    # the reference's banded forward benchmark (b200/bench_b200.py)
    (300, 100, 50, 20),
    (100, 300, 20, 50),
    (10, 1000, 3, 5),      # k2 window far wider than k1 window + band: rows that see no column at all
    (1000, 10, 300, 0),
    (1, 1, 1, 1),          # the entry point's defaults
    (0, 0, 0, 0),          # only j = k = q
    (200, 200, 0, 200),
]


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("windows", WINDOWS)
def test_forward_windows_match_oracle(windows, D):
    """Causal mask with k1 / k2 windows and the (j, k) band on the tensor-core forward."""
    B, N, T, dtype = 1, 2, 333, torch.bfloat16
    q, k1, k2, v1, v2, _ = orc.make_inputs(B, N, T, D, scale=0.5, seed=11 + D, dtype=dtype)
    code = _native.dtype_code(dtype)
    assert _native.tdp_path(_native.OP_TDP_FWD, T, D, code, True, *windows) == _native.PATH_TCGEN05
    dq, dk1, dk2, dv1, dv2 = (t.to(DEV) for t in (q, k1, k2, v1, v2))
    o = torch.empty_like(dq)
    lse = torch.empty(B, N, T, device=DEV)
    _native.tdp_fwd(dq, dk1, dk2, dv1, dv2, o, lse, 1.0 / D, True, *windows)
    torch.cuda.synchronize()
    assert _native.read_status(torch.device(DEV)) == 0, "a bounded barrier wait ran out"
    z_ref, lse_ref = orc.tdp_forward(*(t.float() for t in (q, k1, k2, v1, v2)), 1.0 / D, True, *windows)
    assert torch.isfinite(lse).all()
    assert_close("o", o.cpu(), z_ref, dtype)
    assert float((lse.cpu() - lse_ref).abs().max()) <= 5e-3


def test_forward_windows_large_logits_fp16():
    """Unit-variance inputs with alpha = 1/8 under a narrow band: rows whose first slab is empty and a moving maximum."""
    B, N, T, D, dtype = 1, 2, 400, 64, torch.float16
    windows = (150, 90, 40, 10)
    q, k1, k2, v1, v2, _ = orc.make_inputs(B, N, T, D, scale=1.0, seed=23, dtype=dtype)
    dq, dk1, dk2, dv1, dv2 = (t.to(DEV) for t in (q, k1, k2, v1, v2))
    o = torch.empty_like(dq)
    lse = torch.empty(B, N, T, device=DEV)
    _native.tdp_fwd(dq, dk1, dk2, dv1, dv2, o, lse, 1 / 8, True, *windows)
    torch.cuda.synchronize()
    assert _native.read_status(torch.device(DEV)) == 0
    z_ref, _ = orc.tdp_forward(*(t.float() for t in (q, k1, k2, v1, v2)), 1 / 8, True, *windows)
    assert_close("o", o.cpu(), z_ref, dtype)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("windows", WINDOWS)
def test_backward_windows_match_oracle(windows, D):
    """All five gradients under k1 / k2 windows and the (j, k) band, through the autograd entry point."""
    B, N, T, dtype = 1, 2, 300, torch.bfloat16
    alpha = 1.0 / D
    q, k1, k2, v1, v2, dz = orc.make_inputs(B, N, T, D, scale=0.5, seed=31 + D, dtype=dtype)
    code = _native.dtype_code(dtype)
    assert _native.tdp_path(_native.OP_TDP_BWD, T, D, code, True, *windows) == _native.PATH_TCGEN05
    leaves = [x.to(DEV).requires_grad_(True) for x in (q, k1, k2, v1, v2)]
    k1w, k2w, kkl, kkr = windows
    out = flash_trittention(*leaves, alpha, kkl, kkr, k1w, k2w, True)
    out.backward(dz.to(DEV))
    torch.cuda.synchronize()
    assert _native.read_status(torch.device(DEV)) == 0, "a bounded barrier wait ran out"
    f = [x.float() for x in (q, k1, k2, v1, v2)]
    g_ref = orc.tdp_backward(*f, dz.float(), alpha, True, *windows)
    # windows (0, 0, 0, 0): every query attends the single pair (q, q), so dQ, dK1 and dK2 are exactly zero and the
    # oracle's values for them are fp32 rounding noise (~1e-8, against ~1e-3 for the other window sets)
    for name, leaf, ref in zip(("dq", "dk1", "dk2", "dv1", "dv2"), leaves, g_ref):
        assert_close(name, leaf.grad.cpu(), ref, dtype, zero_below=1e-6 if windows == (0, 0, 0, 0) else 0.0)


@pytest.mark.parametrize("windows", [(64, 150, 30, 10), (8, 8, 4, 4)])
def test_windows_with_query_shards(windows):
    """Query-row sharding under a windowed mask: forward shards write disjoint rows, backward shards leave fp32
    partial key-side sums whose total, finalised once, equals the unsharded gradients."""
    B, N, T, D, alpha = 1, 2, 300, 64, 1 / 64
    q, k1, k2, v1, v2, dz = orc.make_inputs(B, N, T, D, scale=0.5, seed=29, dtype=torch.bfloat16)
    t = [x.to(DEV) for x in (q, k1, k2, v1, v2)]
    do = dz.to(DEV)
    o, lse = torch.empty_like(t[0]), torch.empty(B, N, T, device=DEV)
    _native.tdp_fwd(*t, o, lse, alpha, True, *windows)
    o2, lse2 = torch.zeros_like(o), torch.zeros_like(lse)
    for rem in range(4):
        _native.tdp_fwd(*t, o2, lse2, alpha, True, *windows, q_mod=4, q_rem=rem)
    assert_close("o (shards vs whole)", o2, o, torch.bfloat16)
    assert float((lse2 - lse).abs().max()) <= 1e-3
    full = [torch.empty_like(t[0]) for _ in range(5)]
    _native.tdp_bwd(*t, o, do, lse, *full, alpha, True, *windows)
    dq = torch.zeros_like(t[0])
    n = t[0].numel()
    acc = torch.zeros(4 * n, device=DEV)
    for rem in range(4):
        ws = _native.tdp_bwd(*t, o, do, lse, dq, None, None, None, None, alpha, True, *windows,
                             q_mod=4, q_rem=rem, flags=_native.FLAG_BWD_PARTIAL)
        acc += ws[: 16 * n].view(torch.float32)
    ws = _native.workspace(_native.OP_TDP_BWD, B, N, T, D, _native.BF16, DEV)
    ws[: 16 * n].view(torch.float32).copy_(acc)
    outs = [torch.empty_like(t[0]) for _ in range(4)]
    _native.tdp_bwd_finalize(t[3], *outs, ws)
    torch.cuda.synchronize()
    assert _native.read_status(torch.device(DEV)) == 0
    for name, a, b in zip(("dq", "dk1", "dk2", "dv1", "dv2"), [dq] + outs, full):
        assert_close(name + " (shards vs whole)", a, b, torch.bfloat16)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_forward_with_and_without_the_score_bound(dtype):
    """The forward takes the score bound |A_row| max|K1_j| as soft-max reference when the workspace has the tail for
    the K1 row norms, and the two-pass row maximum when it has not: same result up to the rounding of P."""
    B, N, T, D, alpha = 1, 2, 384, 128, 1.0 / 128
    q, k1, k2, v1, v2, _ = orc.make_inputs(B, N, T, D, scale=0.5, seed=77, dtype=dtype)
    t = [x.to(DEV) for x in (q, k1, k2, v1, v2)]
    n = B * N * T * D
    outs = []
    for ws in (None, torch.empty(n * 2, dtype=torch.uint8, device=DEV)):
        o, lse = torch.empty_like(t[0]), torch.empty(B, N, T, device=DEV)
        _native.tdp_fwd(*t, o, lse, alpha, True, None, None, None, None, ws=ws)
        torch.cuda.synchronize()
        assert _native.read_status(torch.device(DEV)) == 0
        outs.append((o.float(), lse))
    assert_close("o (score bound vs two-pass)", outs[0][0], outs[1][0], dtype)
    assert float((outs[0][1] - outs[1][1]).abs().max()) <= 1e-3
    z_ref, lse_ref = orc.tdp_forward(*[x.float() for x in (q, k1, k2, v1, v2)], alpha, True)
    for o, lse in outs:
        assert_close("o", o.cpu(), z_ref, dtype)
        assert float((lse.cpu() - lse_ref).abs().max()) <= 5e-3
