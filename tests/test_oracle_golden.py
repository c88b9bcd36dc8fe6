"""The CPU oracle must reproduce every fixture generated from the reference's own
naive einsum modules (outputs and all five gradients)."""
import os

import numpy as np
import pytest
import torch

from conftest import golden_cases
from oracle import trittention_oracle as orc


def _load(path):
    d = np.load(path)
    t = {k: torch.from_numpy(d[k]) for k in ("q", "k1", "k2", "v1", "v2", "dz", "z", "dq", "dk1", "dk2", "dv1", "dv2")}
    meta = {k: d[k].item() for k in d.files if d[k].ndim == 0 and k != "variant"}
    return t, meta


def _win(meta):
    f = lambda v: None if v < 0 else int(v)
    return dict(k1_window=f(meta["k1_window"]), k2_window=f(meta["k2_window"]),
                kk_left=f(meta["kk_left"]), kk_right=f(meta["kk_right"]))


@pytest.mark.parametrize("path", golden_cases("tdp_"), ids=os.path.basename)
def test_tdp_oracle_matches_reference_fixture(path):
    t, meta = _load(path)
    kw = dict(softmax_scale=meta["softmax_scale"], causal=bool(meta["causal"]), **_win(meta))
    z, lse = orc.tdp_forward(t["q"], t["k1"], t["k2"], t["v1"], t["v2"], chunk=7, **kw)
    torch.testing.assert_close(z, t["z"], rtol=1e-4, atol=2e-5)
    grads = orc.tdp_backward(t["q"], t["k1"], t["k2"], t["v1"], t["v2"], t["dz"], chunk=7, **kw)
    for name, g in zip(("dq", "dk1", "dk2", "dv1", "dv2"), grads):
        torch.testing.assert_close(g, t[name], rtol=1e-4, atol=5e-5, msg=lambda m, n=name: f"{n}: {m}")
    assert torch.isfinite(lse).all()


@pytest.mark.parametrize("path", golden_cases("dps_"), ids=os.path.basename)
def test_dps_oracle_matches_reference_fixture(path):
    t, meta = _load(path)
    kw = dict(softmax_scale=meta["softmax_scale"], causal=bool(meta["causal"]), k_diff=int(meta["k_diff"]))
    z, lse = orc.dps_forward(t["q"], t["k1"], t["k2"], t["v1"], t["v2"], chunk=5, **kw)
    torch.testing.assert_close(z, t["z"], rtol=1e-4, atol=2e-5)
    zf, lsef = orc.dps_forward_factorised(t["q"], t["k1"], t["k2"], t["v1"], t["v2"], **kw)
    torch.testing.assert_close(zf, t["z"], rtol=1e-4, atol=2e-5)
    torch.testing.assert_close(lsef, lse, rtol=1e-5, atol=1e-4)
    grads = orc.dps_backward(t["q"], t["k1"], t["k2"], t["v1"], t["v2"], t["dz"], chunk=5, **kw)
    # logits of several hundred leave ~1e-4 of fp32 rounding in the reference's own run
    atol = 2e-3 if "large_logits" in path else 1e-4
    for name, g in zip(("dq", "dk1", "dk2", "dv1", "dv2"), grads):
        torch.testing.assert_close(g, t[name], rtol=2e-4, atol=atol, msg=lambda m, n=name: f"{n}: {m}")


def test_explicit_backward_matches_autograd_fp64():
    """The hand-written backward formulas agree with autograd through a dense fp64 einsum."""
    B, N, T, D = 1, 1, 12, 8
    q, k1, k2, v1, v2, dz = orc.make_inputs(B, N, T, D, seed=3, dtype=torch.float64)
    leaves = [x.clone().requires_grad_(True) for x in (q, k1, k2, v1, v2)]
    Q, K1, K2, V1, V2 = leaves
    s = 0.3 * torch.einsum("bnqh,bnjh,bnkh->bnqjk", Q, K1, K2)
    m = orc.tdp_valid_mask(torch.arange(T), T, True, (5, 7, 2, 3))
    s = s.masked_fill(~m, float("-inf"))
    p = torch.softmax(s.reshape(B, N, T, -1), -1).reshape(B, N, T, T, T)
    z = torch.einsum("bnqjk,bnjh,bnkh->bnqh", p, torch.nn.functional.silu(V1), V2)
    z.backward(dz)
    z2, _ = orc.tdp_forward(q, k1, k2, v1, v2, 0.3, True, 5, 7, 2, 3, dtype=torch.float64)
    torch.testing.assert_close(z2, z.detach(), rtol=1e-10, atol=1e-12)
    grads = orc.tdp_backward(q, k1, k2, v1, v2, dz, 0.3, True, 5, 7, 2, 3, dtype=torch.float64)
    for g, leaf in zip(grads, leaves):
        torch.testing.assert_close(g, leaf.grad, rtol=1e-9, atol=1e-11)


def test_flop_model():
    # 1*16 heads, T=2048: 4.585e10 attended triples, 93.89 TFLOP forward+backward at D=128
    v = orc.tdp_valid_triples(1, 16, 2048)
    assert abs(v / 4.585e10 - 1) < 1e-3
    assert abs(orc.tdp_flops(1, 16, 2048, 128) / 93.89e12 - 1) < 1e-3
