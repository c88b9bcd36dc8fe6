"""CPU oracle for three-way ("trittention") attention.  TEST INFRASTRUCTURE ONLY.

This module is the checker that the CUDA kernels are compared against.  It is
imported by the test-suite, by the smoke check and by the CPU-baseline leg of the
benchmark; the product code never imports it and never falls back to it.

It restates, in plain PyTorch on the CPU (fp32 by default, fp64 on request), the
algorithm of the reference implementation's naive einsum modules:

* triple-dot-product (TDP): ``src/flash_trittention/triple_dot_product/trittention_pytorch.py:78-102``
  (forward) with the mask of ``:45-76`` and ``kernels/utils.py:6-17`` (``None`` window -> seq_len);
* dot-product-sum (DPS): ``src/flash_trittention/dot_product_sum/trittention_pytorch.py:54-82``
  with the mask of ``:24-52``.

Differences from the reference modules, none of which change results at fp32
resolution: masked logits are ``-inf`` instead of ``-1e6`` (the reference's fill
underflows to exactly 0 after the soft-max as well), the ``L + 0.01`` diagnostic is
not reproduced (no caller reads it), queries are processed in chunks so that the
``[T, T, T]`` score cube is never materialised, the 3-operand einsum is written as a
pre-scaled dense matmul, and the backward pass is written out explicitly instead
of being left to autograd.

Parity pin: ``tests/golden/*.npz`` hold outputs *and* gradients produced by the
reference modules themselves (autograd through them) on seeded inputs;
``tests/test_oracle_golden.py`` checks this file against every one of them.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

__all__ = [
    "resolve_windows",
    "tdp_valid_mask",
    "tdp_forward",
    "tdp_backward",
    "dps_valid_mask",
    "dps_forward",
    "dps_backward",
    "dps_forward_factorised",
    "tdp_valid_triples",
    "tdp_flops",
    "make_inputs",
]


# --------------------------------------------------------------------------- helpers
def resolve_windows(seq_len: int, k1_window, k2_window, kk_left, kk_right):
    """``None`` means "the whole sequence" (reference ``kernels/utils.py:6-17``)."""
    f = lambda w: seq_len if w is None else int(w)
    return f(k1_window), f(k2_window), f(kk_left), f(kk_right)


def tdp_valid_mask(q_idx: torch.Tensor, T: int, causal: bool, windows) -> Optional[torch.Tensor]:
    """Boolean ``[len(q_idx), T(j), T(k)]`` tensor, True where (q, j, k) is attended.

    Negation of the reference's fill predicate
    (``triple_dot_product/trittention_pytorch.py:68-75``): valid iff
    ``j <= q <= j + k1_window``, ``k <= q <= k + k2_window`` and
    ``k - kk_left <= j <= k + kk_right``.  Non-causal: everything is valid.
    """
    if not causal:
        return None
    k1w, k2w, kkl, kkr = windows
    q = q_idx.view(-1, 1, 1)
    j = torch.arange(T, device=q_idx.device).view(1, -1, 1)
    k = torch.arange(T, device=q_idx.device).view(1, 1, -1)
    return (
        (j <= q) & (q <= j + k1w) & (k <= q) & (q <= k + k2w) & (j + kkl >= k) & (k + kkr >= j)
    )


def dps_valid_mask(q_idx: torch.Tensor, T: int, causal: bool, k_diff: int) -> Optional[torch.Tensor]:
    """Boolean ``[len(q_idx), T(s: K1/V1 index), T(t: K2/V2 index)]``.

    Reference ``dot_product_sum/trittention_pytorch.py:47-51`` (its first index is
    the K1 position, its second the K2 position): valid iff ``s <= t <= q`` and
    ``t - s <= k_diff``.  Non-causal: everything is valid and ``k_diff`` is ignored.
    """
    if not causal:
        return None
    q = q_idx.view(-1, 1, 1)
    s = torch.arange(T).view(1, -1, 1)
    t = torch.arange(T).view(1, 1, -1)
    return (s <= t) & (t <= q) & (t - s <= k_diff)


def _silu_grad(x: torch.Tensor) -> torch.Tensor:
    sig = torch.sigmoid(x)
    return sig * (1 + x * (1 - sig))


def _chunks(T: int, chunk: int):
    for q0 in range(0, T, chunk):
        yield q0, min(T, q0 + chunk)


def _auto_chunk(T: int, chunk: Optional[int]) -> int:
    if chunk is not None:
        return max(1, int(chunk))
    # keep chunk*T*T*4 bytes around 64 MiB
    return max(1, min(T, (16 << 20) // max(1, T * T)))


# --------------------------------------------------------------------------- TDP
def _tdp_scores(qc, k1, k2, alpha):
    """S[c, j, k] = alpha * sum_h qc[c,h] k1[j,h] k2[k,h] as a dense matmul."""
    a = qc[:, None, :] * k1[None, :, :]  # [c, j, h]
    return alpha * torch.matmul(a, k2.t())  # [c, j, k]


def tdp_forward(
    q, k1, k2, v1, v2, softmax_scale: float, causal: bool = True,
    k1_window=None, k2_window=None, kk_left=None, kk_right=None,
    chunk: Optional[int] = None, dtype=torch.float32, device="cpu",
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(z [B,N,T,D], lse [B,N,T])`` (natural-log log-sum-exp of the scaled logits).

    ``device``: where the restatement is evaluated.  The default is the CPU; the benchmark-size parity tests
    pass a CUDA device (with TF32 matmuls switched off) because one head at T = 2048 takes minutes on host cores.
    """
    B, N, T, D = q.shape
    windows = resolve_windows(T, k1_window, k2_window, kk_left, kk_right)
    q, k1, k2, v1, v2 = (t.detach().to(device, dtype) for t in (q, k1, k2, v1, v2))
    z = torch.empty(B, N, T, D, dtype=dtype, device=device)
    lse = torch.empty(B, N, T, dtype=dtype, device=device)
    ch = _auto_chunk(T, chunk)
    for b in range(B):
        for n in range(N):
            sv1 = F.silu(v1[b, n])
            for q0, q1 in _chunks(T, ch):
                s = _tdp_scores(q[b, n, q0:q1], k1[b, n], k2[b, n], softmax_scale)
                m = tdp_valid_mask(torch.arange(q0, q1, device=device), T, causal, windows)
                if m is not None:
                    s = s.masked_fill(~m, float("-inf"))
                l = torch.logsumexp(s.reshape(q1 - q0, -1), dim=-1)
                p = torch.exp(s - l[:, None, None])
                # z[c,h] = sum_jk p[c,j,k] sv1[j,h] v2[k,h]
                u = torch.matmul(p, v2[b, n])  # [c, j, h]
                z[b, n, q0:q1] = (u * sv1[None]).sum(1)
                lse[b, n, q0:q1] = l
    return z, lse


def tdp_backward(
    q, k1, k2, v1, v2, dz, softmax_scale: float, causal: bool = True,
    k1_window=None, k2_window=None, kk_left=None, kk_right=None,
    chunk: Optional[int] = None, dtype=torch.float32, device="cpu",
):
    """Explicit backward; returns ``(dq, dk1, dk2, dv1, dv2)`` (on ``device``, see ``tdp_forward``).

    With ``sV1 = SiLU(V1)``, ``Dq = sum_h dZ*Z``, ``dP = sum_h dZ[q] sV1[j] V2[k]`` and
    ``dS = P * (dP - Dq)``: ``dQ = a*sum_jk dS K1 K2``, ``dK1 = a*sum_qk dS Q K2``,
    ``dK2 = a*sum_qj dS Q K1``, ``dsV1 = sum_qk P dZ V2``, ``dV2 = sum_qj P dZ sV1``,
    ``dV1 = dsV1 * SiLU'(V1)`` (reference ``flash_trittention.py:390-391``).
    """
    B, N, T, D = q.shape
    windows = resolve_windows(T, k1_window, k2_window, kk_left, kk_right)
    q, k1, k2, v1, v2, dz = (t.detach().to(device, dtype) for t in (q, k1, k2, v1, v2, dz))
    dq = torch.zeros_like(q)
    dk1 = torch.zeros_like(q)
    dk2 = torch.zeros_like(q)
    dsv1 = torch.zeros_like(q)
    dv2 = torch.zeros_like(q)
    ch = _auto_chunk(T, chunk)
    a = softmax_scale
    for b in range(B):
        for n in range(N):
            K1, K2, V2 = k1[b, n], k2[b, n], v2[b, n]
            sv1 = F.silu(v1[b, n])
            for q0, q1 in _chunks(T, ch):
                Qc, dZc = q[b, n, q0:q1], dz[b, n, q0:q1]
                s = _tdp_scores(Qc, K1, K2, a)
                m = tdp_valid_mask(torch.arange(q0, q1, device=device), T, causal, windows)
                if m is not None:
                    s = s.masked_fill(~m, float("-inf"))
                l = torch.logsumexp(s.reshape(q1 - q0, -1), dim=-1)
                p = torch.exp(s - l[:, None, None])  # [c,j,k]
                u = torch.matmul(p, V2)  # [c,j,h] = sum_k p v2
                zc = (u * sv1[None]).sum(1)
                Dq = (dZc * zc).sum(-1)
                dp = torch.matmul(dZc[:, None, :] * sv1[None], V2.t())  # [c,j,k]
                ds = p * (dp - Dq[:, None, None])
                g = torch.matmul(ds, K2)  # [c,j,h] = sum_k ds k2
                dq[b, n, q0:q1] = a * (g * K1[None]).sum(1)
                dk1[b, n] += a * (g * Qc[:, None, :]).sum(0)
                gt = torch.matmul(ds.transpose(1, 2), K1)  # [c,k,h] = sum_j ds k1
                dk2[b, n] += a * (gt * Qc[:, None, :]).sum(0)
                dsv1[b, n] += (u * dZc[:, None, :]).sum(0)
                ut = torch.matmul(p.transpose(1, 2), sv1)  # [c,k,h] = sum_j p sv1
                dv2[b, n] += (ut * dZc[:, None, :]).sum(0)
    dv1 = dsv1 * _silu_grad(v1)
    return dq, dk1, dk2, dv1, dv2


# --------------------------------------------------------------------------- DPS
def _dps_scores(qc, k1, k2, alpha):
    """S[c, s, t] = alpha * (qc[c].k2[t] + k1[s].k2[t])."""
    qk = torch.matmul(qc, k2.t())  # [c, t]
    kk = torch.matmul(k1, k2.t())  # [s, t]
    return alpha * (qk[:, None, :] + kk[None, :, :])


def dps_forward(
    q, k1, k2, v1, v2, softmax_scale: float, causal: bool = True, k_diff: int = 1024,
    chunk: Optional[int] = None, dtype=torch.float32,
):
    """Direct (three-index) restatement.  Returns ``(z, lse)``; ``lse`` is what the
    reference kernels return as ``m`` (``dot_product_sum/kernels/fwd_kernel.py:366-370``)."""
    B, N, T, D = q.shape
    q, k1, k2, v1, v2 = (t.detach().to("cpu", dtype) for t in (q, k1, k2, v1, v2))
    z = torch.empty(B, N, T, D, dtype=dtype)
    lse = torch.empty(B, N, T, dtype=dtype)
    ch = _auto_chunk(T, chunk)
    for b in range(B):
        for n in range(N):
            sv1 = F.silu(v1[b, n])
            for q0, q1 in _chunks(T, ch):
                s = _dps_scores(q[b, n, q0:q1], k1[b, n], k2[b, n], softmax_scale)
                m = dps_valid_mask(torch.arange(q0, q1), T, causal, k_diff)
                if m is not None:
                    s = s.masked_fill(~m, float("-inf"))
                l = torch.logsumexp(s.reshape(q1 - q0, -1), dim=-1)
                p = torch.exp(s - l[:, None, None])  # [c, s, t]
                u = torch.matmul(p, v2[b, n])  # [c, s, h]
                z[b, n, q0:q1] = (u * sv1[None]).sum(1)
                lse[b, n, q0:q1] = l
    return z, lse


def dps_backward(
    q, k1, k2, v1, v2, dz, softmax_scale: float, causal: bool = True, k_diff: int = 1024,
    chunk: Optional[int] = None, dtype=torch.float32,
):
    """Explicit backward of the direct form; returns ``(dq, dk1, dk2, dv1, dv2)``."""
    B, N, T, D = q.shape
    q, k1, k2, v1, v2, dz = (t.detach().to("cpu", dtype) for t in (q, k1, k2, v1, v2, dz))
    dq = torch.zeros_like(q)
    dk1 = torch.zeros_like(q)
    dk2 = torch.zeros_like(q)
    dsv1 = torch.zeros_like(q)
    dv2 = torch.zeros_like(q)
    ch = _auto_chunk(T, chunk)
    a = softmax_scale
    for b in range(B):
        for n in range(N):
            K1, K2, V2 = k1[b, n], k2[b, n], v2[b, n]
            sv1 = F.silu(v1[b, n])
            for q0, q1 in _chunks(T, ch):
                Qc, dZc = q[b, n, q0:q1], dz[b, n, q0:q1]
                s = _dps_scores(Qc, K1, K2, a)
                m = dps_valid_mask(torch.arange(q0, q1), T, causal, k_diff)
                if m is not None:
                    s = s.masked_fill(~m, float("-inf"))
                l = torch.logsumexp(s.reshape(q1 - q0, -1), dim=-1)
                p = torch.exp(s - l[:, None, None])  # [c,s,t]
                u = torch.matmul(p, V2)  # [c,s,h]
                zc = (u * sv1[None]).sum(1)
                Dq = (dZc * zc).sum(-1)
                dp = torch.matmul(dZc[:, None, :] * sv1[None], V2.t())  # [c,s,t]
                ds = p * (dp - Dq[:, None, None])
                ds_t = ds.sum(1)  # [c,t]
                ds_st = ds.sum(0)  # [s,t]
                dq[b, n, q0:q1] = a * torch.matmul(ds_t, K2)
                dk2[b, n] += a * (torch.matmul(ds_t.t(), Qc) + torch.matmul(ds_st.t(), K1))
                dk1[b, n] += a * torch.matmul(ds_st, K2)
                dsv1[b, n] += (u * dZc[:, None, :]).sum(0)
                ut = torch.matmul(p.transpose(1, 2), sv1)  # [c,t,h]
                dv2[b, n] += (ut * dZc[:, None, :]).sum(0)
    dv1 = dsv1 * _silu_grad(v1)
    return dq, dk1, dk2, dv1, dv2


def dps_forward_factorised(
    q, k1, k2, v1, v2, softmax_scale: float, causal: bool = True, k_diff: int = 1024,
    dtype=torch.float32,
):
    """O(T^2 D) restatement: the separable score makes DPS two chained soft-max
    attentions (the reference kernels use the same two-level log-sum-exp,
    ``dot_product_sum/kernels/fwd_kernel.py:102-108,196-204``).

    inner (per K2 row t):  E[s,t] = a K1[s].K2[t],  LSEin[t],  Y[t] = softmax_s(E) sV1
    outer (per query q):   F[q,t] = a Q[q].K2[t] + LSEin[t],  Z = softmax_t(F) (Y*V2)
    """
    B, N, T, D = q.shape
    q, k1, k2, v1, v2 = (t.detach().to("cpu", dtype) for t in (q, k1, k2, v1, v2))
    a = softmax_scale
    sv1 = F.silu(v1)
    E = a * torch.matmul(k1, k2.transpose(-1, -2))  # [B,N,s,t]
    if causal:
        s = torch.arange(T).view(-1, 1)
        t = torch.arange(T).view(1, -1)
        E = E.masked_fill(~((s <= t) & (t - s <= k_diff)), float("-inf"))
    lse_in = torch.logsumexp(E, dim=-2)  # [B,N,t]
    Ain = torch.exp(E - lse_in[..., None, :])
    Y = torch.matmul(Ain.transpose(-1, -2), sv1)  # [B,N,t,h]
    Fq = a * torch.matmul(q, k2.transpose(-1, -2)) + lse_in[..., None, :]  # [B,N,q,t]
    if causal:
        qi = torch.arange(T).view(-1, 1)
        t = torch.arange(T).view(1, -1)
        Fq = Fq.masked_fill(~(t <= qi), float("-inf"))
    lse = torch.logsumexp(Fq, dim=-1)
    A = torch.exp(Fq - lse[..., None])
    z = torch.matmul(A, Y * v2)
    return z, lse


# --------------------------------------------------------------------------- work model
def tdp_valid_triples(B: int, N: int, T: int, causal: bool = True) -> int:
    """Number of attended (q, j, k) triples with full windows."""
    per_head = T * (T + 1) * (2 * T + 1) // 6 if causal else T ** 3
    return B * N * per_head


def tdp_flops(B: int, N: int, T: int, D: int, causal: bool = True, mode: str = "fwd+bwd") -> float:
    """Algorithmic flops: forward 2 GEMM-shaped contractions (4*D per triple),
    backward 6 (12*D per triple)."""
    per = {"fwd": 4, "bwd": 12, "fwd+bwd": 16}[mode]
    return float(per * D * tdp_valid_triples(B, N, T, causal))


# --------------------------------------------------------------------------- inputs
def make_inputs(B, N, T, D, scale: float = 1.0, seed: int = 0, dtype=torch.float32, n: int = 6):
    """Seeded synthetic tensors, drawn in the order Q, K1, K2, V1, V2, dZ as fp32
    ``randn`` on a CPU generator, scaled, then cast."""
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        out.append((torch.randn(B, N, T, D, generator=g, dtype=torch.float32) * scale).to(dtype))
    return out
