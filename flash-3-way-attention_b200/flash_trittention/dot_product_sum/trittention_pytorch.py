"""Dense PyTorch formulation of dot-product-sum trittention (``Trittention_pytorch``).

Kept for interface parity with ``src/flash_trittention/dot_product_sum/trittention_pytorch.py``
of the reference (its ground truth).  Materialises ``[B, N, T, T, T]``; small problems only.
Nothing in the CUDA path calls it.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F


class Trittention_pytorch(nn.Module):
    def __init__(self, causal: bool = True, softmax_scale: float = 1 / 8, n_ctx: int = 1024, k_diff: int = 1024):
        super().__init__()
        self.n_ctx = n_ctx
        self.softmax_scale = softmax_scale
        self.causal = causal
        self.k_diff = k_diff

    def masked_positions(self, T: int, device) -> torch.Tensor:
        """``[T(s: K1 index), T(t: K2 index), T(q)]``, True where NOT attended:
        attended iff ``s <= t <= q`` and ``t - s <= k_diff``."""
        s = torch.arange(T, device=device).view(T, 1, 1)
        t = torch.arange(T, device=device).view(1, T, 1)
        q = torch.arange(T, device=device).view(1, 1, T)
        return ~((s <= t) & (t <= q) & (t - s <= self.k_diff))

    def forward(self, q, k1, k2, v1, v2):
        T = q.shape[2]
        qk = torch.einsum("bnth,bnqh->bntq", k2, q)
        kk = torch.einsum("bnsh,bnth->bnst", k1, k2)
        scores = qk.unsqueeze(2) + kk.unsqueeze(-1)  # [b, n, s, t, q]
        if self.causal:
            scores = scores.masked_fill(self.masked_positions(T, q.device), -1e6)
        pre_softmax = scores
        flat = scores.permute(0, 1, 4, 2, 3).reshape(*q.shape[:3], T * T) * self.softmax_scale
        M = torch.logsumexp(flat, dim=-1)
        probs = flat.softmax(dim=-1)
        v_gated = F.silu(v1.unsqueeze(3)) * v2.unsqueeze(2)  # [b, n, s, t, h]
        z = torch.einsum("bnql,bnlh->bnqh", probs, v_gated.reshape(*q.shape[:2], T * T, q.shape[-1]))
        return z, pre_softmax, v_gated, M
