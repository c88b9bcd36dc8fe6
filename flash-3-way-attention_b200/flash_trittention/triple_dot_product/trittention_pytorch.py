"""Dense PyTorch formulation of triple-dot-product trittention (``Trittention_pytorch``).

Kept for interface parity with ``src/flash_trittention/triple_dot_product/trittention_pytorch.py``
of the reference, where it is the ground truth the kernels are tested against.  It
materialises the full ``[B, N, T, T, T]`` score cube, so it is for small problems only.
It is a stand-alone module: nothing in the CUDA path calls it.
"""
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .kernels.utils import process_masking_variables


class Trittention_pytorch(nn.Module):
    def __init__(
        self,
        causal: bool = True,
        softmax_scale: float = 1 / 8,
        n_ctx: int = 1024,
        k1_window: Optional[int] = None,
        k2_window: Optional[int] = None,
        kk_left: Optional[int] = None,
        kk_right: Optional[int] = None,
    ):
        super().__init__()
        self.n_ctx = n_ctx
        self.softmax_scale = softmax_scale
        self.causal = causal
        self.k1_window, self.k2_window, self.kk_left, self.kk_right = process_masking_variables(
            n_ctx, k1_window, k2_window, kk_left, kk_right)

    def masked_positions(self, T: int, device) -> torch.Tensor:
        """``[T(j), T(k), T(q)]`` boolean tensor, True where the triple is NOT attended."""
        j = torch.arange(T, device=device).view(T, 1, 1)
        k = torch.arange(T, device=device).view(1, T, 1)
        q = torch.arange(T, device=device).view(1, 1, T)
        attended = (
            (j <= q) & (q <= j + self.k1_window) & (k <= q) & (q <= k + self.k2_window)
            & (k <= j + self.kk_left) & (j <= k + self.kk_right)
        )
        return ~attended

    def forward(self, q, k1, k2, v1, v2):
        T = q.shape[2]
        scores = torch.einsum("bnjh,bnkh,bnqh->bnjkq", k1, k2, q)
        if self.causal:
            scores = scores.masked_fill(self.masked_positions(T, q.device), -1e6)
        pre_softmax = scores
        flat = scores.permute(0, 1, 4, 2, 3).reshape(*q.shape[:3], T * T) * self.softmax_scale
        M = flat.max(dim=-1)[0]
        L = torch.exp(flat - M.unsqueeze(-1)).sum(dim=-1) + 0.01
        probs = flat.softmax(dim=-1)
        v_gated = F.silu(v1.unsqueeze(3)) * v2.unsqueeze(2)  # [b, n, j, k, h]
        z = torch.einsum("bnql,bnlh->bnqh", probs, v_gated.reshape(*q.shape[:2], T * T, q.shape[-1]))
        return z, pre_softmax, v_gated, M, L
