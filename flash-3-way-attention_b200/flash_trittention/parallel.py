"""Multi-GPU use of triple-dot-product trittention (one process per GPU, ``torch.distributed``).

The reference has no distributed code.  Two partitionings are offered here:

* head sharding - ``(batch*head)`` slices are independent, so every rank simply calls
  ``flash_trittention`` on its slice (``shard_heads``); no collective is involved;
* query-row sharding (``flash_trittention_query_sharded``) for problems with fewer
  ``batch*head`` slices than GPUs: K1, K2, V1, V2 are replicated, rank ``r`` of ``W`` owns the query
  rows ``q`` with ``q % W == r`` (interleaved, because the causal cost of row ``q`` grows like
  ``(q+1)^2``), computes their outputs and their ``dQ`` rows, and contributes fp32 partial sums of
  the key-side gradients that are summed by one all-reduce (NCCL over NVLink on GPUs) before the
  final cast and SiLU derivative.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from . import _native


def shard_heads(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Slice ``[B, N, T, D]`` into this rank's contiguous share of the ``B*N`` (batch*head) slices,
    returned as ``[1, B*N/world, T, D]``."""
    B, N, T, D = t.shape
    if (B * N) % world:
        raise ValueError(f"{B * N} (batch*head) slices do not divide over {world} ranks")
    per = B * N // world
    return t.reshape(B * N, T, D)[rank * per:(rank + 1) * per].reshape(1, per, T, D)


def owned_rows(T: int, rank: int, world: int) -> torch.Tensor:
    """Query rows owned by ``rank`` under interleaved sharding."""
    return torch.arange(rank, T, world)


def _supported_world(world: int) -> bool:
    return world >= 1 and world <= 64 and (world & (world - 1)) == 0


class _QueryShardedTrittention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k1, k2, v1, v2, softmax_scale, causal, group):
        world = dist.get_world_size(group)
        rank = dist.get_rank(group)
        if not _supported_world(world):
            raise ValueError(f"query sharding needs a power-of-two group size <= 64, got {world}")
        q, k1, k2, v1, v2 = (t.contiguous() for t in (q, k1, k2, v1, v2))
        o = torch.zeros_like(q)
        lse = torch.zeros(q.shape[:3], dtype=torch.float32, device=q.device)
        _native.tdp_fwd(q, k1, k2, v1, v2, o, lse, softmax_scale, causal, None, None, None, None,
                        q_mod=world, q_rem=rank)
        # rows are disjoint across ranks: a sum is a gather
        o32 = o.float()
        dist.all_reduce(o32, group=group)
        dist.all_reduce(lse, group=group)
        o = o32.to(q.dtype)
        ctx.save_for_backward(q, k1, k2, v1, v2, o, lse)
        ctx.softmax_scale, ctx.causal, ctx.group = softmax_scale, causal, group
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k1, k2, v1, v2, o, lse = ctx.saved_tensors
        group = ctx.group
        world = dist.get_world_size(group)
        rank = dist.get_rank(group)
        d_o = d_o.contiguous().to(q.dtype)
        dq = torch.zeros_like(q)
        ws = _native.tdp_bwd(q, k1, k2, v1, v2, o, d_o, lse, dq, None, None, None, None, ctx.softmax_scale,
                             ctx.causal, None, None, None, None, q_mod=world, q_rem=rank,
                             flags=_native.FLAG_BWD_PARTIAL)
        n = q.numel()
        partials = ws[: 16 * n].view(torch.float32)  # dK1 | dK2 | dSiLU(V1) | dV2, fp32
        dist.all_reduce(partials, group=group)
        dq32 = dq.float()
        dist.all_reduce(dq32, group=group)
        dk1, dk2, dv1, dv2 = (torch.empty_like(q) for _ in range(4))
        _native.tdp_bwd_finalize(v1, dk1, dk2, dv1, dv2, ws)
        return dq32.to(q.dtype), dk1, dk2, dv1, dv2, None, None, None


def flash_trittention_query_sharded(q, k1, k2, v1, v2, softmax_scale: float = 1 / 8, causal: bool = True,
                                    group: Optional[dist.ProcessGroup] = None):
    """Triple-dot-product trittention (full windows) with the query rows split over the ranks of ``group``.

    Every rank passes the same full ``[B, N, T, D]`` tensors and receives the full output; gradients
    returned by autograd are complete on every rank.
    """
    return _QueryShardedTrittention.apply(q, k1, k2, v1, v2, softmax_scale, causal, group)
