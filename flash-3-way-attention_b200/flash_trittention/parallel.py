"""Multi-GPU use of triple-dot-product trittention (one process per GPU, ``torch.distributed``).

The reference has no distributed code.  Two partitionings are offered here:

* head sharding - ``(batch*head)`` slices are independent, so every rank simply calls
  ``flash_trittention`` on its slice (``shard_heads``); no collective is involved;
* query-row sharding (``flash_trittention_query_sharded``) for problems with fewer
  ``batch*head`` slices than GPUs: K1, K2, V1, V2 are replicated, rank ``r`` of ``W`` owns the query
  rows ``q`` with ``q % W == r`` (interleaved, because the causal cost of row ``q`` grows like
  ``(q+1)^2``), computes their outputs and their ``dQ`` rows, and contributes fp32 partial sums of
  the key-side gradients that are summed by one all-reduce (NCCL over NVLink on GPUs) before the
  final cast and SiLU derivative.  The forward needs no exchange (an optional all-gather hands every rank the full
  output); the backward has that one all-reduce plus an all-gather of the ``dQ`` rows.
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


def _gather_rows(x: torch.Tensor, rank: int, world: int, group) -> torch.Tensor:
    """All ranks hold ``x`` ``[B, N, T, D]`` with only their own interleaved rows (``q % world == rank``) filled in;
    returns the tensor with every row filled in.  One all-gather of the rows in the tensor's own (16-bit) type: each
    rank contributes ``ceil(T / world)`` rows (the last one padded when ``T`` does not divide)."""
    B, N, T, D = x.shape
    per = (T + world - 1) // world
    mine = x[:, :, rank::world, :]
    send = x.new_zeros(B, N, per, D)
    send[:, :, : mine.shape[2]] = mine
    recv = x.new_empty(world, B, N, per, D)
    dist.all_gather_into_tensor(recv.view(-1), send.view(-1), group=group)
    out = torch.empty_like(x)
    for r in range(world):
        n = (T - r + world - 1) // world
        out[:, :, r::world, :] = recv[r, :, :, :n]
    return out


class _QueryShardedTrittention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k1, k2, v1, v2, softmax_scale, causal, group, gather_output):
        from .triple_dot_product.flash_trittention import _validate

        world = dist.get_world_size(group)
        rank = dist.get_rank(group)
        if not _supported_world(world):
            raise ValueError(f"query sharding needs a power-of-two group size <= 64, got {world}")
        _validate(q, k1, k2, v1, v2)
        q, k1, k2, v1, v2 = (_native.aligned(t) for t in (q, k1, k2, v1, v2))
        # own rows only; rows of other ranks stay zero.  Neither the output nor the log-sum-exp of another rank's rows
        # is needed by this rank's backward, so the forward itself exchanges nothing.
        o = torch.zeros_like(q)
        lse = torch.zeros(q.shape[:3], dtype=torch.float32, device=q.device)
        _native.tdp_fwd(q, k1, k2, v1, v2, o, lse, softmax_scale, causal, None, None, None, None,
                        q_mod=world, q_rem=rank)
        ctx.save_for_backward(q, k1, k2, v1, v2, o, lse)
        ctx.softmax_scale, ctx.causal, ctx.group = softmax_scale, causal, group
        return _gather_rows(o, rank, world, group) if gather_output and world > 1 else o

    @staticmethod
    def backward(ctx, d_o):
        q, k1, k2, v1, v2, o, lse = ctx.saved_tensors
        group = ctx.group
        world = dist.get_world_size(group)
        rank = dist.get_rank(group)
        d_o = _native.aligned(d_o.to(q.dtype))
        dq = torch.zeros_like(q)
        ws = _native.tdp_bwd(q, k1, k2, v1, v2, o, d_o, lse, dq, None, None, None, None, ctx.softmax_scale,
                             ctx.causal, None, None, None, None, q_mod=world, q_rem=rank,
                             flags=_native.FLAG_BWD_PARTIAL)
        n = q.numel()
        partials = ws[: 16 * n].view(torch.float32)  # dK1 | dK2 | dSiLU(V1) | dV2, fp32, one flat buffer
        # The one exchange of the backward: the key-side partial sums.  It runs on the process group's own stream while
        # this stream gathers the dQ rows (disjoint across ranks, moved in the 16-bit type).
        work = dist.all_reduce(partials, group=group, async_op=True) if world > 1 else None
        if world > 1:
            dq = _gather_rows(dq, rank, world, group)
            work.wait()
        dk1, dk2, dv1, dv2 = (torch.empty_like(q) for _ in range(4))
        _native.tdp_bwd_finalize(v1, dk1, dk2, dv1, dv2, ws)
        return dq, dk1, dk2, dv1, dv2, None, None, None, None


def flash_trittention_query_sharded(q, k1, k2, v1, v2, softmax_scale: float = 1 / 8, causal: bool = True,
                                    group: Optional[dist.ProcessGroup] = None, gather_output: bool = True):
    """Triple-dot-product trittention (full windows) with the query rows split over the ranks of ``group``.

    Every rank passes the same full ``[B, N, T, D]`` tensors.  With ``gather_output`` (default) every rank receives
    the full output (one all-gather of the rows in the inputs' 16-bit type); without it the rows of other ranks are
    zero and the forward does not communicate at all.  The backward all-reduces the fp32 key-side partial sums once
    and gathers the ``dQ`` rows; the gradients returned by autograd are complete on every rank.
    """
    return _QueryShardedTrittention.apply(q, k1, k2, v1, v2, softmax_scale, causal, group, gather_output)
