"""``torch.library`` registration of the four device calls, and ``nn.Module`` wrappers built on them.

The reference exposes its kernels through ``torch.autograd.Function`` classes only
(``src/flash_trittention/triple_dot_product/flash_trittention.py:14-395``,
``src/flash_trittention/dot_product_sum/trittention_triton.py:15-360``), which ``torch.compile`` has to
trace into.  Here the same calls are also registered as custom operators

    torch.ops.flash_trittention.tdp_fwd / tdp_bwd      (triple-dot-product)
    torch.ops.flash_trittention.dps_fwd / dps_bwd      (dot-product-sum)

with fake (shape-only) implementations and autograd formulas, so that a compiled graph carries each of them as
one opaque node and needs no graph break.  ``flash_trittention()`` switches to these operators by itself while it
is being compiled; ``TrittentionTDP`` is a module for the triple-dot-product variant with the constructor /
``forward`` conventions of the reference's ``TrittentionTriton`` (returns ``(o, lse)``).

Importing this module does not load the CUDA library; the operators do, on their first call, and raise if it is
missing (there is no CPU implementation behind them).
"""
from typing import Optional, Tuple

import torch
import torch.nn as nn
from torch import Tensor

from . import _native

__all__ = ["tdp_fwd", "tdp_bwd", "dps_fwd", "dps_bwd", "tdp_attention", "dps_attention", "TrittentionTDP"]


def _check_inputs(q, k1, k2, v1, v2):
    if q.dim() != 4:
        raise ValueError(f"expected [batch, heads, seq_len, head_dim] tensors, got shape {tuple(q.shape)}")
    for name, t in (("k1", k1), ("k2", k2), ("v1", v1), ("v2", v2)):
        if t.shape != q.shape:
            raise ValueError(f"{name} shape {tuple(t.shape)} does not match q shape {tuple(q.shape)}")
        if t.dtype != q.dtype:
            raise ValueError(f"{name} dtype {t.dtype} does not match q dtype {q.dtype}")
        if t.device != q.device:
            raise ValueError(f"{name} device {t.device} does not match q device {q.device}")
    d = q.shape[-1]
    if d <= 0 or d & (d - 1):
        raise ValueError(f"head_dim must be a power of 2, got {d}")


# ------------------------------------------------------------------ triple-dot-product

@torch.library.custom_op("flash_trittention::tdp_fwd", mutates_args=(), device_types="cuda")
def tdp_fwd(q: Tensor, k1: Tensor, k2: Tensor, v1: Tensor, v2: Tensor, softmax_scale: float, causal: bool,
            k1_window: Optional[int], k2_window: Optional[int], kk_left: Optional[int], kk_right: Optional[int],
            convert_to_float32: bool) -> Tuple[Tensor, Tensor]:
    """``(o [B,N,T,D], lse [B,N,T] fp32)`` of ``tritt_tdp_fwd``; a window of ``None`` spans the sequence."""
    _check_inputs(q, k1, k2, v1, v2)
    _native.dtype_code(q.dtype)
    q, k1, k2, v1, v2 = (_native.aligned(t) for t in (q, k1, k2, v1, v2))
    o = torch.empty_like(q)
    lse = torch.empty(q.shape[:3], dtype=torch.float32, device=q.device)
    flags = _native.FLAG_WIDE_OPERANDS if convert_to_float32 else 0
    _native.tdp_fwd(q, k1, k2, v1, v2, o, lse, softmax_scale, causal, k1_window, k2_window, kk_left, kk_right,
                    flags=flags)
    return o, lse


@tdp_fwd.register_fake
def _(q, k1, k2, v1, v2, softmax_scale, causal, k1_window, k2_window, kk_left, kk_right, convert_to_float32):
    _check_inputs(q, k1, k2, v1, v2)
    return (torch.empty(q.shape, dtype=q.dtype, device=q.device),
            torch.empty(q.shape[:3], dtype=torch.float32, device=q.device))


@torch.library.custom_op("flash_trittention::tdp_bwd", mutates_args=(), device_types="cuda")
def tdp_bwd(q: Tensor, k1: Tensor, k2: Tensor, v1: Tensor, v2: Tensor, o: Tensor, d_o: Tensor, lse: Tensor,
            softmax_scale: float, causal: bool, k1_window: Optional[int], k2_window: Optional[int],
            kk_left: Optional[int], kk_right: Optional[int],
            convert_to_float32: bool) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    """``(dq, dk1, dk2, dv1, dv2)`` of ``tritt_tdp_bwd`` for the upstream gradient ``d_o`` of ``o``."""
    q, k1, k2, v1, v2, o, lse = (_native.aligned(t) for t in (q, k1, k2, v1, v2, o, lse))
    d_o = _native.aligned(d_o.to(q.dtype))
    grads = tuple(torch.empty_like(q) for _ in range(5))
    flags = _native.FLAG_WIDE_OPERANDS if convert_to_float32 else 0
    _native.tdp_bwd(q, k1, k2, v1, v2, o, d_o, lse, *grads, softmax_scale, causal, k1_window, k2_window, kk_left,
                    kk_right, flags=flags)
    return grads


@tdp_bwd.register_fake
def _(q, k1, k2, v1, v2, o, d_o, lse, softmax_scale, causal, k1_window, k2_window, kk_left, kk_right,
      convert_to_float32):
    return tuple(torch.empty(q.shape, dtype=q.dtype, device=q.device) for _ in range(5))


def _tdp_setup(ctx, inputs, output):
    q, k1, k2, v1, v2, *rest = inputs
    o, lse = output
    ctx.save_for_backward(q, k1, k2, v1, v2, o, lse)
    ctx.mark_non_differentiable(lse)
    ctx.rest = tuple(rest)


def _tdp_backward(ctx, d_o, d_lse):
    # (the log-sum-exp output carries no gradient, as in the reference where it is not returned at all)
    grads = tdp_bwd(*ctx.saved_tensors[:6], d_o, ctx.saved_tensors[6], *ctx.rest)
    return (*grads, None, None, None, None, None, None, None)


tdp_fwd.register_autograd(_tdp_backward, setup_context=_tdp_setup)


def tdp_attention(q, k1, k2, v1, v2, softmax_scale=1 / 8, causal=True, k1_window=None, k2_window=None,
                  kk_left=None, kk_right=None, convert_to_float32=False):
    """Differentiable triple-dot-product trittention through the registered operators: ``(o, lse)``."""
    return tdp_fwd(q, k1, k2, v1, v2, float(softmax_scale), bool(causal), k1_window, k2_window, kk_left, kk_right,
                   bool(convert_to_float32))


# ------------------------------------------------------------------ dot-product-sum

@torch.library.custom_op("flash_trittention::dps_fwd", mutates_args=(), device_types="cuda")
def dps_fwd(q: Tensor, k1: Tensor, k2: Tensor, v1: Tensor, v2: Tensor, softmax_scale: float, causal: bool,
            k_diff: int, convert_to_float32: bool = False) -> Tuple[Tensor, Tensor]:
    """``(o [B,N,S,D], m [B,N,S] fp32 log-sum-exp)`` of ``tritt_dps_fwd``; ``convert_to_float32`` selects the
    fp32 CUDA-core kernels on every dtype."""
    _check_inputs(q, k1, k2, v1, v2)
    _native.dtype_code(q.dtype)
    q, k1, k2, v1, v2 = (_native.aligned(t) for t in (q, k1, k2, v1, v2))
    o = torch.empty_like(q)
    m = torch.empty(q.shape[:3], dtype=torch.float32, device=q.device)
    _native.dps_fwd(q, k1, k2, v1, v2, o, m, softmax_scale, causal, k_diff,
                    flags=_native.FLAG_FORCE_SIMT if convert_to_float32 else 0)
    return o, m


@dps_fwd.register_fake
def _(q, k1, k2, v1, v2, softmax_scale, causal, k_diff, convert_to_float32=False):
    _check_inputs(q, k1, k2, v1, v2)
    return (torch.empty(q.shape, dtype=q.dtype, device=q.device),
            torch.empty(q.shape[:3], dtype=torch.float32, device=q.device))


@torch.library.custom_op("flash_trittention::dps_bwd", mutates_args=(), device_types="cuda")
def dps_bwd(q: Tensor, k1: Tensor, k2: Tensor, v1: Tensor, v2: Tensor, o: Tensor, d_o: Tensor, m: Tensor,
            softmax_scale: float, causal: bool, k_diff: int,
            convert_to_float32: bool = False) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    q, k1, k2, v1, v2, o, m = (_native.aligned(t) for t in (q, k1, k2, v1, v2, o, m))
    d_o = _native.aligned(d_o.to(q.dtype))
    grads = tuple(torch.empty_like(q) for _ in range(5))
    _native.dps_bwd(q, k1, k2, v1, v2, o, d_o, m, *grads, softmax_scale, causal, k_diff,
                    flags=_native.FLAG_FORCE_SIMT if convert_to_float32 else 0)
    return grads


@dps_bwd.register_fake
def _(q, k1, k2, v1, v2, o, d_o, m, softmax_scale, causal, k_diff, convert_to_float32=False):
    return tuple(torch.empty(q.shape, dtype=q.dtype, device=q.device) for _ in range(5))


def _dps_setup(ctx, inputs, output):
    q, k1, k2, v1, v2, *rest = inputs
    o, m = output
    ctx.save_for_backward(q, k1, k2, v1, v2, o, m)
    ctx.mark_non_differentiable(m)
    ctx.rest = tuple(rest)


def _dps_backward(ctx, d_o, d_m):
    grads = dps_bwd(*ctx.saved_tensors[:6], d_o, ctx.saved_tensors[6], *ctx.rest)
    return (*grads, None, None, None, None)


dps_fwd.register_autograd(_dps_backward, setup_context=_dps_setup)


def dps_attention(q, k1, k2, v1, v2, softmax_scale=1 / 8, causal=True, k_diff=1024, convert_to_float32=False):
    """Differentiable dot-product-sum trittention through the registered operators: ``(o, m)``."""
    return dps_fwd(q, k1, k2, v1, v2, float(softmax_scale), bool(causal), int(k_diff), bool(convert_to_float32))


# ------------------------------------------------------------------ module

class TrittentionTDP(nn.Module):
    """Triple-dot-product trittention as a module, in the shape of the reference's ``TrittentionTriton``
    (``dot_product_sum/trittention_triton.py:362-403``): the mask and scale are constructor arguments,
    ``forward(q, k1, k2, v1, v2)`` takes ``[B, N, T, D]`` tensors and returns ``(o, lse)``."""

    def __init__(self, causal: bool = True, softmax_scale: float = 1 / 8, k1_window: Optional[int] = None,
                 k2_window: Optional[int] = None, kk_left: Optional[int] = None, kk_right: Optional[int] = None,
                 convert_to_float32: bool = False):
        super().__init__()
        self.causal = causal
        self.softmax_scale = softmax_scale
        self.k1_window, self.k2_window, self.kk_left, self.kk_right = k1_window, k2_window, kk_left, kk_right
        self.convert_to_float32 = convert_to_float32

    def forward(self, q, k1, k2, v1, v2):
        return tdp_attention(q, k1, k2, v1, v2, self.softmax_scale, self.causal, self.k1_window, self.k2_window,
                             self.kk_left, self.kk_right, self.convert_to_float32)

    def extra_repr(self) -> str:
        return (f"causal={self.causal}, softmax_scale={self.softmax_scale}, k1_window={self.k1_window}, "
                f"k2_window={self.k2_window}, kk_left={self.kk_left}, kk_right={self.kk_right}")
