"""Triple-dot-product trittention: ``flash_trittention`` and its autograd function.

Drop-in for ``src/flash_trittention/triple_dot_product/flash_trittention.py`` of the
reference: same positional argument order, ``[B, N, T, D]`` tensors, window / causal /
scale semantics, ``ValueError`` on mismatched inputs or a non-power-of-two head
dimension, five gradients plus seven ``None`` from backward.  The device work is done by
``libtritt_sm100.so`` (``tritt_tdp_fwd`` / ``tritt_tdp_bwd``); SiLU gating, the
log-sum-exp fix-up, ``D = sum(dO*O)`` and the SiLU derivative, which the reference runs
as separate PyTorch passes (``:61-62,128,158-167,390-391``), are fused into those calls.
"""
import warnings

import torch

from .. import _native
from .kernels.utils import process_masking_variables


def _validate(Q, K1, K2, V1, V2):
    if Q.dim() != 4:
        raise ValueError(f"expected [batch, heads, seq_len, head_dim] tensors, got shape {tuple(Q.shape)}")
    for name, tensor in (("K1", K1), ("K2", K2), ("V1", V1), ("V2", V2)):
        if tensor.shape != Q.shape:
            raise ValueError(f"{name} shape {tuple(tensor.shape)} does not match Q shape {tuple(Q.shape)}")
        if tensor.dtype != Q.dtype:
            raise ValueError(f"{name} dtype {tensor.dtype} does not match Q dtype {Q.dtype}")
        if tensor.device != Q.device:
            raise ValueError(f"{name} device {tensor.device} does not match Q device {Q.device}")
    head_dim = Q.shape[-1]
    if head_dim <= 0 or head_dim & (head_dim - 1):
        nxt = 1 << max(head_dim - 1, 0).bit_length()
        raise ValueError(f"head_dim must be a power of 2, got {head_dim} (next power of 2 is {nxt})")
    if not Q.is_cuda:
        raise RuntimeError("flash_trittention runs on CUDA tensors only (there is no CPU path)")
    _native.dtype_code(Q.dtype)


class FlashTrittention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, Q, K1, K2, V1, V2, softmax_scale, kk_left, kk_right, k1_window, k2_window, causal,
                convert_to_float32, *extra):
        # `extra`: at most one more positional argument, True for the exact-fp32 CUDA-core kernels
        # (``input_precision="ieee"`` of the functional entry point); the reference's signature ends before it
        _validate(Q, K1, K2, V1, V2)
        seq_len = Q.shape[2]
        Q, K1, K2, V1, V2 = (_native.aligned(t) for t in (Q, K1, K2, V1, V2))
        k1_window, k2_window, kk_left, kk_right = process_masking_variables(
            seq_len, k1_window, k2_window, kk_left, kk_right)
        O = torch.empty_like(Q)
        lse = torch.empty(Q.shape[:3], dtype=torch.float32, device=Q.device)
        # convert_to_float32 asks for fp32 operands inside the kernel, which the reference then feeds to TF32 dot
        # products: here bf16 inputs get operands of TF32's 11 significant bits (fp16 copies) on the tensor cores;
        # fp16 inputs have them already, fp32 inputs always run that way
        flags = _native.FLAG_WIDE_OPERANDS if convert_to_float32 else 0
        if extra and extra[0]:
            flags = _native.FLAG_FORCE_SIMT
        ctx.n_extra = len(extra)
        _native.tdp_fwd(Q, K1, K2, V1, V2, O, lse, softmax_scale, causal, k1_window, k2_window, kk_left, kk_right,
                        flags=flags)
        ctx.save_for_backward(Q, K1, K2, V1, V2, O, lse)
        ctx.softmax_scale = softmax_scale
        ctx.windows = (k1_window, k2_window, kk_left, kk_right)
        ctx.causal = causal
        ctx.flags = flags
        return O

    @staticmethod
    def backward(ctx, dO):
        Q, K1, K2, V1, V2, O, lse = ctx.saved_tensors
        dO = _native.aligned(dO)
        if dO.dtype != Q.dtype:
            dO = dO.to(Q.dtype)
        dq, dk1, dk2, dv1, dv2 = (torch.empty_like(Q) for _ in range(5))
        k1_window, k2_window, kk_left, kk_right = ctx.windows
        _native.tdp_bwd(Q, K1, K2, V1, V2, O, dO, lse, dq, dk1, dk2, dv1, dv2, ctx.softmax_scale, ctx.causal,
                        k1_window, k2_window, kk_left, kk_right, flags=ctx.flags)
        return (dq, dk1, dk2, dv1, dv2, None, None, None, None, None, None, None) + (None,) * ctx.n_extra


def flash_trittention(
    q,
    k1,
    k2,
    v1,
    v2,
    softmax_scale=1 / 8,
    kk_left=1,
    kk_right=1,
    k1_window=1,
    k2_window=1,
    causal=True,
    convert_to_float32=False,
    input_precision=None,
):
    """Triple-dot-product trittention, forward and (through autograd) backward.

    ``S[q,j,k] = softmax_scale * sum_h q[q,h] k1[j,h] k2[k,h]``; soft-max over the attended
    ``(j, k)``; ``out[q,h] = sum_jk P[q,j,k] SiLU(v1[j,h]) v2[k,h]``.  With ``causal`` a triple
    is attended iff ``j <= q <= j + k1_window``, ``k <= q <= k + k2_window`` and
    ``k - kk_left <= j <= k + kk_right``; a window of ``None`` spans the sequence.

    Precision: 16-bit inputs run with 16-bit tensor-core operands and fp32 accumulation; fp32 inputs (head dimension 64
    or 128) and ``convert_to_float32=True`` on bf16 inputs run on the tensor cores with operands of 11 significant
    bits, the precision of the TF32 dot products the reference feeds them to.  ``input_precision="ieee"`` selects
    exact-fp32 arithmetic on the CUDA cores (much slower); any other value is accepted and ignored with a warning, as
    the reference does for every value (``flash_trittention.py:418-424``).
    """
    exact = input_precision == "ieee"
    if input_precision is not None and not exact:
        warnings.warn(
            "flash_trittention: `input_precision` is currently unused and has no "
            f"effect (got {input_precision!r}); matmuls run at the kernel's default precision.",
            stacklevel=2,
        )
    if torch.compiler.is_compiling():
        # one opaque graph node instead of tracing into the autograd function
        from ..ops import tdp_attention

        return tdp_attention(q, k1, k2, v1, v2, softmax_scale, causal, k1_window, k2_window, kk_left, kk_right,
                             convert_to_float32)[0]
    if exact:
        return FlashTrittention.apply(q, k1, k2, v1, v2, softmax_scale, kk_left, kk_right, k1_window, k2_window, causal,
                                      convert_to_float32, True)
    return FlashTrittention.apply(q, k1, k2, v1, v2, softmax_scale, kk_left, kk_right, k1_window, k2_window, causal,
                                  convert_to_float32)
