"""Dot-product-sum trittention: ``TrittentionTriton`` module and its autograd function.

Drop-in for ``src/flash_trittention/dot_product_sum/trittention_triton.py`` of the
reference (the class keeps its historical name although nothing here uses Triton):
``forward`` returns ``(o, m)`` with ``m`` the fp32 log-sum-exp, inputs may be
non-contiguous, ``ValueError`` on shape / dtype / device mismatch, backward returns five
gradients plus five ``None`` and ignores the gradient of ``m``.
"""
from typing import Optional

import torch
import torch.nn as nn

from .. import _native


class TrittentionTritonFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k1, k2, v1, v2, causal, softmax_scale, k_diff, convert_to_float32=False,
                input_precision=None):
        if not (q.shape == k1.shape == k2.shape == v1.shape == v2.shape):
            raise ValueError(
                f"Shape mismatch: q={q.shape}, k1={k1.shape}, k2={k2.shape}, v1={v1.shape}, v2={v2.shape}")
        if not (q.dtype == k1.dtype == k2.dtype == v1.dtype == v2.dtype):
            raise ValueError("q, k1, k2, v1, v2 must all have the same dtype")
        if not (q.device == k1.device == k2.device == v1.device == v2.device):
            raise ValueError("q, k1, k2, v1, v2 must all be on the same device")
        if q.dim() != 4:
            raise ValueError(f"expected [batch, heads, seq_len, head_dim] tensors, got shape {tuple(q.shape)}")
        d = q.shape[-1]
        if d <= 0 or d & (d - 1):
            raise ValueError(f"head_dim must be a power of 2, got {d}")
        if not q.is_cuda:
            raise RuntimeError("TrittentionTriton runs on CUDA tensors only (there is no CPU path)")
        _native.dtype_code(q.dtype)
        q, k1, k2, v1, v2 = (_native.aligned(t) for t in (q, k1, k2, v1, v2))
        o = torch.empty_like(q)
        m = torch.empty(q.shape[:3], device=q.device, dtype=torch.float32)
        # convert_to_float32 asks for fp32 operands inside the kernels (reference trittention_triton.py:98-117
        # forwards it to its launches): the CUDA-core path computes in fp32 on every dtype
        flags = _native.FLAG_FORCE_SIMT if (convert_to_float32 or input_precision == "ieee") else 0
        ws = _native.dps_fwd(q, k1, k2, v1, v2, o, m, softmax_scale, causal, k_diff, flags=flags)
        # the forward's workspace holds the inner attention's results; kept for the backward (the reference saves
        # only the inputs, o and m and recomputes, trittention_triton.py:122-128)
        ctx.fwd_ws = ws if any(ctx.needs_input_grad[:5]) else None
        ctx.flags = flags
        ctx.causal = causal
        ctx.softmax_scale = softmax_scale
        ctx.k_diff = k_diff
        ctx.save_for_backward(q, k1, k2, v1, v2, o, m)
        ctx.mark_non_differentiable(m)
        return o, m

    @staticmethod
    def backward(ctx, grad_output, m_grad=None):
        q, k1, k2, v1, v2, o, m = ctx.saved_tensors
        assert grad_output.shape == o.shape, f"Shape mismatch: O={o.shape}, dO={grad_output.shape}"
        assert o.device == grad_output.device, "O and dO must be on the same device"
        assert o.dtype == grad_output.dtype, "O and dO must have the same dtype"
        grad_output = _native.aligned(grad_output)
        dq, dk1, dk2, dv1, dv2 = (torch.empty_like(q) for _ in range(5))
        _native.dps_bwd(q, k1, k2, v1, v2, o, grad_output, m, dq, dk1, dk2, dv1, dv2, ctx.softmax_scale,
                        ctx.causal, ctx.k_diff, flags=ctx.flags, fwd_ws=ctx.fwd_ws)
        ctx.fwd_ws = None
        return dq, dk1, dk2, dv1, dv2, None, None, None, None, None


class TrittentionTriton(nn.Module):
    def __init__(
        self,
        causal: bool = True,
        softmax_scale: float = 1 / 8,
        k_diff: int = 1024,
        convert_to_float32: bool = False,
        input_precision: Optional[str] = None,
    ):
        super().__init__()
        self.causal = causal
        self.softmax_scale = softmax_scale
        self.k_diff = k_diff
        self.convert_to_float32 = convert_to_float32
        self.input_precision = input_precision

    def forward(self, q, k1, k2, v1, v2):
        """``q, k1, k2, v1, v2``: ``[B, N, S, D]``.  Returns ``(o [B,N,S,D], m [B,N,S] fp32)``.

        ``S[q,s,t] = softmax_scale * (q[q].k2[t] + k1[s].k2[t])``, causal mask
        ``s <= t <= q`` and ``t - s <= k_diff``; ``o = sum_st P SiLU(v1[s]) v2[t]``.
        16-bit inputs with a head dimension of 64 or 128 run on the tensor cores with 16-bit operands (the
        probabilities and ``Y*V2`` are rounded to the inputs' type, accumulation and soft-max state are fp32);
        ``convert_to_float32=True`` selects the fp32 CUDA-core kernels instead, as do fp32 inputs and other
        head dimensions, and ``input_precision="ieee"`` (the reference's name for exact fp32 dot products).
        """
        return TrittentionTritonFunction.apply(q, k1, k2, v1, v2, self.causal, self.softmax_scale, self.k_diff,
                                               self.convert_to_float32, self.input_precision)
