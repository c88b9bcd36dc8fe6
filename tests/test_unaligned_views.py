"""Tensors whose storage does not start on a 16-byte boundary (a contiguous view at an odd element offset) cannot
be TMA or vector-load operands and the C ABI rejects them; the Python entry points copy such views first, so that
callers see the same results as for aligned tensors (the reference's Triton kernels accept any alignment)."""
import pytest
import torch

from flash_trittention import TrittentionTriton, flash_trittention
from oracle import trittention_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _offset_view(x, off=4):
    """A contiguous copy of ``x`` that starts ``off`` elements into its storage (8 bytes for 16-bit types)."""
    buf = torch.empty(x.numel() + off, dtype=x.dtype, device=x.device)
    view = buf[off:].view(x.shape)
    view.copy_(x)
    assert view.data_ptr() % 16 != 0 and view.is_contiguous()
    return view


@pytest.mark.parametrize("variant", ["tdp", "dps"])
def test_views_at_an_odd_offset(variant):
    B, N, T, D = 1, 2, 160, 64
    q, k1, k2, v1, v2, dz = orc.make_inputs(B, N, T, D, scale=0.5, seed=41, dtype=torch.float16)
    base = [x.to(DEV) for x in (q, k1, k2, v1, v2)]
    dzd = dz.to(DEV)

    def run(tensors):
        leaves = [x.detach().requires_grad_(True) for x in tensors]
        if variant == "tdp":
            out = flash_trittention(*leaves, softmax_scale=1 / D, kk_left=None, kk_right=None, k1_window=None,
                                    k2_window=None, causal=True)
        else:
            out, _ = TrittentionTriton(causal=True, softmax_scale=1 / 8, k_diff=50)(*leaves)
        out.backward(dzd)
        return out, [x.grad for x in leaves]

    out_a, g_a = run(base)
    out_b, g_b = run([_offset_view(x) for x in base])
    assert float((out_a.float() - out_b.float()).abs().max()) <= 5e-3 * float(out_a.float().abs().max())
    for a, b in zip(g_a, g_b):
        assert float((a.float() - b.float()).abs().max()) <= 5e-3 * float(a.float().abs().max())
