"""CPU-side checks of the drop-in boundary: the C-ABI library loads, exports every symbol
the header declares, rejects bad arguments before touching a device, and the Python entry
points keep the reference's validation behaviour."""
import ctypes
import os
import re

import pytest
import torch

from flash_trittention import _native

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_functions():
    src = open(os.path.join(ROOT, "include", "tritt.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(tritt_[a-z0-9_]+)\s*\(", src)))


def test_library_exports_every_declared_symbol():
    lib = _native.lib()
    declared = _header_functions()
    assert len(declared) >= 11
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/tritt.h but not exported"
    assert set(_native.SYMBOLS) <= set(declared)
    assert lib.tritt_version() >= 100


def test_workspace_sizes():
    lib = _native.lib()
    B, N, T, D = 1, 16, 2048, 128
    n = B * N * T * D
    assert lib.tritt_workspace_bytes(_native.OP_TDP_BWD, B, N, T, D, _native.BF16) >= 4 * n * 4
    assert lib.tritt_workspace_bytes(_native.OP_DPS_FWD, B, N, T, D, _native.F16) >= n * 4
    assert lib.tritt_workspace_bytes(_native.OP_DPS_BWD, B, N, T, D, _native.F16) >= 5 * n * 4
    assert lib.tritt_workspace_bytes(99, B, N, T, D, 0) == 0
    assert lib.tritt_workspace_bytes(_native.OP_TDP_FWD, 0, N, T, D, 0) == 0


def test_c_abi_rejects_bad_arguments_without_a_device():
    lib = _native.lib()
    buf = ctypes.create_string_buffer(4096 + 256)
    p = (ctypes.addressof(buf) + 255) & ~255  # aligned host address: never dereferenced on these paths
    args = lambda D, dtype, q_mod=1, q_rem=0: [p] * 7 + [1, 1, 8, D, dtype, 0.125, 1, 8, 8, 8, 8, q_mod, q_rem,
                                                        None, 0, None, 0, None]
    assert lib.tritt_tdp_fwd(*args(24, _native.F32)) == -2  # head_dim not a power of two
    assert b"power of 2" in lib.tritt_last_error()
    assert lib.tritt_tdp_fwd(*args(16, 7)) == -3  # unknown dtype
    assert lib.tritt_tdp_fwd(*args(16, _native.F32, q_mod=2, q_rem=2)) == -8
    bad = args(16, _native.F32)
    bad[2] = None
    assert lib.tritt_tdp_fwd(*bad) == -4  # null tensor
    bad = args(16, _native.F32)
    bad[1] = p + 4
    assert lib.tritt_tdp_fwd(*bad) == -5  # misaligned tensor
    # DPS needs a workspace: a missing one is an argument error, not a crash
    dps = [p] * 7 + [1, 1, 8, 16, _native.F32, 0.125, 1, 8, None, 0, None, 0, None]
    assert lib.tritt_dps_fwd(*dps) == -6
    # windows are distances: a negative one is refused under a causal mask (the reference would apply it literally
    # and leave rows without anything to attend), and ignored without one
    neg = args(16, _native.F32)
    neg[14] = -1  # k1_window
    assert lib.tritt_tdp_fwd(*neg) == -10
    assert b"window" in lib.tritt_last_error()
    dps_neg = [p] * 7 + [1, 1, 8, 16, _native.F32, 0.125, 1, -2, None, 0, None, 0, None]
    assert lib.tritt_dps_fwd(*dps_neg) == -10
    # B*N is a grid dimension of the CUDA-core kernels
    big = args(16, _native.F32)
    big[7], big[8] = 256, 257
    assert lib.tritt_tdp_fwd(*big) == -11
    assert b"65535" in lib.tritt_last_error()
    # the saved-state backward refuses a missing forward workspace
    saved = [p] * 13 + [1, 1, 8, 16, _native.F32, 0.125, 1, 8, p, 1 << 20, None, 0, None, 0, None]
    assert lib.tritt_dps_bwd_saved(*saved) == -4


def test_tdp_path_selection():
    T = 512
    full = dict(causal=True, k1w=None, k2w=None, kkl=None, kkr=None)
    # 16-bit inputs run on the tensor cores under every mask; fp32 inputs too when the head dimension allows (through
    # fp16 operand copies), otherwise and with TRITT_FLAG_FORCE_SIMT on the exact-fp32 CUDA-core kernels
    assert _native.tdp_path(_native.OP_TDP_FWD, T, 64, _native.F32, **full) == _native.PATH_TCGEN05
    assert _native.tdp_path(_native.OP_TDP_BWD, T, 128, _native.F32, **full) == _native.PATH_TCGEN05
    assert _native.tdp_path(_native.OP_TDP_FWD, T, 32, _native.F32, **full) == _native.PATH_SIMT
    assert _native.tdp_path(_native.OP_TDP_FWD, T, 64, _native.F32, **full,
                            flags=_native.FLAG_FORCE_SIMT) == _native.PATH_SIMT
    lib = _native.lib()
    n = 2 * 3 * T * 64
    assert lib.tritt_workspace_bytes_flags(_native.OP_TDP_BWD, 2, 3, T, 64, _native.BF16, _native.FLAG_WIDE_OPERANDS) > \
        lib.tritt_workspace_bytes(_native.OP_TDP_BWD, 2, 3, T, 64, _native.BF16) >= 18 * n
    assert lib.tritt_workspace_bytes(_native.OP_TDP_FWD, 2, 3, T, 64, _native.F32) >= 14 * n
    assert _native.tdp_path(_native.OP_TDP_FWD, T, 64, _native.BF16, True, 8, 8, 4, 4) == _native.PATH_TCGEN05
    assert _native.tdp_path(_native.OP_TDP_BWD, T, 64, _native.BF16, True, 8, 8, 4, 4) == _native.PATH_TCGEN05
    assert _native.tdp_path(_native.OP_TDP_FWD, T, 64, _native.BF16, **full,
                            flags=_native.FLAG_FORCE_SIMT) == _native.PATH_SIMT


def test_python_entry_points_validate_like_the_reference():
    from flash_trittention import flash_trittention, TrittentionTriton

    q, k1, k2, v1, v2 = (torch.randn(2, 2, 32, 32) for _ in range(5))
    with pytest.raises(ValueError):
        flash_trittention(q, k1, k2, v1, v2[:, :, :16].contiguous())
    with pytest.raises(ValueError):
        flash_trittention(q, k1, k2, v1, v2.double())
    with pytest.raises(ValueError):
        flash_trittention(*(torch.randn(2, 2, 32, 24) for _ in range(5)))
    with pytest.raises(ValueError):
        TrittentionTriton()(q, k1, k2, v1, v2[:, :, :16].contiguous())
    # valid arguments on CPU tensors: refused loudly, never computed on the host
    with pytest.raises(RuntimeError, match="no CPU path"):
        flash_trittention(q, k1, k2, v1, v2)
    with pytest.raises(RuntimeError, match="no CPU path"):
        TrittentionTriton()(q, k1, k2, v1, v2)


def test_input_precision_warns():
    import warnings

    from flash_trittention import flash_trittention

    q = torch.randn(1, 1, 8, 8)
    with pytest.warns(UserWarning, match="input_precision"):
        with pytest.raises(RuntimeError):
            flash_trittention(q, q, q, q, q, input_precision="tf32x3")
    # "ieee" has an effect here (exact-fp32 kernels), so it does not warn
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        with pytest.raises(RuntimeError):
            flash_trittention(q, q, q, q, q, input_precision="ieee")


def test_package_surface_matches_reference_names():
    import flash_trittention as ft

    assert set(ft.__all__) == {"flash_trittention", "TrittentionTriton"}
    from flash_trittention.triple_dot_product.flash_trittention import FlashTrittention, flash_trittention  # noqa
    from flash_trittention.triple_dot_product.trittention_pytorch import Trittention_pytorch  # noqa
    from flash_trittention.triple_dot_product.kernels.utils import process_masking_variables
    from flash_trittention.dot_product_sum.trittention_triton import TrittentionTriton, TrittentionTritonFunction  # noqa
    from flash_trittention.dot_product_sum.trittention_pytorch import Trittention_pytorch as P2  # noqa

    assert process_masking_variables(7, None, 3, None, 2) == (7, 3, 7, 2)
    import inspect

    sig = inspect.signature(flash_trittention)
    assert list(sig.parameters) == ["q", "k1", "k2", "v1", "v2", "softmax_scale", "kk_left", "kk_right",
                                    "k1_window", "k2_window", "causal", "convert_to_float32", "input_precision"]
    assert sig.parameters["kk_left"].default == 1 and sig.parameters["softmax_scale"].default == 1 / 8


def test_aligned_copies_only_views_off_a_16_byte_boundary():
    from flash_trittention import _native

    buf = torch.arange(4 * 64 + 8, dtype=torch.float16)
    on = buf[8:].view(4, 64)    # 16 bytes into the storage
    off = buf[4:4 + 256].view(4, 64)  # 8 bytes into the storage
    assert _native.aligned(on).data_ptr() == on.data_ptr()
    fixed = _native.aligned(off)
    assert fixed.data_ptr() != off.data_ptr() and fixed.data_ptr() % 16 == 0 and torch.equal(fixed, off)
    strided = buf[:256].view(64, 4).t()
    assert _native.aligned(strided).is_contiguous() and torch.equal(_native.aligned(strided), strided)
