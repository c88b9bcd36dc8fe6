"""ctypes binding of ``libtritt_sm100.so`` (declared in ``include/tritt.h``).

The library is the only compute path: if it is missing, loading raises and every entry
point of the package fails loudly.  There is no PyTorch or CPU fallback.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtritt_sm100.so")

F32, F16, BF16 = 0, 1, 2
OP_TDP_FWD, OP_TDP_BWD, OP_DPS_FWD, OP_DPS_BWD = 0, 1, 2, 3
FLAG_FORCE_SIMT, FLAG_BWD_PARTIAL, FLAG_WIDE_OPERANDS, FLAG_BWD_CTA_PAIRS = 1, 2, 4, 8
PATH_SIMT, PATH_TCGEN05 = 0, 1

_DTYPES = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}

# every symbol include/tritt.h declares
SYMBOLS = (
    "tritt_version", "tritt_kernel_launches", "tritt_last_error", "tritt_workspace_bytes", "tritt_workspace_bytes_flags",
    "tritt_tdp_fwd_min_workspace", "tritt_tdp_path", "tritt_dps_path", "tritt_tdp_fwd",
    "tritt_tdp_bwd", "tritt_tdp_bwd_finalize", "tritt_tdp_bwd_partials_offset", "tritt_dps_fwd",
    "tritt_dps_bwd", "tritt_dps_bwd_saved", "tritt_selftest_umma", "tritt_selftest_wait_expiry", "tritt_tdp_fwd_noalloc",
    "tritt_noalloc_scratch_bytes",
)

_lib = None
_lock = threading.Lock()
_status = {}  # device index -> pinned int32 status word (created under _lock)
_status_np = {}  # device index -> numpy view of the same word (a host read without any tensor machinery)
launches = 0  # kernels-enqueuing library calls made by this process (bench bookkeeping)


class TrittError(RuntimeError):
    pass


def lib():
    """Loads the shared library on first use."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise TrittError(
                        f"{LIB_PATH} not found: build it with `python flash-3-way-attention_b200/build.py` "
                        "(there is no fallback path)")
                L = C.CDLL(LIB_PATH)
                vp, i, f, sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t
                L.tritt_version.restype = i
                L.tritt_kernel_launches.restype = C.c_ulonglong
                L.tritt_last_error.restype = C.c_char_p
                L.tritt_workspace_bytes.restype = sz
                L.tritt_workspace_bytes.argtypes = [i] * 6
                L.tritt_workspace_bytes_flags.restype = sz
                L.tritt_workspace_bytes_flags.argtypes = [i] * 7
                L.tritt_tdp_fwd_min_workspace.restype = sz
                L.tritt_tdp_fwd_min_workspace.argtypes = [i] * 11
                L.tritt_tdp_path.restype = i
                L.tritt_tdp_path.argtypes = [i] * 10
                L.tritt_dps_path.restype = i
                L.tritt_dps_path.argtypes = [i] * 5
                L.tritt_tdp_bwd_partials_offset.restype = sz
                L.tritt_tdp_bwd_partials_offset.argtypes = [i] * 5
                L.tritt_tdp_fwd.restype = i
                L.tritt_tdp_fwd.argtypes = [vp] * 7 + [i] * 5 + [f] + [i] * 7 + [vp, sz, vp, i, vp]
                L.tritt_tdp_bwd.restype = i
                L.tritt_tdp_bwd.argtypes = [vp] * 13 + [i] * 5 + [f] + [i] * 7 + [vp, sz, vp, i, vp]
                L.tritt_tdp_bwd_finalize.restype = i
                L.tritt_tdp_bwd_finalize.argtypes = [vp] * 5 + [i] * 5 + [vp, sz, vp]
                L.tritt_dps_fwd.restype = i
                L.tritt_dps_fwd.argtypes = [vp] * 7 + [i] * 5 + [f] + [i] * 2 + [vp, sz, vp, i, vp]
                L.tritt_dps_bwd.restype = i
                L.tritt_dps_bwd.argtypes = [vp] * 13 + [i] * 5 + [f] + [i] * 2 + [vp, sz, vp, i, vp]
                L.tritt_dps_bwd_saved.restype = i
                L.tritt_dps_bwd_saved.argtypes = [vp] * 13 + [i] * 5 + [f] + [i] * 2 + [vp, sz, vp, sz, vp, i, vp]
                L.tritt_tdp_fwd_noalloc.restype = i
                L.tritt_tdp_fwd_noalloc.argtypes = [vp] * 7 + [i] * 5 + [f] + [i] * 5 + [vp, i, vp]
                L.tritt_noalloc_scratch_bytes.restype = sz
                L.tritt_selftest_umma.restype = i
                L.tritt_selftest_umma.argtypes = [vp] * 5 + [i, vp, vp]
                L.tritt_selftest_wait_expiry.restype = i
                L.tritt_selftest_wait_expiry.argtypes = [i, C.c_longlong, vp, vp]
                _lib = L
    return _lib


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise ValueError(f"unsupported dtype {dt}: expected float32, float16 or bfloat16") from None


def _check(rc: int, what: str):
    if rc != 0:
        msg = lib().tritt_last_error().decode("utf-8", "replace")
        if rc < 0:
            raise ValueError(f"{what}: {msg} (code {rc})")
        raise TrittError(f"{what}: {msg} (CUDA error {rc})")


STATUS_BITS = {1: "self-test kernel", 2: "triple-dot-product forward", 4: "triple-dot-product backward",
               8: "shared memory of a tensor-core kernel was not 1024-byte aligned",
               16: "soft-max attention forward (dot-product-sum)", 32: "soft-max attention backward (dot-product-sum)",
               64: "an input element beyond the fp16 operand range (65504) in an fp32 / wide-operand call",
               128: "wait-expiry self-test"}


def _device_index(device) -> int:
    d = torch.device(device)
    return torch.cuda.current_device() if d.index is None else d.index


def status_word(device) -> torch.Tensor:
    """Per-device int32 that kernels OR a code into when a bounded barrier wait ran out.

    The word lives in page-locked host memory, which the GPU addresses directly (unified addressing): only a
    kernel that gives up ever writes it, and the host can look at it without a copy or a synchronisation."""
    key = _device_index(device)
    t = _status.get(key)
    if t is None:
        with _lock:
            t = _status.get(key)
            if t is None:
                t = torch.zeros(1, dtype=torch.int32).pin_memory()
                _status_np[key] = t.numpy()
                _status[key] = t
    return t


def _describe(v: int) -> str:
    return ", ".join(name for bit, name in STATUS_BITS.items() if v & bit) or f"code {v}"


def read_status(device) -> int:
    """Synchronises the device and returns (then clears) its kernel status word."""
    torch.cuda.synchronize(torch.device("cuda", _device_index(device)))
    t = status_word(device)
    v = int(t[0])
    if v:
        t.zero_()
    return v


def check_status(device=None, synchronize: bool = True) -> None:
    """Raises ``TrittError`` if a kernel enqueued earlier on ``device`` gave up on a bounded wait (its results are
    then invalid).  With ``synchronize=False`` only kernels that have already finished are seen; every compute
    entry point of this module makes that cheap check on entry, so a time-out surfaces at the latest on the next
    call after the failed kernel has retired."""
    if not synchronize:
        # the per-call check: one host read of the pinned word
        idx = device.index if isinstance(device, torch.device) else None
        arr = _status_np.get(idx) if idx is not None else None
        if arr is not None and arr[0] == 0:
            return
    dev = _device_index(torch.cuda.current_device() if device is None else device)
    if synchronize:
        v = read_status(dev)
    else:
        t = status_word(dev)
        v = int(t[0])
        if v:
            t.zero_()
    if v:
        raise TrittError(f"a kernel of an earlier call on cuda:{dev} reported a failure: gave up waiting on a barrier "
                         f"after its time limit, or met unusable input ({_describe(v)}); the results of that call "
                         "are invalid")


def workspace(op: int, B: int, N: int, T: int, D: int, dtype: int, device, flags: int = 0) -> torch.Tensor:
    nbytes = lib().tritt_workspace_bytes_flags(op, B, N, T, D, dtype, flags)
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


def aligned(t: torch.Tensor) -> torch.Tensor:
    """``t`` made contiguous and, if its storage offset leaves it off a 16-byte boundary (a view into a larger
    buffer), copied: the library's vector and TMA accesses require that alignment and reject other pointers."""
    t = t.contiguous()
    return t if t.data_ptr() % 16 == 0 else t.clone(memory_format=torch.contiguous_format)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class _on_device:
    """``torch.cuda.device(dev)`` only when ``dev`` is not already the current device (the common case costs one
    query instead of a get / set / restore)."""

    __slots__ = ("ctx",)

    def __init__(self, dev: torch.device):
        self.ctx = None if dev.index == torch.cuda.current_device() else torch.cuda.device(dev)

    def __enter__(self):
        if self.ctx is not None:
            self.ctx.__enter__()

    def __exit__(self, *exc):
        if self.ctx is not None:
            return self.ctx.__exit__(*exc)
        return False


def _win(w, T):
    return T if w is None else int(w)


def tdp_path(op, T, D, dtype, causal, k1w, k2w, kkl, kkr, flags=0) -> int:
    return lib().tritt_tdp_path(op, T, D, dtype, int(bool(causal)), _win(k1w, T), _win(k2w, T), _win(kkl, T),
                                _win(kkr, T), flags)


def dps_path(T, D, dtype, k_diff, flags=0) -> int:
    return lib().tritt_dps_path(T, D, dtype, int(k_diff), flags)


def tdp_fwd(q, k1, k2, v1, v2, o, lse, alpha, causal, k1w, k2w, kkl, kkr, q_mod=1, q_rem=0, flags=0, ws=None):
    """``ws``: a caller-provided workspace (uint8 tensor) instead of one of ``tritt_workspace_bytes`` bytes."""
    global launches
    B, N, T, D = q.shape
    dt = dtype_code(q.dtype)
    check_status(q.device, synchronize=False)
    with _on_device(q.device):
        if ws is None:
            ws = workspace(OP_TDP_FWD, B, N, T, D, dt, q.device, flags)
        rc = lib().tritt_tdp_fwd(q.data_ptr(), k1.data_ptr(), k2.data_ptr(), v1.data_ptr(), v2.data_ptr(),
                                 o.data_ptr(), lse.data_ptr(), B, N, T, D, dt, float(alpha), int(bool(causal)),
                                 _win(k1w, T), _win(k2w, T), _win(kkl, T), _win(kkr, T), q_mod, q_rem,
                                 ws.data_ptr(), ws.numel(), status_word(q.device).data_ptr(), flags, _stream())
    _check(rc, "tritt_tdp_fwd")
    launches += 1


def tdp_bwd(q, k1, k2, v1, v2, o, do, lse, dq, dk1, dk2, dv1, dv2, alpha, causal, k1w, k2w, kkl, kkr,
            q_mod=1, q_rem=0, flags=0, ws=None):
    """Returns the workspace tensor (holds the fp32 partial sums when FLAG_BWD_PARTIAL is set)."""
    global launches
    B, N, T, D = q.shape
    dt = dtype_code(q.dtype)
    ptr = lambda t: 0 if t is None else t.data_ptr()
    check_status(q.device, synchronize=False)
    with _on_device(q.device):
        if ws is None:
            ws = workspace(OP_TDP_BWD, B, N, T, D, dt, q.device, flags)
        rc = lib().tritt_tdp_bwd(q.data_ptr(), k1.data_ptr(), k2.data_ptr(), v1.data_ptr(), v2.data_ptr(),
                                 o.data_ptr(), do.data_ptr(), lse.data_ptr(), dq.data_ptr(), ptr(dk1), ptr(dk2),
                                 ptr(dv1), ptr(dv2), B, N, T, D, dt, float(alpha), int(bool(causal)),
                                 _win(k1w, T), _win(k2w, T), _win(kkl, T), _win(kkr, T), q_mod, q_rem,
                                 ws.data_ptr(), ws.numel(), status_word(q.device).data_ptr(), flags, _stream())
    _check(rc, "tritt_tdp_bwd")
    launches += 1
    return ws


def tdp_bwd_finalize(v1, dk1, dk2, dv1, dv2, ws):
    global launches
    B, N, T, D = v1.shape
    check_status(v1.device, synchronize=False)
    with _on_device(v1.device):
        rc = lib().tritt_tdp_bwd_finalize(v1.data_ptr(), dk1.data_ptr(), dk2.data_ptr(), dv1.data_ptr(),
                                          dv2.data_ptr(), B, N, T, D, dtype_code(v1.dtype), ws.data_ptr(),
                                          ws.numel(), _stream())
    _check(rc, "tritt_tdp_bwd_finalize")
    launches += 1


def dps_fwd(q, k1, k2, v1, v2, o, m, alpha, causal, k_diff, flags=0):
    """Returns the workspace tensor: handed to ``dps_bwd(..., fwd_ws=...)`` it spares the backward the inner
    attention's recomputation (keep it untouched until then)."""
    global launches
    B, N, T, D = q.shape
    dt = dtype_code(q.dtype)
    check_status(q.device, synchronize=False)
    with _on_device(q.device):
        ws = workspace(OP_DPS_FWD, B, N, T, D, dt, q.device)
        rc = lib().tritt_dps_fwd(q.data_ptr(), k1.data_ptr(), k2.data_ptr(), v1.data_ptr(), v2.data_ptr(),
                                 o.data_ptr(), m.data_ptr(), B, N, T, D, dt, float(alpha), int(bool(causal)),
                                 int(k_diff), ws.data_ptr(), ws.numel(), status_word(q.device).data_ptr(), flags,
                                 _stream())
    _check(rc, "tritt_dps_fwd")
    launches += 1
    return ws


def dps_bwd(q, k1, k2, v1, v2, o, do, m, dq, dk1, dk2, dv1, dv2, alpha, causal, k_diff, flags=0, fwd_ws=None):
    """``fwd_ws``: the tensor ``dps_fwd`` returned for the same inputs, if it was kept untouched."""
    global launches
    B, N, T, D = q.shape
    dt = dtype_code(q.dtype)
    check_status(q.device, synchronize=False)
    with _on_device(q.device):
        ws = workspace(OP_DPS_BWD, B, N, T, D, dt, q.device)
        args = (q.data_ptr(), k1.data_ptr(), k2.data_ptr(), v1.data_ptr(), v2.data_ptr(), o.data_ptr(), do.data_ptr(),
                m.data_ptr(), dq.data_ptr(), dk1.data_ptr(), dk2.data_ptr(), dv1.data_ptr(), dv2.data_ptr(), B, N, T, D,
                dt, float(alpha), int(bool(causal)), int(k_diff), ws.data_ptr(), ws.numel())
        if fwd_ws is None:
            rc = lib().tritt_dps_bwd(*args, status_word(q.device).data_ptr(), flags, _stream())
        else:
            rc = lib().tritt_dps_bwd_saved(*args, fwd_ws.data_ptr(), fwd_ws.numel(), status_word(q.device).data_ptr(),
                                           flags, _stream())
    _check(rc, "tritt_dps_bwd")
    launches += 1


def tdp_fwd_noalloc(q, k1, k2, v1, v2, o, lse, alpha, causal, k1w, k2w, kkl, kkr, flags=0):
    """Forward through ``tritt_tdp_fwd_noalloc``: no workspace is passed; the library uses the scratch
    array built into its device image (for callers that are not allowed to allocate device memory).
    Calls on one GPU must not overlap in time."""
    global launches
    B, N, T, D = q.shape
    check_status(q.device, synchronize=False)
    with _on_device(q.device):
        rc = lib().tritt_tdp_fwd_noalloc(q.data_ptr(), k1.data_ptr(), k2.data_ptr(), v1.data_ptr(), v2.data_ptr(),
                                         o.data_ptr(), lse.data_ptr(), B, N, T, D, dtype_code(q.dtype), float(alpha),
                                         int(bool(causal)), _win(k1w, T), _win(k2w, T), _win(kkl, T), _win(kkr, T),
                                         status_word(q.device).data_ptr(), flags, _stream())
    _check(rc, "tritt_tdp_fwd_noalloc")
    launches += 1
