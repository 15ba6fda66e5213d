"""ctypes binding of ``libq4b200.so`` (the C ABI declared in ``include/q4b200.h``).

The library is loaded on first use.  There is no fallback: if it is missing and cannot be
built, or a call returns an error code, a ``RuntimeError`` carrying the library's own message
is raised.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_char_p, c_int, c_size_t, c_uint, c_void_p

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libq4b200.so")

Q4_F16, Q4_F32 = 0, 1
GEMV_ACCUMULATE, GEMV_ACT_ORDER, GEMV_V1 = 1, 2, 4

_lib = None
_lock = threading.Lock()

# name -> (restype, argtypes); mirrors include/q4b200.h one to one
_SIGNATURES = {
    "q4_version": (c_int, []),
    "q4_last_error_string": (c_char_p, []),
    "q4_recons_v2": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "q4_recons_v1": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "q2_recons_v2": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "q4_gemv_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "q4_layer_create": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int]),
    "q4_layer_gemv": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_size_t, c_void_p]),
    "q4_layer_destroy": (None, [c_void_p]),
    "q4_layer_set_next": (c_int, [c_void_p, c_void_p]),
    "q4_gemv_set_trace": (c_int, [c_void_p]),
    "q4_gemm_set_trace": (c_int, [c_void_p]),
    "q4_gemm_set_variant": (c_int, [c_int]),
    "q4_gemv_set_variant": (c_int, [c_int]),
    "q4_gemv_static_max_bytes": (c_size_t, []),
    "q4_gemv_static": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_int, c_int, c_int, c_int, c_int, c_int, c_uint, c_void_p]),
    "q4_gemm_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                            c_int, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "q4_gemm_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                            c_int, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "q4_gemm_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "q4_zero_term_table": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "q4_gemm_fwd_residual": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "q4_gemm_fwd_table": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_int, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "q4_gemm_bwd_table": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                  c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "q4_gemm_fwd_swiglu": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                   c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "q4_rmsnorm_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, ctypes.c_float, c_void_p]),
    "q4_rmsnorm_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "q4_swiglu_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "q4_swiglu_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "q4_rope": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "q4_lora_project": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, ctypes.c_float, c_void_p]),
    "q4_lora_grads": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "q4_adamw_flat": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, ctypes.c_float, ctypes.c_float, ctypes.c_float,
                              ctypes.c_float, ctypes.c_float, ctypes.c_float, c_void_p, ctypes.c_float, ctypes.c_float, c_int, c_void_p, c_void_p]),
    "q4_device_status": (c_int, [ctypes.POINTER(c_uint)]),
    "q4_gemv_status": (c_int, [c_void_p, c_size_t, ctypes.POINTER(c_uint)]),
    "q4_gemv_static_status": (c_int, [ctypes.POINTER(c_uint)]),
    "q4_gemv": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                        c_int, c_int, c_int, c_int, c_int, c_int, c_uint, c_void_p, c_size_t, c_void_p]),
}


def exported_symbols():
    return sorted(_SIGNATURES)


def lib() -> ctypes.CDLL:
    """The loaded library (built in-tree on first use when nvcc is present)."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            from . import build as _build
            _build.build()
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)          # AttributeError here = header and library disagree
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


_layer_gemv_call = None


def layer_gemv_call():
    """``q4_layer_gemv`` as a callable of seven Python ints that returns the C return code: the ``_q4call``
    extension module (built in-tree with the C compiler on first use), bound to the loaded library.  It
    makes the same foreign call as the ctypes binding without ctypes' per-argument conversion."""
    global _layer_gemv_call
    if _layer_gemv_call is not None:
        return _layer_gemv_call
    handle = lib()
    with _lock:
        if _layer_gemv_call is None:
            from . import build as _build
            _build.build_call()
            from . import _q4call
            _q4call.bind(ctypes.cast(handle.q4_layer_gemv, c_void_p).value)
            _layer_gemv_call = _q4call.layer_gemv
    return _layer_gemv_call


def check(code: int, what: str) -> None:
    if code != 0:
        msg = lib().q4_last_error_string().decode("utf-8", "replace")
        raise RuntimeError(f"q4b200 {what} failed ({code}): {msg}")


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def stream_of(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def require_cuda(*tensors) -> torch.device:
    """All tensors must live on one CUDA device and be contiguous; returns that device."""
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("q4b200: tensors must be CUDA tensors (there is no CPU path)")
        if not t.is_contiguous():
            raise RuntimeError("q4b200: tensors must be contiguous")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"q4b200: tensors on different devices ({dev} vs {t.device})")
    return dev


class on_device:
    """Make ``dev`` the current CUDA device for the duration of a call; free when it already is."""
    __slots__ = ("dev", "prev")

    def __init__(self, dev: torch.device):
        self.dev = dev.index if dev.index is not None else torch.cuda.current_device()
        self.prev = -1

    def __enter__(self):
        cur = torch.cuda.current_device()
        if cur != self.dev:
            self.prev = cur
            torch.cuda.set_device(self.dev)
        return self

    def __exit__(self, *exc):
        if self.prev >= 0:
            torch.cuda.set_device(self.prev)
        return False


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float16:
        return Q4_F16
    if dt == torch.float32:
        return Q4_F32
    raise RuntimeError(f"q4b200: unsupported dtype {dt} (float16 or float32)")


_workspaces: dict = {}
_WS_BYTES = 4 << 20          # covers q4_gemv_workspace_bytes() of every shape the decode kernels accept


def workspace_for(device: torch.device, stream_handle: int) -> torch.Tensor:
    """The decode workspace of one (device, stream): allocated zeroed on first use, then reused."""
    key = (device.index, stream_handle)
    ws = _workspaces.get(key)
    if ws is None:
        ws = torch.zeros(_WS_BYTES, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


_gemm_workspaces: dict = {}


def gemm_workspace_for(device: torch.device, stream_handle: int, nbytes: int) -> torch.Tensor:
    """Scratch of the fused GEMM for one (device, stream): zeroed when (re)allocated, only ever grows.
    The kernels leave its counter head zero, so calls ordered on the stream can share it."""
    key = (device.index, stream_handle)
    ws = _gemm_workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 24 << 20), dtype=torch.uint8, device=device)
        _gemm_workspaces[key] = ws
    return ws


def workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Per-(device, stream) zero-initialised scratch that only ever grows.

    The decode kernel keeps its arrival counters zero between launches, so the buffer is
    cleared once, when it is (re)allocated.
    """
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws
