"""The C ABI without a GPU: the library loads, exports what the header declares, and rejects
bad arguments before touching the device."""
import ctypes
import os
import re

import pytest

from alpaca_lora_4bit_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = set()
    for fn in os.listdir(os.path.join(ROOT, "include")):
        if fn.endswith(".h"):
            text = open(os.path.join(ROOT, "include", fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(q[24]_[a-z0-9_]+)\s*\(", text))
    return names


def test_header_and_binding_agree():
    assert _declared() == set(_lib.exported_symbols())


def test_library_exports_every_symbol():
    L = _lib.lib()
    for name in _declared():
        assert getattr(L, name) is not None
    assert L.q4_version() == 100


def test_bad_arguments_are_rejected_without_a_device():
    L = _lib.lib()
    fake = ctypes.c_void_p(0x1000)        # aligned, never dereferenced on the host
    # null pointer
    assert L.q4_recons_v2(None, fake, fake, fake, fake, 128, 128, 1, 0, None) == -1
    # N not a multiple of 8
    assert L.q4_recons_v2(fake, fake, fake, fake, fake, 128, 100, 1, 0, None) == -2
    assert b"multiples" in L.q4_last_error_string()
    # unknown dtype
    assert L.q4_recons_v2(fake, fake, fake, fake, fake, 128, 128, 1, 7, None) == -1
    # misaligned
    assert L.q4_recons_v2(ctypes.c_void_p(0x1004), fake, fake, fake, fake, 128, 128, 1, 0, None) == -3
    # gemv: M out of range, bad K, missing g_idx for act-order
    args = (fake, fake, fake, fake, fake, None, None)
    assert L.q4_gemv(*args, 17, 128, 128, 1, 128, 0, 0, None, 0, None) == -2
    assert L.q4_gemv(*args, 1, 100, 128, 1, 128, 0, 0, None, 0, None) == -2
    assert L.q4_gemv(*args, 1, 128, 128, 1, 128, 0, 2, None, 0, None) == -1
    assert L.q4_gemv(*args, 1, 128, 128, 1, 48, 0, 0, None, 0, None) == -2
    assert L.q4_gemv(*args, 1, 4192, 128, 1, 4192, 0, 4, None, 0, None) == -2       # v1 layer, K not a multiple of 128
    # decode status: null pointers and a size no decode workspace has are refused before any device call
    v = ctypes.c_uint(0)
    assert L.q4_gemv_status(None, 1 << 20, ctypes.byref(v)) == -1
    assert L.q4_gemv_status(fake, 100, ctypes.byref(v)) == -4
    assert L.q4_gemv_static_status(None) == -1
    assert L.q4_gemv_set_variant(3) == -1 and L.q4_gemv_set_variant(128) == -1 and L.q4_gemv_set_variant(4 + 8 + 1) == 0
    assert L.q4_gemv_set_variant(0) == 0
    assert L.q4_gemv_workspace_bytes(1, 100, 128) == 0
    assert L.q4_gemv_workspace_bytes(16, 11008, 4096) > 0
    # layer handle: made and destroyed on the host; bad geometry and null pointers give no handle
    h = ctypes.c_void_p()
    assert L.q4_layer_create(ctypes.byref(h), fake, fake, None, 128, 128, 1, 128) == -1 and not h.value
    assert L.q4_layer_create(ctypes.byref(h), fake, fake, fake, 100, 128, 1, 128) == -2 and not h.value
    assert L.q4_layer_create(None, fake, fake, fake, 128, 128, 1, 128) == -1
    assert L.q4_layer_create(ctypes.byref(h), fake, fake, fake, 128, 128, 1, 128) == 0 and h.value
    assert L.q4_layer_gemv(h, fake, fake, 17, None, 0, None) == -2            # the checks of q4_gemv apply
    assert L.q4_layer_gemv(None, fake, fake, 1, None, 0, None) == -1
    L.q4_layer_destroy(h)
    L.q4_layer_destroy(None)


def test_facade_refuses_cpu_tensors():
    import torch
    from alpaca_lora_4bit_b200 import quant_cuda
    q = torch.zeros((16, 128), dtype=torch.int32)
    with pytest.raises(RuntimeError, match="no CPU path"):
        quant_cuda.vecquant4recons_v2(q, torch.zeros((128, 128), dtype=torch.half), torch.zeros((1, 128), dtype=torch.half),
                                      torch.zeros((1, 16), dtype=torch.int32), torch.zeros(128, dtype=torch.int32))
    with pytest.raises(NotImplementedError):
        quant_cuda.vecquant3matmul()


def test_call_module_makes_the_same_foreign_call():
    """The `_q4call` extension is bound to the loaded library and returns its codes: a null handle is
    refused on the host (no device involved), the wrong number of arguments raises."""
    call = _lib.layer_gemv_call()
    assert call(0, 0x1000, 0x1000, 1, 0, 0, 0) == -1
    assert b"null handle" in _lib.lib().q4_last_error_string()
    L = _lib.lib()
    h = ctypes.c_void_p()
    fake = ctypes.c_void_p(0x1000)
    assert L.q4_layer_create(ctypes.byref(h), fake, fake, fake, 128, 128, 1, 128) == 0
    assert call(h.value, 0x1000, 0x1000, 17, 0, 0, 0) == -2            # M out of range: q4_gemv's own check
    L.q4_layer_destroy(h)
    with pytest.raises(TypeError):
        call(0, 0, 0)
    with pytest.raises(ValueError):
        call(0, 0, 0, -5, 0, 0, 0)
