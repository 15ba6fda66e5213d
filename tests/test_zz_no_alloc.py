"""q4_gemv_static, the decode entry point for callers that cannot allocate device memory (a server
that owns all of HBM, a plugin barred from the host allocator, a latency path that must avoid the
synchronising cudaMalloc): its built-in scratch must give the same result as q4_gemv with a
caller-provided workspace, call after call.  The shapes are ones whose partial sums really travel
through the scratch: an even split of all units over the CTAs (straddled column tiles meet there)
and an act-order layer (its K-splits meet there).  Collected last on purpose."""
import ctypes

import pytest
import torch

from alpaca_lora_4bit_b200 import _lib, quant_cuda, synth
from oracle import q4_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
REL_TOL = 2e-3


def _call(fn, x, L, y, M, K, N, flags, extra):
    st = torch.cuda.current_stream().cuda_stream
    rc = fn(x.data_ptr(), L.qweight.data_ptr(), y.data_ptr(), L.scales.data_ptr(), L.qzeros.data_ptr(),
            L.g_idx.data_ptr() if flags & _lib.GEMV_ACT_ORDER else None, None,
            M, K, N, K // 128, 128, _lib.Q4_F32, flags, *extra, st)
    _lib.check(rc, "gemv")


def _rel(a, b):
    return float((a.double().cpu() - b.double().cpu()).norm() / b.double().cpu().norm())


# (M, K, N, act-order, variant): variant 4 forces the even split on shapes that would get whole tiles
@pytest.mark.parametrize("M,K,N,act,variant", [(1, 4096, 4096, False, 4), (5, 4096, 11008, False, 4), (3, 32768, 1024, False, 0),
                                               (8, 28672, 512, False, 0), (2, 4096, 4096, True, 0), (1, 4096, 4096, False, 0)])
def test_static_scratch_matches_workspace_entry_point_twice(M, K, N, act, variant):
    lib = _lib.lib()
    dev = torch.device(DEV)
    layer = synth.make_layer(K, N, 128, act, seed=K + N)
    L = layer.to(DEV)
    flags = _lib.GEMV_ACT_ORDER if act else 0
    ws = _lib.workspace(dev, lib.q4_gemv_workspace_bytes(M, K, N))
    status = ctypes.c_uint(1)
    quant_cuda.gemv_set_variant(variant)
    try:
        with torch.cuda.device(dev):
            for rep in range(2):                                   # two calls in a row share the built-in scratch
                x = synth.make_acts(M, K, seed=rep)
                oracle = orc.gemv_fp32(x, layer.qweight, layer.scales, layer.qzeros, layer.g_idx)
                xd = x.to(DEV)
                want = torch.empty((M, N), dtype=torch.float32, device=DEV)
                got = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
                _call(lib.q4_gemv, xd, L, want, M, K, N, flags, (ws.data_ptr(), ws.numel()))
                _call(lib.q4_gemv_static, xd, L, got, M, K, N, flags, ())
                torch.cuda.synchronize()
                assert _rel(got, want) <= REL_TOL, f"call {rep}: against q4_gemv"
                assert _rel(got, oracle) <= REL_TOL, f"call {rep}: against the oracle"
                _lib.check(lib.q4_gemv_static_status(ctypes.byref(status)), "static status")
                assert status.value == 0
    finally:
        quant_cuda.gemv_set_variant(0)


def test_static_scratch_refuses_oversized_shapes():
    lib = _lib.lib()
    assert lib.q4_gemv_static_max_bytes() == 131072 + (2 << 20)
    L = synth.make_layer(128, 128, 128, False, seed=1).to(DEV)
    x = synth.make_acts(1, 128, seed=2).to(DEV)
    y = torch.empty((1, 128), dtype=torch.float32, device=DEV)
    with torch.cuda.device(torch.device(DEV)):
        # a shape the built-in scratch cannot serve is refused by size, before anything is launched
        # (the split partial sums of a 16-row product over 18432 columns)
        rc = lib.q4_gemv_static(x.data_ptr(), L.qweight.data_ptr(), y.data_ptr(), L.scales.data_ptr(), L.qzeros.data_ptr(),
                                None, None, 16, 8192, 18432, 64, 128, _lib.Q4_F32, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == -4 and b"built-in scratch" in lib.q4_last_error_string()
