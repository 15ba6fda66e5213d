"""q4_gemv_static, the decode entry point for callers that cannot allocate device memory (a server
that owns all of HBM, a plugin barred from the host allocator, a latency path that must avoid the
synchronising cudaMalloc): its built-in scratch must give the same result as q4_gemv with a
caller-provided workspace, call after call.  Collected last on purpose."""
import pytest
import torch

from alpaca_lora_4bit_b200 import _lib, synth

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
REL_TOL = 2e-3


def _call(fn, x, L, y, M, K, N, extra):
    st = torch.cuda.current_stream().cuda_stream
    rc = fn(x.data_ptr(), L.qweight.data_ptr(), y.data_ptr(), L.scales.data_ptr(), L.qzeros.data_ptr(), None, None,
            M, K, N, K // 128, 128, _lib.Q4_F32, 0, *extra, st)
    _lib.check(rc, "gemv")


@pytest.mark.parametrize("M,K,N", [(1, 4096, 4096), (5, 4096, 11008)])
def test_static_scratch_matches_workspace_entry_point_twice(M, K, N):
    lib = _lib.lib()
    dev = torch.device(DEV)
    L = synth.make_layer(K, N, 128, False, seed=K + N).to(DEV)
    ws = _lib.workspace(dev, lib.q4_gemv_workspace_bytes(M, K, N))
    with torch.cuda.device(dev):
        for rep in range(2):                                   # two calls in a row share the built-in scratch
            x = synth.make_acts(M, K, seed=rep).to(DEV)
            want = torch.empty((M, N), dtype=torch.float32, device=DEV)
            got = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
            _call(lib.q4_gemv, x, L, want, M, K, N, (ws.data_ptr(), ws.numel()))
            _call(lib.q4_gemv_static, x, L, got, M, K, N, ())
            torch.cuda.synchronize()
            err = float((got.double() - want.double()).norm() / want.double().norm())
            assert err <= REL_TOL, f"call {rep}: relative error {err}"


def test_static_scratch_refuses_oversized_shapes():
    lib = _lib.lib()
    assert lib.q4_gemv_static_max_bytes() == 65536 + (2 << 20)
    L = synth.make_layer(128, 128, 128, False, seed=1).to(DEV)
    x = synth.make_acts(1, 128, seed=2).to(DEV)
    y = torch.empty((1, 128), dtype=torch.float32, device=DEV)
    with torch.cuda.device(torch.device(DEV)):
        # a shape the built-in scratch cannot serve is refused by size, before anything is launched
        # (the split partial sums of a 16-row product over 18432 columns)
        rc = lib.q4_gemv_static(x.data_ptr(), L.qweight.data_ptr(), y.data_ptr(), L.scales.data_ptr(), L.qzeros.data_ptr(),
                                None, None, 16, 8192, 18432, 64, 128, _lib.Q4_F32, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == -4 and b"built-in scratch" in lib.q4_last_error_string()
