"""The rank-r LoRA kernels (q4_lora_project, q4_lora_grads) through the C ABI against fp32 torch products of
the same fp16 operands (the mathematics of Linear4bitLt.forward, models.py:58-66 of the reference, and of its
autograd gradients)."""
import pytest
import torch

from alpaca_lora_4bit_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rel(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm())


def project(x, w, scale):
    out = torch.full((x.shape[0], 64), 7.0, dtype=torch.float16, device=x.device)
    _lib.check(_lib.lib().q4_lora_project(x.data_ptr(), w.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1], w.shape[0],
                                          float(scale), _lib.stream_of(x)), "lora_project")
    return out


@pytest.mark.parametrize("M,C,r", [(1024, 4096, 8), (1024, 11008, 16), (37, 256, 3), (2048, 5120, 33), (9, 32, 64), (512, 8192, 1)])
def test_project_matches_fp32_product(M, C, r):
    g = torch.Generator(device=DEV).manual_seed(M + C + r)
    x = torch.randn(M, C, generator=g, device=DEV).half()
    w = (torch.randn(r, C, generator=g, device=DEV) * 0.05).half()
    out = project(x, w, 2.0)
    want = 2.0 * (x.float() @ w.float().t())
    assert rel(out[:, :r].float(), want) <= 1e-3
    assert int(out[:, r:].ne(0).sum()) == 0


@pytest.mark.parametrize("M,K,N,r", [(1024, 4096, 4096, 8), (1024, 4096, 11008, 16), (100, 64, 96, 5), (256, 5120, 1280, 64), (77, 320, 32, 40)])
def test_grads_match_fp32_products(M, K, N, r):
    g = torch.Generator(device=DEV).manual_seed(M + K + N + r)
    x = torch.randn(M, K, generator=g, device=DEV).half()
    dy = torch.randn(M, N, generator=g, device=DEV).half()
    u = torch.zeros(M, 64, dtype=torch.float16, device=DEV)
    v = torch.zeros(M, 64, dtype=torch.float16, device=DEV)
    u[:, :r] = torch.randn(M, r, generator=g, device=DEV).half()
    v[:, :r] = torch.randn(M, r, generator=g, device=DEV).half()
    want_a = v[:, :r].float().t() @ x.float()
    want_b = dy.float().t() @ u[:, :r].float()
    for a_on, b_on in ((True, True), (True, False), (False, True)):
        d_a = torch.full((r, K), 3.0, dtype=torch.float32, device=DEV)
        d_b = torch.full((N, r), 3.0, dtype=torch.float32, device=DEV)
        _lib.check(_lib.lib().q4_lora_grads(v.data_ptr(), x.data_ptr(), d_a.data_ptr() if a_on else None, K,
                                            dy.data_ptr(), u.data_ptr(), d_b.data_ptr() if b_on else None, N,
                                            M, r, _lib.stream_of(x)), "lora_grads")
        if a_on:
            assert rel(d_a, want_a) <= 1e-5
        else:
            assert float(d_a.min()) == 3.0 == float(d_a.max())
        if b_on:
            assert rel(d_b, want_b) <= 1e-5
        else:
            assert float(d_b.min()) == 3.0 == float(d_b.max())


def test_argument_checks():
    x = torch.zeros(8, 48, dtype=torch.float16, device=DEV)
    w = torch.zeros(4, 48, dtype=torch.float16, device=DEV)
    out = torch.zeros(8, 64, dtype=torch.float16, device=DEV)
    L = _lib.lib()
    assert L.q4_lora_project(x.data_ptr(), w.data_ptr(), out.data_ptr(), 8, 48, 4, 1.0, None) < 0        # 48 % 32
    assert L.q4_lora_project(x.data_ptr(), w.data_ptr(), out.data_ptr(), 8, 32, 65, 1.0, None) < 0       # r > 64
    assert L.q4_lora_project(None, w.data_ptr(), out.data_ptr(), 8, 32, 4, 1.0, None) < 0
    assert L.q4_lora_grads(None, None, None, 32, None, None, None, 32, 8, 4, None) == 0                  # nothing asked
