"""The reference's own CUDA kernels (built unmodified into oracle/_ref/ by oracle/build_ref.py) against
the CPU oracle and against this library, on the same seeded inputs.  This is what pins the oracle to
the reference: reconstruct must agree bit for bit, the decode products within the tolerance."""
import pytest
import torch

from alpaca_lora_4bit_b200 import quant_cuda, synth
from oracle import build_ref
from oracle import q4_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
REL_TOL = 2e-3


@pytest.fixture(scope="module")
def ref():
    mod = build_ref.load()
    if mod is None:
        pytest.skip("oracle/_ref/quant_cuda_ref.so was not built (python oracle/build_ref.py)")
    return mod


def rel_fro(got, want):
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).norm() / want.norm())


def same_bits(a, b):
    a, b = a.cpu().contiguous(), b.cpu().contiguous()
    it = torch.int16 if a.dtype == torch.float16 else torch.int32
    return torch.equal(a.view(it), b.view(it))


@pytest.mark.parametrize("K,N,g,act", [(1024, 512, 128, True), (4096, 4096, 128, False), (2048, 1280, 64, True),
                                       (512, 256, -1, False)])
def test_reconstruct_v2_half_is_bit_identical(ref, K, N, g, act):
    layer = synth.make_layer(K, N, g, act, seed=K + N)
    L = layer.to(DEV)
    theirs = torch.zeros((K, N), dtype=torch.float16, device=DEV)
    ref.vecquant4recons_v2(L.qweight, theirs, L.scales, L.qzeros, L.g_idx)
    torch.cuda.synchronize()
    ours = torch.zeros_like(theirs)
    quant_cuda.vecquant4recons_v2(L.qweight, ours, L.scales, L.qzeros, L.g_idx)
    torch.cuda.synchronize()
    oracle = orc.recons_v2(layer.qweight, layer.scales, layer.qzeros, layer.g_idx)
    assert same_bits(theirs, oracle), "CPU oracle differs from the reference kernel"
    assert same_bits(ours, theirs), "library differs from the reference kernel"


def test_reconstruct_v2_float_scales(ref):
    layer = synth.make_layer(1024, 512, 128, True, seed=3)
    L = layer.to(DEV)
    s32 = (L.scales.float() * 1.37).contiguous()
    theirs = torch.zeros((1024, 512), dtype=torch.float32, device=DEV)
    ref.vecquant4recons_v2(L.qweight, theirs, s32, L.qzeros, L.g_idx)
    torch.cuda.synchronize()
    ours = torch.zeros_like(theirs)
    quant_cuda.vecquant4recons_v2(L.qweight, ours, s32, L.qzeros, L.g_idx)
    torch.cuda.synchronize()
    oracle = orc.recons_v2(layer.qweight, s32.cpu(), layer.qzeros, layer.g_idx)
    assert same_bits(theirs, oracle)
    assert same_bits(ours, theirs)


def test_reconstruct_v1_and_2bit(ref):
    gen = torch.Generator().manual_seed(5)
    layer = synth.make_layer(1024, 512, 1024, False, seed=5)
    sc = (torch.rand(512, generator=gen) * 0.018 + 0.002).half()
    ze = (sc.float() * torch.randint(1, 16, (512,), generator=gen)).half()
    theirs = torch.zeros((1024, 512), dtype=torch.float16, device=DEV)
    ref.vecquant4recons_v1(layer.qweight.to(DEV), theirs, sc.to(DEV), ze.to(DEV))
    torch.cuda.synchronize()
    ours = torch.zeros_like(theirs)
    quant_cuda.vecquant4recons_v1(layer.qweight.to(DEV), ours, sc.to(DEV), ze.to(DEV))
    torch.cuda.synchronize()
    assert same_bits(theirs, orc.recons_v1(layer.qweight, sc, ze)) and same_bits(ours, theirs)

    l2 = synth.make_layer(2048, 512, 128, True, seed=6, bits=2)
    L2 = l2.to(DEV)
    theirs = torch.zeros((2048, 512), dtype=torch.float16, device=DEV)
    ref.vecquant2recons_v2(L2.qweight, theirs, L2.scales, L2.qzeros, L2.g_idx)
    torch.cuda.synchronize()
    ours = torch.zeros_like(theirs)
    quant_cuda.vecquant2recons_v2(L2.qweight, ours, L2.scales, L2.qzeros, L2.g_idx)
    torch.cuda.synchronize()
    assert same_bits(theirs, orc.recons2_v2(l2.qweight, l2.scales, l2.qzeros, l2.g_idx)) and same_bits(ours, theirs)


@pytest.mark.parametrize("M", [1, 5])
def test_decode_products_against_reference_variants(ref, M):
    K, N = 4096, 4096
    layer = synth.make_layer(K, N, 128, False, seed=9)
    L = layer.to(DEV)
    x = synth.make_acts(M, K, seed=M).to(DEV)
    exact = orc.gemv_fp32(x.cpu(), layer.qweight, layer.scales, layer.qzeros, layer.g_idx)
    # the reference's default decode kernel: half in, float out, groups from the row index
    y_ref = torch.zeros((M, N), dtype=torch.float32, device=DEV)
    ref.vecquant4matmul_old_faster(x, L.qweight, y_ref, L.scales.float(), L.qzeros, 128, K // 2)
    # its fp32 kernel with g_idx
    y_ref32 = torch.zeros((M, N), dtype=torch.float32, device=DEV)
    ref.vecquant4matmul(x.float(), L.qweight, y_ref32, L.scales.float(), L.qzeros, L.g_idx)
    torch.cuda.synchronize()
    y_ours = torch.zeros((M, N), dtype=torch.float32, device=DEV)
    quant_cuda.vecquant4matmul_old_faster(x, L.qweight, y_ours, L.scales.float(), L.qzeros, 128, K // 2)
    torch.cuda.synchronize()
    assert rel_fro(y_ref32, exact) <= REL_TOL            # oracle vs the reference's fp32 kernel
    assert rel_fro(y_ref, exact) <= 5e-3                 # its half2 kernel rounds every dequantised pair to fp16
    assert rel_fro(y_ours, y_ref32) <= REL_TOL
    assert rel_fro(y_ours, exact) <= rel_fro(y_ref, exact) + 1e-4   # never worse than the kernel it replaces


def test_act_order_decode_against_reference(ref):
    K, N, M = 2048, 1024, 3
    layer = synth.make_layer(K, N, 128, True, seed=11)
    L = layer.to(DEV)
    x = synth.make_acts(M, K, seed=12).to(DEV)
    y_ref = torch.zeros((M, N), dtype=torch.float32, device=DEV)
    ref.vecquant4matmul(x.float(), L.qweight, y_ref, L.scales.float(), L.qzeros, L.g_idx)
    torch.cuda.synchronize()
    y_ours = torch.zeros((M, N), dtype=torch.float32, device=DEV)
    quant_cuda.vecquant4matmul(x.float(), L.qweight, y_ours, L.scales.float(), L.qzeros, L.g_idx)
    torch.cuda.synchronize()
    exact = orc.gemv_fp32(x.cpu(), layer.qweight, layer.scales, layer.qzeros, layer.g_idx)
    assert rel_fro(y_ref, exact) <= REL_TOL and rel_fro(y_ours, y_ref) <= REL_TOL
