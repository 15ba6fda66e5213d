"""Parity of the CUDA kernels (through the C ABI) with the CPU oracle and the golden fixtures."""
import glob
import os

import numpy as np
import pytest
import torch

from alpaca_lora_4bit_b200 import _lib, quant_cuda, synth
from oracle import q4_oracle as orc

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda:0"
REL_TOL = 2e-3          # relative Frobenius error allowed on matmul outputs


def rel_fro(got, want):
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).norm() / want.norm())


def bits_equal(a, b):
    a, b = a.cpu().contiguous(), b.cpu().contiguous()
    nan = torch.isnan(b)
    if not torch.equal(torch.isnan(a), nan):
        return False
    it = torch.int16 if a.dtype == torch.float16 else torch.int32
    return torch.equal(a.view(it)[~nan], b.view(it)[~nan])


def guarded(shape, dtype, fill=-777.0):
    """Output tensor with canary rows before and after, to catch out-of-bounds stores."""
    rows = shape[0]
    full = torch.full((rows + 16, shape[1]), fill, dtype=dtype, device=DEV)
    return full, full[8:8 + rows]


def canaries_intact(full, rows, fill=-777.0):
    return bool((full[:8] == fill).all()) and bool((full[8 + rows:] == fill).all())


def recons_gpu(layer, dtype=torch.float16):
    L = layer.to(DEV)
    full, out = guarded((layer.K, layer.N), dtype)
    sc = L.scales.to(dtype)
    if layer.bits == 4:
        quant_cuda.vecquant4recons_v2(L.qweight, out, sc, L.qzeros, L.g_idx)
    else:
        quant_cuda.vecquant2recons_v2(L.qweight, out, sc, L.qzeros, L.g_idx)
    torch.cuda.synchronize()
    assert canaries_intact(full, layer.K)
    return out


def load_layer(npz):
    d = np.load(npz)
    return synth.QuantLayer(torch.from_numpy(d["qweight"]), torch.from_numpy(d["qzeros"]),
                            torch.from_numpy(d["scales"]), torch.from_numpy(d["g_idx"]),
                            int(d["K"]), int(d["N"]), int(d["groupsize"]), int(d["bits"])), d


# ---------------------------------------------------------------- reconstruct: bit-exact
@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "recons*_v2_*.npz"))))
def test_recons_v2_golden(path):
    layer, d = load_layer(path)
    assert bits_equal(recons_gpu(layer), torch.from_numpy(d["w"]))


def test_recons_v1_golden():
    d = np.load(os.path.join(GOLD, "recons_v1_k128_n64.npz"))
    qw = torch.from_numpy(d["qweight"]).to(DEV)
    full, out = guarded((128, 64), torch.float16)
    quant_cuda.vecquant4recons_v1(qw, out, torch.from_numpy(d["scales"]).to(DEV).reshape(-1),
                                  torch.from_numpy(d["zeros"]).to(DEV).reshape(-1))
    torch.cuda.synchronize()
    assert canaries_intact(full, 128)
    assert bits_equal(out, torch.from_numpy(d["w"]))


@pytest.mark.parametrize("K,N,g,act", [(4096, 4096, 128, False), (4096, 4096, 128, True), (1024, 11008, 128, True),
                                       (5120, 1024, 128, True), (256, 136, 64, True), (4096, 4096, -1, False),
                                       (8, 8, 8, False)])
def test_recons_v2_oracle(K, N, g, act):
    layer = synth.make_layer(K, N, g, act, seed=K + N)
    want = orc.recons_v2(layer.qweight, layer.scales, layer.qzeros, layer.g_idx)
    assert bits_equal(recons_gpu(layer), want)


def test_recons_v2_fp32_scales():
    layer = synth.make_layer(1024, 512, 128, True, seed=5)
    layer.scales = layer.scales  # fp16 source
    L32 = synth.QuantLayer(layer.qweight, layer.qzeros, layer.scales.float() * 1.37, layer.g_idx, 1024, 512, 128)
    want = orc.recons_v2(L32.qweight, L32.scales, L32.qzeros, L32.g_idx)
    got = recons_gpu(L32, torch.float32)
    assert bits_equal(got, want)


def test_recons2_v2_oracle():
    layer = synth.make_layer(2048, 1024, 128, True, seed=9, bits=2)
    want = orc.recons2_v2(layer.qweight, layer.scales, layer.qzeros, layer.g_idx)
    assert bits_equal(recons_gpu(layer), want)
    got32 = recons_gpu(synth.QuantLayer(layer.qweight, layer.qzeros, layer.scales.float(), layer.g_idx,
                                        2048, 1024, 128, 2), torch.float32)
    assert bits_equal(got32, orc.recons2_v2(layer.qweight, layer.scales.float(), layer.qzeros, layer.g_idx))


def test_recons_v1_oracle_both_dtypes():
    gen = torch.Generator().manual_seed(21)
    layer = synth.make_layer(2048, 1024, 2048, False, seed=21)
    sc = (torch.rand(1024, generator=gen) * 0.018 + 0.002)
    ze = sc * torch.randint(1, 16, (1024,), generator=gen)
    for dt in (torch.float16, torch.float32):
        full, out = guarded((2048, 1024), dt)
        quant_cuda.vecquant4recons_v1(layer.qweight.to(DEV), out, sc.to(dt).to(DEV), ze.to(dt).to(DEV))
        torch.cuda.synchronize()
        assert canaries_intact(full, 2048)
        assert bits_equal(out, orc.recons_v1(layer.qweight, sc.to(dt), ze.to(dt)))


def test_recons_idempotent_and_full_overwrite():
    layer = synth.make_layer(512, 256, 128, True, seed=2).to(DEV)
    a = torch.full((512, 256), float("nan"), dtype=torch.float16, device=DEV)
    quant_cuda.vecquant4recons_v2(layer.qweight, a, layer.scales, layer.qzeros, layer.g_idx)
    b = torch.zeros_like(a)
    quant_cuda.vecquant4recons_v2(layer.qweight, b, layer.scales, layer.qzeros, layer.g_idx)
    assert not torch.isnan(a).any() and torch.equal(a, b)


# ---------------------------------------------------------------- decode product
def gemv_gpu(layer, x, ydtype=torch.float16, flags=0, groupsize=None, y0=None, bias=None):
    L = layer.to(DEV)
    M = x.shape[0]
    full, y = guarded((M, layer.N), ydtype)
    if y0 is not None:
        y.copy_(y0)
    quant_cuda.gemv(x.to(DEV), L.qweight, y, L.scales, L.qzeros,
                    L.g_idx if flags & _lib.GEMV_ACT_ORDER else None,
                    groupsize or layer.groupsize, flags, bias=bias)
    torch.cuda.synchronize()
    assert canaries_intact(full, M)
    return y


@pytest.mark.parametrize("name", ["recons_v2_seq_k128_n64_g32.npz", "recons_v2_act_k128_n64_g32.npz",
                                  "recons_v2_act_k256_n32_g128.npz"])
def test_gemv_golden(name):
    layer, d = load_layer(os.path.join(GOLD, name))
    act = "act" in name
    y = gemv_gpu(layer, torch.from_numpy(d["x"]), torch.float32, _lib.GEMV_ACT_ORDER if act else 0)
    assert rel_fro(y, torch.from_numpy(d["y"])) <= REL_TOL


@pytest.mark.parametrize("K,N", [(4096, 4096), (4096, 11008), (11008, 4096)])
@pytest.mark.parametrize("M", [1, 4, 8, 16])
def test_gemv_llama7b_shapes(K, N, M):
    layer = synth.make_layer(K, N, 128, False, seed=K // 7 + N)
    x = synth.make_acts(M, K, seed=M)
    want = orc.gemv_fp32(x, layer.qweight, layer.scales, layer.qzeros, layer.g_idx)
    for dt in (torch.float16, torch.float32):
        assert rel_fro(gemv_gpu(layer, x, dt), want) <= REL_TOL
    # against the reference composition too: fp16 reconstruct, fp32 matmul
    ref = orc.matmul4bit_ref(x, layer.qweight, layer.scales, layer.qzeros, layer.g_idx)
    assert rel_fro(gemv_gpu(layer, x, torch.float32), ref) <= REL_TOL


@pytest.mark.parametrize("M", [1, 3, 9, 16])
@pytest.mark.parametrize("K,N,g", [(5120, 5120, 128), (512, 96, 64), (1024, 2048, 32)])
def test_gemv_act_order(K, N, g, M):
    layer = synth.make_layer(K, N, g, True, seed=K + M)
    x = synth.make_acts(M, K, seed=M + 50)
    want = orc.gemv_fp32(x, layer.qweight, layer.scales, layer.qzeros, layer.g_idx)
    assert rel_fro(gemv_gpu(layer, x, torch.float32, _lib.GEMV_ACT_ORDER), want) <= REL_TOL


@pytest.mark.parametrize("K,N,g,M", [(32, 32, 32, 1), (64, 32, 32, 5), (4096, 32, 128, 2), (2048, 4096, 64, 7),
                                     (8192, 1024, -1, 16), (1056, 64, 96, 3)])
def test_gemv_ragged_sizes(K, N, g, M):
    layer = synth.make_layer(K, N, g, False, seed=K + N + M)
    x = synth.make_acts(M, K, seed=3)
    want = orc.gemv_fp32(x, layer.qweight, layer.scales, layer.qzeros, layer.g_idx)
    assert rel_fro(gemv_gpu(layer, x, torch.float32), want) <= REL_TOL


@pytest.mark.parametrize("K,N,g,M", [(1056, 64, 32, 1), (4160, 2048, 128, 1), (4160, 2048, 128, 12), (4224, 2048, 384, 1),
                                     (4224, 2048, 384, 5), (4224, 1024, 128, 13), (1152, 512, 128, 3)])
def test_gemv_half_filled_last_unit(K, N, g, M):
    """Layers whose last 256-row unit is partly out of bounds, with groups of 128-row multiples: the lean
    kernel where it applies (K a multiple of 128, groups of 128), the general streaming instance elsewhere."""
    layer = synth.make_layer(K, N, g, False, seed=K + N + M)
    x = synth.make_acts(M, K, seed=3)
    want = orc.gemv_fp32(x, layer.qweight, layer.scales, layer.qzeros, layer.g_idx)
    assert rel_fro(gemv_gpu(layer, x, torch.float32), want) <= REL_TOL
    torch.cuda.synchronize()
    assert quant_cuda.device_status() == 0


def test_gemv_accumulates_bias_and_is_reproducible():
    layer = synth.make_layer(4096, 4096, 128, False, seed=77)
    x = synth.make_acts(4, 4096, seed=8)
    want = orc.gemv_fp32(x, layer.qweight, layer.scales, layer.qzeros, layer.g_idx)
    y0 = torch.randn(4, 4096)
    y = gemv_gpu(layer, x, torch.float32, _lib.GEMV_ACCUMULATE, y0=y0.to(DEV))
    assert rel_fro(y, want + y0.double()) <= REL_TOL
    bias = torch.randn(4096).half()
    yb = gemv_gpu(layer, x, torch.float32, 0, bias=bias.to(DEV))
    assert rel_fro(yb, want + bias.double()) <= REL_TOL
    a = gemv_gpu(layer, x, torch.float32)
    for _ in range(3):
        assert torch.equal(a, gemv_gpu(layer, x, torch.float32))


def test_gemv_linearity_full_size():
    """y(x1 + x2) = y(x1) + y(x2) at the largest decode case (M=16, 11008x4096), where the
    scalar oracle is too slow to be the checker; the fp16 rounding of x1 + x2 is inside the tolerance."""
    layer = synth.make_layer(11008, 4096, 128, False, seed=1)
    x1 = synth.make_acts(16, 11008, seed=31)
    x2 = synth.make_acts(16, 11008, seed=32)
    xs = (x1.float() + x2.float()).half()
    y1, y2, ys = (gemv_gpu(layer, v, torch.float32) for v in (x1, x2, xs))
    assert rel_fro(ys, y1 + y2) <= REL_TOL


def test_gemv_v1_facade():
    gen = torch.Generator().manual_seed(23)
    layer = synth.make_layer(4096, 1024, 4096, False, seed=23)
    sc = (torch.rand(1024, generator=gen) * 0.018 + 0.002).half()
    ze = (sc.float() * torch.randint(1, 16, (1024,), generator=gen)).half()
    x = synth.make_acts(2, 4096, seed=4)
    y = torch.zeros((2, 1024), dtype=torch.float16, device=DEV)
    quant_cuda.vecquant4matmul_v1_faster(x.to(DEV), layer.qweight.to(DEV), y, sc.reshape(-1, 1).to(DEV),
                                         ze.reshape(-1, 1).to(DEV))
    want = orc.matmul_recons(x, orc.recons_v1(layer.qweight, sc, ze))
    assert rel_fro(y, want) <= REL_TOL


@pytest.mark.parametrize("M", [1, 4, 8, 13])
@pytest.mark.parametrize("K,N", [(4096, 4096), (11008, 1024), (1024, 5120), (512, 4768), (4224, 2048), (384, 512)])
def test_gemv_v1_shapes(K, N, M):
    """First-format layers (one scale and one fp16 zero term per column) through the C ABI, against the
    oracle's reconstruct + matmul; output rows beyond M untouched.  K = 4224 and 384 end in a half-filled
    256-row unit (the reference's kernel takes K in multiples of 128)."""
    gen = torch.Generator().manual_seed(K + N + M)
    layer = synth.make_layer(K, N, K, False, seed=K + N)
    sc = (torch.rand(N, generator=gen) * 0.018 + 0.002).half()
    ze = (sc.float() * torch.randint(1, 16, (N,), generator=gen)).half()
    x = synth.make_acts(M, K, seed=M)
    full, y = guarded((M, N), torch.float16)
    L = _lib.lib()
    ws = _lib.workspace(torch.device(DEV), L.q4_gemv_workspace_bytes(M, K, N))
    xd, qd, sd, zd = x.to(DEV), layer.qweight.to(DEV), sc.to(DEV), ze.to(DEV)
    _lib.check(L.q4_gemv(xd.data_ptr(), qd.data_ptr(), y.data_ptr(), sd.data_ptr(), zd.data_ptr(), None, None, M, K, N, 1, K,
                         _lib.Q4_F16, _lib.GEMV_V1, ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream), "v1")
    torch.cuda.synchronize()
    assert canaries_intact(full, M)
    want = orc.matmul_recons(x, orc.recons_v1(layer.qweight, sc, ze))
    assert rel_fro(y, want) <= REL_TOL
    assert quant_cuda.device_status() == 0


def test_facade_matmul_variants_add_into_mul():
    layer = synth.make_layer(4096, 4096, 128, False, seed=41)
    L = layer.to(DEV)
    x = synth.make_acts(20, 4096, seed=42)          # more than one 16-row slab
    want = orc.gemv_fp32(x, layer.qweight, layer.scales, layer.qzeros, layer.g_idx)
    y = torch.ones((20, 4096), dtype=torch.float32, device=DEV)
    quant_cuda.vecquant4matmul_old_faster(x.to(DEV), L.qweight, y, L.scales.float(), L.qzeros, 128, 2048)
    assert rel_fro(y, want + 1.0) <= REL_TOL
    y = torch.zeros((20, 4096), dtype=torch.float16, device=DEV)
    quant_cuda.vecquant4matmul_faster(x.to(DEV), L.qweight, y, L.scales, L.qzeros, L.g_idx, 2048)
    assert rel_fro(y, want) <= REL_TOL
    y = torch.zeros((20, 4096), dtype=torch.float32, device=DEV)
    quant_cuda.vecquant4matmul(x.float().to(DEV), L.qweight, y, L.scales.float(), L.qzeros, L.g_idx)
    assert rel_fro(y, want) <= REL_TOL


@pytest.mark.parametrize("M", [1, 2])
@pytest.mark.parametrize("K,N", [(4096, 5120), (1024, 5120), (2048, 9600), (512, 4768)])
def test_gemv_work_dealing_modes(K, N, M):
    """Column-tile counts just above the SM count (160, 300 and 149 tiles on a 148-SM part), where the
    lean kernel chooses between whole tiles per CTA and an even split of all units whose straddled
    tiles meet in the workspace.  Twice on the same workspace: the counters must come back to zero."""
    layer = synth.make_layer(K, N, 128, False, seed=K + N)
    x = synth.make_acts(M, K, seed=M + 5)
    want = orc.gemv_fp32(x, layer.qweight, layer.scales, layer.qzeros, layer.g_idx)
    first = gemv_gpu(layer, x, torch.float32)
    again = gemv_gpu(layer, x, torch.float32)
    assert rel_fro(first, want) <= REL_TOL
    assert torch.equal(first, again)
    for ws in _lib._workspaces.values():
        assert int(ws[:65536].view(torch.int32).abs().sum()) == 0


@pytest.mark.parametrize("M", [1, 3, 8])
@pytest.mark.parametrize("K,N", [(4096, 4096), (1024, 5120), (11008, 4096), (4224, 9600), (8192, 8192)])
def test_gemv_x_per_unit_and_per_cta_agree(K, N, M):
    """The fp16-MMA decode kernel (variant bit 16) with x brought and re-laid per 4 KiB unit (17) and with the
    whole of x re-laid once per CTA (18; K = 4224 has a half-filled last unit whose padding must read as zero):
    both within tolerance of the oracle, and its automatic choice (16) equal to one of them bit for bit.  The
    default (0) is the int8-MMA kernel where it applies: within tolerance as well."""
    layer = synth.make_layer(K, N, 128, False, seed=K // 7 + N)
    x = synth.make_acts(M, K, seed=3 + M)
    want = orc.gemv_fp32(x, layer.qweight, layer.scales, layer.qzeros, layer.g_idx)
    got = {}
    try:
        for v in (17, 18, 16, 0):
            quant_cuda.gemv_set_variant(v)
            got[v] = gemv_gpu(layer, x, torch.float32)
            assert rel_fro(got[v], want) <= REL_TOL, v
    finally:
        quant_cuda.gemv_set_variant(0)
    assert torch.equal(got[16], got[17]) or torch.equal(got[16], got[18])
    torch.cuda.synchronize()
    assert quant_cuda.device_status() == 0


@pytest.mark.parametrize("M", [2, 5, 8, 9, 11, 16])
@pytest.mark.parametrize("K,N", [(4096, 4096), (11008, 4096), (4096, 11008), (2048, 1024), (512, 8192)])
def test_gemv_rows_kernel(K, N, M):
    """2..16 rows on the int8-MMA kernel fed by the conversion pass (its 8-row and its 16-row form), fp16 and fp32
    outputs, accumulate and bias; twice, since the digits of x live in the workspace between the two kernels."""
    layer = synth.make_layer(K, N, 128, False, seed=K + N + M)
    x = synth.make_acts(M, K, seed=M)
    want = orc.gemv_fp32(x, layer.qweight, layer.scales, layer.qzeros, layer.g_idx)
    first = gemv_gpu(layer, x, torch.float32)
    assert rel_fro(first, want) <= 1e-4                        # exact integer sums: only x is rounded (block fixed point)
    assert torch.equal(first, gemv_gpu(layer, x, torch.float32))
    assert rel_fro(gemv_gpu(layer, x, torch.float16), want) <= REL_TOL
    y0 = torch.randn(M, N)
    bias = torch.randn(N).half()
    got = gemv_gpu(layer, x, torch.float32, _lib.GEMV_ACCUMULATE, y0=y0.to(DEV), bias=bias.to(DEV))
    assert rel_fro(got, want + y0.double() + bias.double()) <= REL_TOL
    assert quant_cuda.device_status() == 0


def _head_is_zero():
    # counters and status word (first 64 KiB) and the exchange slots of the one-row kernel (second 64 KiB, whose
    # last word is a running count that is never reset)
    return all(int(ws[:131072 - 4].view(torch.int32).abs().sum()) == 0 for ws in _lib._workspaces.values())


@pytest.mark.parametrize("M", [1, 3, 8])
@pytest.mark.parametrize("K,N,forced", [(32768, 1024, False), (28672, 512, False), (4096, 4096, True), (4096, 11008, True),
                                        (11008, 4096, True), (4224, 2048, True)])
def test_gemv_even_split_meets_in_workspace(K, N, forced, M):
    """The lean kernel dealing an even share of all units to every CTA: column tiles straddle CTAs, their
    partial sums go through the workspace (partial, fence, counter, the last CTA to arrive adds them in CTA
    order).  Long-K, few-column layers take this dealing by the host's own choice; on the LLaMA-7B shapes
    (and one with a half-filled last unit) it is forced with variant bit 4: the one-row kernel's exchange of
    (sum, flag) words at one and at two CTAs per SM (4, 12) and the counter scheme of the other kernel (20).
    Twice on one workspace: same bits, counters and slots back to zero, no expired wait."""
    layer = synth.make_layer(K, N, 128, False, seed=K // 5 + N + M)
    x = synth.make_acts(M, K, seed=M + 9)
    want = orc.gemv_fp32(x, layer.qweight, layer.scales, layer.qzeros, layer.g_idx)
    try:
        for variant in ((4, 12, 20) if forced else (0, 8, 16)):
            quant_cuda.gemv_set_variant(variant)
            first = gemv_gpu(layer, x, torch.float32)
            again = gemv_gpu(layer, x, torch.float32)
            assert rel_fro(first, want) <= REL_TOL, variant
            assert torch.equal(first, again), variant
            assert _head_is_zero(), variant
    finally:
        quant_cuda.gemv_set_variant(0)
    assert quant_cuda.device_status() == 0


@pytest.mark.parametrize("K,N", [(4096, 4096), (4096, 11008), (11008, 4096), (4224, 1024), (512, 4768)])
def test_gemv_one_row_forms_agree(K, N):
    """One-row products through every form: the warp-specialised int8-MMA kernel at one CTA per SM (the
    default), at two per SM (8), without L2 prefetch (64), and the fp16-MMA kernel of the 2..8-row products at
    one (16) and two (24) CTAs per SM.  Each within tolerance of the oracle; the int8 forms differ only in
    which warp adds which units, the fp16 forms round differently, so they agree to a few 1e-5."""
    layer = synth.make_layer(K, N, 128, False, seed=K + 3 * N)
    x = synth.make_acts(1, K, seed=17)
    want = orc.gemv_fp32(x, layer.qweight, layer.scales, layer.qzeros, layer.g_idx)
    got = {}
    try:
        for variant in (0, 8, 64, 16, 24):
            quant_cuda.gemv_set_variant(variant)
            got[variant] = gemv_gpu(layer, x, torch.float32)
            assert rel_fro(got[variant], want) <= REL_TOL, variant
    finally:
        quant_cuda.gemv_set_variant(0)
    for variant in (8, 64, 16, 24):
        assert rel_fro(got[variant], got[0]) <= 3e-4
    assert rel_fro(got[0], want) <= 1e-4                      # block fixed point of x: well inside the fp16 kernels' error
    assert quant_cuda.device_status() == 0


def test_decode_status_word_is_reported_and_cleared():
    """An expired bounded wait in a decode kernel is recorded in the last word of the workspace head.  Nothing
    here makes a wait expire on the GPU: the word is written from the host, then ``q4_gemv_status`` must return
    it, ``quant_cuda.device_status`` must report it and hand back a clean workspace, and the next product on
    that workspace must be right."""
    import ctypes
    layer = synth.make_layer(1024, 2048, 128, False, seed=5)
    x = synth.make_acts(2, 1024, seed=6)
    want = orc.gemv_fp32(x, layer.qweight, layer.scales, layer.qzeros, layer.g_idx)
    assert rel_fro(gemv_gpu(layer, x, torch.float32), want) <= REL_TOL
    assert quant_cuda.device_status() == 0
    dev = torch.device(DEV)
    ws = _lib.workspace_for(dev, torch.cuda.current_stream(dev).cuda_stream)
    word = ws[65536 - 4:65536].view(torch.int32)
    word.fill_(0xDEAD0001 - (1 << 32))
    ws[:8].view(torch.int32).fill_(3)                      # counters an aborted launch could leave behind
    v = ctypes.c_uint(0)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().q4_gemv_status(ws.data_ptr(), ws.numel(), ctypes.byref(v)), "status")
        assert v.value == 0xDEAD0001
        assert _lib.lib().q4_gemv_status(ws.data_ptr(), 100, ctypes.byref(v)) == -4
        assert quant_cuda.device_status() == 0xDEAD0001
        assert quant_cuda.device_status() == 0
    assert _head_is_zero()
    assert rel_fro(gemv_gpu(layer, x, torch.float32), want) <= REL_TOL


def test_workspace_counters_return_to_zero():
    layer = synth.make_layer(4096, 4096, 128, False, seed=3)
    gemv_gpu(layer, synth.make_acts(1, 4096), torch.float16)
    for ws in _lib._workspaces.values():
        assert int(ws[:65536].view(torch.int32).abs().sum()) == 0      # the counter head of the workspace


def test_recorded_layer_plan_serves_repeated_calls_and_expires():
    """``matmul4bit`` records a layer on its first per-token call and serves the next calls from the
    record: same results as the oracle for 1..8 rows, a new output tensor per call, the general path
    again for calls the record does not cover (other tensors, more rows than the switch threshold),
    and no record left once the layer's tensors are gone."""
    from alpaca_lora_4bit_b200 import matmul_utils_4bit as mm4b
    layer = synth.make_layer(1024, 2048, 128, False, seed=11)
    L = layer.to(DEV)
    before = len(quant_cuda._plans)
    outs = []
    for M in (1, 1, 3, 8, 1):
        x = synth.make_acts(M, 1024, seed=20 + M)
        y = mm4b.matmul4bit(x.to(DEV), L.qweight, L.scales, L.qzeros, L.g_idx, 128)
        assert y.shape == (M, 2048) and y.dtype == torch.float16
        assert rel_fro(y, orc.matmul4bit_ref(x, layer.qweight, layer.scales, layer.qzeros, layer.g_idx)) <= REL_TOL
        outs.append(y)
    assert len(quant_cuda._plans) == before + 1 and id(L.qweight) in quant_cuda._plans
    assert outs[0].data_ptr() != outs[1].data_ptr() and torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[4])
    # 12 rows are above the switch threshold: reconstruct + GEMM path, not the record
    x12 = synth.make_acts(12, 1024, seed=4)
    y12 = mm4b.matmul4bit(x12.to(DEV), L.qweight, L.scales, L.qzeros, L.g_idx, 128)
    assert rel_fro(y12, orc.matmul4bit_ref(x12, layer.qweight, layer.scales, layer.qzeros, layer.g_idx)) <= REL_TOL
    # other scales with the same qweight: the record does not apply, the result follows the new scales
    s2 = (L.scales * 2).contiguous()
    x = synth.make_acts(1, 1024, seed=21)
    y2 = mm4b.matmul4bit(x.to(DEV), L.qweight, s2, L.qzeros, L.g_idx, 128)
    assert rel_fro(y2, 2 * outs[0].float()) <= REL_TOL
    assert quant_cuda._plans[id(L.qweight)].scales is s2          # re-recorded for the tensors last seen
    # a CPU x is refused by the general path, not handed to the kernel
    with pytest.raises(RuntimeError):
        mm4b.matmul4bit(x, L.qweight, s2, L.qzeros, L.g_idx, 128)
    key = id(L.qweight)
    del L, y, y2, s2
    import gc
    gc.collect()
    assert key not in quant_cuda._plans
    torch.cuda.synchronize()
    assert quant_cuda.device_status() == 0
