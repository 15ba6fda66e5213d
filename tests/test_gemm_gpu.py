"""Parity of the fused dequant-GEMM kernels (forward x*W, backward dy*W^T) through the C ABI, and of
the autograd / module surface built on them."""
import pytest
import torch

from alpaca_lora_4bit_b200 import autograd_4bit as a4, matmul_utils_4bit as mm4b, models, quant_cuda, synth
from oracle import q4_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
REL_TOL = 2e-3          # relative Frobenius error allowed on matmul outputs (fp16 output rounding ~2e-4)


def rel_fro(got, want):
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).norm() / want.norm())


def run_gemm(layer, x, transpose, bias=None):
    L = layer.to(DEV)
    M = x.shape[0]
    out = torch.full((M + 16, layer.K if transpose else layer.N), -777.0, dtype=torch.float16, device=DEV)
    view = out[8:8 + M]
    quant_cuda.gemm(x.to(DEV), L.qweight, view, L.scales, L.qzeros, L.g_idx, transpose=transpose,
                    bias=None if bias is None else bias.to(DEV))
    torch.cuda.synchronize()
    assert quant_cuda.device_status() == 0
    assert bool((out[:8] == -777.0).all()) and bool((out[8 + M:] == -777.0).all())    # canary rows intact
    return view


@pytest.mark.parametrize("transpose", [False, True])
@pytest.mark.parametrize("M,K,N,g,act", [(128, 128, 128, 128, False), (1, 256, 128, 128, True), (17, 128, 384, 32, True),
                                         (200, 512, 384, 64, True), (129, 1024, 256, -1, False), (300, 4096, 512, 128, True)])
def test_gemm_vs_oracle(M, K, N, g, act, transpose):
    layer = synth.make_layer(K, N, g, act, seed=M + K)
    x = synth.make_acts(M, N if transpose else K, seed=M)
    want = orc.matmul4bit_ref(x, layer.qweight, layer.scales, layer.qzeros, layer.g_idx, transpose=transpose)
    assert rel_fro(run_gemm(layer, x, transpose), want) <= REL_TOL


@pytest.mark.parametrize("transpose", [False, True])
def test_gemm_selects_rows_of_w_bit_exactly(transpose):
    """One-hot activations copy rows (columns) of W through the tensor core: the in-kernel dequant
    must equal the reference reconstruct bit for bit."""
    layer = synth.make_layer(256, 384, 128, True, seed=5)
    w = orc.recons_v2(layer.qweight, layer.scales, layer.qzeros, layer.g_idx)
    inner = 384 if transpose else 256
    x = torch.zeros((inner, inner), dtype=torch.float16)
    x[torch.arange(inner), torch.arange(inner)] = 1.0
    got = run_gemm(layer, x, transpose).cpu()
    want = w.t().contiguous() if transpose else w
    assert torch.equal(got.view(torch.int16), want.contiguous().view(torch.int16))


@pytest.mark.parametrize("transpose", [False, True])
@pytest.mark.parametrize("act", [False, True])
@pytest.mark.parametrize("scale_case", ["usual", "subnormal", "large", "mixed"])
def test_gemm_dequant_is_bit_exact_over_the_scale_range(scale_case, act, transpose):
    """The same one-hot selection on the CTA-pair kernels (N a multiple of 256), for scales whose products are
    subnormal, for scales of 2 and more - where a task of one group takes the three-instruction form of rn(s q)
    instead of the fused multiply-add with -1024 s - and for layers that mix both in neighbouring columns; with
    the kept zero-term table and the sequential-group promise (no act-order) and with shared-memory tables."""
    layer = synth.make_layer(512, 512, 128, act, seed=7)
    g = torch.Generator().manual_seed(3)
    if scale_case == "subnormal":
        layer.scales.mul_(2.0 ** -9)
    elif scale_case == "large":
        layer.scales.mul_(300.0)
    elif scale_case == "mixed":
        layer.scales.mul_(torch.where(torch.rand(512, generator=g) < 0.3, 300.0, 1.0).half())
        layer.scales[1, 5] = 0.0
    w = orc.recons_v2(layer.qweight, layer.scales, layer.qzeros, layer.g_idx)
    x = torch.zeros((512, 512), dtype=torch.float16)
    x[torch.arange(512), torch.arange(512)] = 1.0
    want = w.t().contiguous() if transpose else w
    for variant in (2, 3):
        for cached in (True, False):
            quant_cuda.gemm_set_variant(variant)
            quant_cuda.cache_zero_terms = cached
            try:
                got = run_gemm(layer, x, transpose).cpu()
            finally:
                quant_cuda.gemm_set_variant(0)
                quant_cuda.cache_zero_terms = True
            assert torch.equal(got.view(torch.int16), want.contiguous().view(torch.int16)), (variant, cached)


def test_gemm_bias_forward():
    layer = synth.make_layer(512, 256, 128, False, seed=7)
    x = synth.make_acts(64, 512, seed=8)
    bias = torch.randn(256).half()
    want = orc.matmul4bit_ref(x, layer.qweight, layer.scales, layer.qzeros, layer.g_idx) + bias.float()
    assert rel_fro(run_gemm(layer, x, False, bias=bias), want) <= REL_TOL


@pytest.mark.parametrize("K,N", [(5120, 5120), (5120, 13824), (13824, 5120)])
def test_gemm_llama13b_shapes_act_order(K, N):
    """C2 sizes (M=2048, act-order, g128): checked against fp32 matmul of the bit-exact reconstruct on the GPU."""
    layer = synth.make_layer(K, N, 128, True, seed=K // 128 + N)
    L = layer.to(DEV)
    w = torch.empty((K, N), dtype=torch.float16, device=DEV)
    quant_cuda.vecquant4recons_v2(L.qweight, w, L.scales, L.qzeros, L.g_idx)
    torch.backends.cuda.matmul.allow_tf32 = False
    for transpose in (False, True):
        x = synth.make_acts(2048, N if transpose else K, seed=3).to(DEV)
        want = x.float() @ (w.float().t() if transpose else w.float())
        got = run_gemm(layer, x.cpu(), transpose)
        assert rel_fro(got, want) <= REL_TOL


def test_backward_is_transpose_of_forward():
    """<dy, x W> = <dy W^T, x> for random x, dy at a full-size layer."""
    layer = synth.make_layer(4096, 11008, 128, False, seed=11)
    x = synth.make_acts(256, 4096, seed=12)
    dy = synth.make_acts(256, 11008, seed=13)
    y = run_gemm(layer, x, False).double()
    dx = run_gemm(layer, dy, True).double()
    lhs = float((dy.double().to(DEV) * y).sum())
    rhs = float((dx * x.double().to(DEV)).sum())
    assert abs(lhs - rhs) <= 2e-3 * max(abs(lhs), abs(rhs))


def _module(K, N, g, act, seed, cls=a4.Autograd4bitQuantLinear, **kw):
    layer = synth.make_layer(K, N, g, act, seed)
    m = cls(K, N, groupsize=g, **kw) if cls is a4.Autograd4bitQuantLinear else cls("default", K, N, groupsize=g, **kw)
    m.qweight, m.qzeros, m.scales, m.g_idx = layer.qweight, layer.qzeros, layer.scales, layer.g_idx
    m.bias = torch.zeros(N, dtype=torch.float16)
    return m.to(DEV), layer


@pytest.mark.parametrize("fused", [True, False])
def test_autograd_module_forward_backward(fused):
    m, layer = _module(1024, 512, 128, True, 21)
    w = orc.recons_v2(layer.qweight, layer.scales, layer.qzeros, layer.g_idx).float()
    x = synth.make_acts(2 * 96, 1024, 22).reshape(2, 96, 1024).to(DEV).requires_grad_(True)
    mm4b.fused_gemm = fused
    try:
        y = m(x)
        dy = torch.randn_like(y)
        y.backward(dy)
    finally:
        mm4b.fused_gemm = True
    assert y.shape == (2, 96, 512) and y.dtype == torch.float16
    assert rel_fro(y.reshape(-1, 512), x.detach().reshape(-1, 1024).float().cpu() @ w) <= REL_TOL
    assert rel_fro(x.grad.reshape(-1, 1024), dy.reshape(-1, 512).float().cpu() @ w.t()) <= REL_TOL


def test_module_routes_by_rows_and_grad_mode():
    m, layer = _module(512, 256, 128, False, 31)
    want = lambda x: orc.matmul4bit_ref(x, layer.qweight, layer.scales, layer.qzeros, layer.g_idx)
    with torch.no_grad():
        for rows in (1, 8, 9, 40):                              # decode kernel up to auto_switch_thd rows, fused GEMM above
            x = synth.make_acts(rows, 512, rows)
            assert rel_fro(m(x.to(DEV)), want(x)) <= REL_TOL


@pytest.mark.parametrize("r", [8, 16, 40])
@pytest.mark.parametrize("transpose", [False, True])
def test_gemm_fused_lora_term(r, transpose):
    """C2: the LoRA update fused into the GEMM as an extra pipeline stage (r=16, alpha=32 -> scale 2)."""
    K, N, M = 1024, 640 if not transpose else 512, 300
    layer = synth.make_layer(K, N, 128, True, seed=r)
    A, B = synth.make_lora(K, N, r, seed=r + 1)
    inner = N if transpose else K
    x = synth.make_acts(M, inner, seed=r + 2)
    w = orc.recons_v2(layer.qweight, layer.scales, layer.qzeros, layer.g_idx).float()
    if transpose:                                           # dx = dy W^T + 2 (dy B) A
        u = ((x.float() @ B.float()) * 2.0).half()
        want = x.float() @ w.t() + u.float() @ A.float()
        lw = A
    else:                                                   # y = x W + 2 (x A^T) B^T
        u = ((x.float() @ A.float().t()) * 2.0).half()
        want = x.float() @ w + u.float() @ B.float().t()
        lw = B
    L = layer.to(DEV)
    out = torch.empty((M, K if transpose else N), dtype=torch.float16, device=DEV)
    u_pad = torch.nn.functional.pad(u, (0, 64 - r)).to(DEV)
    quant_cuda.gemm(x.to(DEV), L.qweight, out, L.scales, L.qzeros, L.g_idx, transpose=transpose, lora_u=u_pad,
                    lora_w=lw.contiguous().to(DEV))
    torch.cuda.synchronize()
    assert quant_cuda.device_status() == 0
    assert rel_fro(out, want) <= REL_TOL


@pytest.fixture
def gemm_variant():
    yield quant_cuda.gemm_set_variant
    quant_cuda.gemm_set_variant(0)


@pytest.mark.parametrize("transpose", [False, True])
@pytest.mark.parametrize("M,K,N,g,act", [(700, 1024, 768, 128, True), (256, 256, 256, 64, False), (5, 512, 1280, 128, True)])
def test_both_gemm_kernels_against_oracle(gemm_variant, M, K, N, g, act, transpose):
    """The single-CTA kernel and the CTA-pair kernel (256- and 512-row tiles) on the same inputs."""
    layer = synth.make_layer(K, N, g, act, seed=M + N)
    x = synth.make_acts(M, N if transpose else K, seed=M + 1)
    want = orc.matmul4bit_ref(x, layer.qweight, layer.scales, layer.qzeros, layer.g_idx, transpose=transpose)
    outs = []
    for variant in (1, 2, 3):
        gemm_variant(variant)
        outs.append(run_gemm(layer, x, transpose).clone())
        assert rel_fro(outs[-1], want) <= REL_TOL
    assert rel_fro(outs[0], outs[1]) <= 5e-4               # same products, different accumulation grouping at most
    assert rel_fro(outs[0], outs[2]) <= 5e-4


@pytest.mark.parametrize("variant", [2, 3])
@pytest.mark.parametrize("transpose", [False, True])
def test_pair_kernel_many_tiles_per_pair(gemm_variant, transpose, variant):
    """More than five 256 x 256 tiles per CTA pair: both accumulators and every pipeline stage are
    reused several times (the barrier phases wrap), with the low-rank stage making the stage count odd."""
    K, N, M, r = (256, 12288, 2048, 16) if not transpose else (12288, 256, 2048, 16)
    layer = synth.make_layer(K, N, 128, True, seed=11)
    A, B = synth.make_lora(K, N, r, seed=12)
    x = synth.make_acts(M, N if transpose else K, seed=13)
    w = orc.recons_v2(layer.qweight, layer.scales, layer.qzeros, layer.g_idx).float()
    if transpose:
        u = ((x.float() @ B.float()) * 2.0).half()
        want, lw = x.float() @ w.t() + u.float() @ A.float(), A
    else:
        u = ((x.float() @ A.float().t()) * 2.0).half()
        want, lw = x.float() @ w + u.float() @ B.float().t(), B
    L = layer.to(DEV)
    gemm_variant(variant)
    out = torch.empty((M, K if transpose else N), dtype=torch.float16, device=DEV)
    quant_cuda.gemm(x.to(DEV), L.qweight, out, L.scales, L.qzeros, L.g_idx, transpose=transpose,
                    lora_u=torch.nn.functional.pad(u, (0, 64 - r)).to(DEV), lora_w=lw.contiguous().to(DEV))
    torch.cuda.synchronize()
    assert quant_cuda.device_status() == 0
    assert rel_fro(out, want) <= REL_TOL


@pytest.mark.parametrize("variant", [2, 3])
@pytest.mark.parametrize("transpose", [False, True])
@pytest.mark.parametrize("act", [False, True])
def test_tail_tiles_split_along_the_contraction(gemm_variant, transpose, act, variant):
    """20 output tiles on 74 SM pairs: with a workspace every tile is cut into slices whose partial
    sums are added in a fixed order (bit-identical from call to call, workspace left clean); without
    one the tiles are computed whole.  Both against the oracle, bias and low-rank term included."""
    from alpaca_lora_4bit_b200 import _lib
    K, N, M, r = (2048, 1280, 1024, 16) if not transpose else (1280, 2048, 1024, 16)
    layer = synth.make_layer(K, N, 128, act, seed=21)
    A, B = synth.make_lora(K, N, r, seed=22)
    x = synth.make_acts(M, N if transpose else K, seed=23)
    bias = None if transpose else torch.randn(N).half()
    w = orc.recons_v2(layer.qweight, layer.scales, layer.qzeros, layer.g_idx).float()
    if transpose:
        u = ((x.float() @ B.float()) * 2.0).half()
        want, lw = x.float() @ w.t() + u.float() @ A.float(), A
    else:
        u = ((x.float() @ A.float().t()) * 2.0).half()
        want, lw = x.float() @ w + u.float() @ B.float().t() + bias.float(), B
    L = layer.to(DEV)
    xd, ud, lwd = x.to(DEV), torch.nn.functional.pad(u, (0, 64 - r)).to(DEV), lw.contiguous().to(DEV)
    bd = None if bias is None else bias.to(DEV)
    gemm_variant(variant)
    outs = []
    for _ in range(2):
        out = torch.empty((M, K if transpose else N), dtype=torch.float16, device=DEV)
        quant_cuda.gemm(xd, L.qweight, out, L.scales, L.qzeros, L.g_idx, transpose=transpose, bias=bd, lora_u=ud, lora_w=lwd)
        torch.cuda.synchronize()
        outs.append(out)
    assert quant_cuda.device_status() == 0
    assert rel_fro(outs[0], want) <= REL_TOL
    assert torch.equal(outs[0], outs[1])
    ws = _lib.gemm_workspace_for(torch.device(DEV), torch.cuda.current_stream().cuda_stream, 0)
    assert int(ws[:65536].view(torch.int32).abs().max()) == 0          # arrival counters back at zero
    # the same call without a workspace
    lib = _lib.lib()
    whole = torch.empty_like(outs[0])
    G, st = L.scales.shape[0], torch.cuda.current_stream().cuda_stream
    if transpose:
        rc = lib.q4_gemm_bwd(xd.data_ptr(), L.qweight.data_ptr(), whole.data_ptr(), L.scales.data_ptr(), L.qzeros.data_ptr(),
                             L.g_idx.data_ptr(), ud.data_ptr(), lwd.data_ptr(), r, M, K, N, G, None, 0, st)
    else:
        rc = lib.q4_gemm_fwd(xd.data_ptr(), L.qweight.data_ptr(), whole.data_ptr(), L.scales.data_ptr(), L.qzeros.data_ptr(),
                             L.g_idx.data_ptr(), bd.data_ptr(), ud.data_ptr(), lwd.data_ptr(), r, M, K, N, G, None, 0, st)
    assert rc == 0
    torch.cuda.synchronize()
    assert rel_fro(whole, want) <= REL_TOL
    assert rel_fro(whole, outs[0]) <= 5e-4


@pytest.mark.parametrize("variant", [1, 2, 3])
@pytest.mark.parametrize("M,r", [(1, 64), (513, 1), (2000, 64)])
def test_gemm_edge_rows_and_ranks(gemm_variant, variant, M, r):
    """One row, one row past a tile boundary and a ragged large M; rank 1 and the largest rank the
    low-rank stage takes (64); forward with bias and backward, on every kernel."""
    K, N = 768, 512
    layer = synth.make_layer(K, N, 128, True, seed=31)
    A, B = synth.make_lora(K, N, r, seed=32)
    w = orc.recons_v2(layer.qweight, layer.scales, layer.qzeros, layer.g_idx).float()
    L = layer.to(DEV)
    gemm_variant(variant)
    for transpose in (False, True):
        x = synth.make_acts(M, N if transpose else K, seed=33 + transpose)
        bias = None if transpose else torch.randn(N).half()
        if transpose:
            u = ((x.float() @ B.float()) * 0.5).half()
            want, lw = x.float() @ w.t() + u.float() @ A.float(), A
        else:
            u = ((x.float() @ A.float().t()) * 0.5).half()
            want, lw = x.float() @ w + u.float() @ B.float().t() + bias.float(), B
        out = torch.full((M + 2, K if transpose else N), 7.0, dtype=torch.float16, device=DEV)
        quant_cuda.gemm(x.to(DEV), L.qweight, out[1:M + 1], L.scales, L.qzeros, L.g_idx, transpose=transpose,
                        bias=None if bias is None else bias.to(DEV),
                        lora_u=torch.nn.functional.pad(u, (0, 64 - r)).to(DEV), lora_w=lw.contiguous().to(DEV))
        torch.cuda.synchronize()
        assert quant_cuda.device_status() == 0
        assert bool((out[0] == 7.0).all()) and bool((out[M + 1] == 7.0).all())         # rows around the view untouched
        assert rel_fro(out[1:M + 1], want) <= REL_TOL


def test_pair_kernel_rejects_shapes_it_cannot_serve(gemm_variant):
    layer = synth.make_layer(256, 384, 128, False, seed=3).to(DEV)
    x = synth.make_acts(16, 256, seed=4).to(DEV)
    out = torch.empty((16, 384), dtype=torch.float16, device=DEV)
    gemm_variant(2)
    with pytest.raises(RuntimeError):
        quant_cuda.gemm(x, layer.qweight, out, layer.scales, layer.qzeros, layer.g_idx)


@pytest.mark.parametrize("fused", [True, False])
def test_linear4bitlt_lora_training_step(fused):
    models.fused_lora = fused
    m, layer = _module(512, 256, 128, True, 41, cls=models.Linear4bitLt, r=8, lora_alpha=16, lora_dropout=0.0)
    A, B = synth.make_lora(512, 256, 8, seed=42, dtype=torch.float32)
    m.lora_A["default"].weight.data.copy_(A)
    m.lora_B["default"].weight.data.copy_(B)
    x = synth.make_acts(160, 512, 43).to(DEV).requires_grad_(True)
    try:
        y = m(x)
        dy = torch.randn_like(y)
        y.backward(dy)
    finally:
        models.fused_lora = True
    w = orc.recons_v2(layer.qweight, layer.scales, layer.qzeros, layer.g_idx).float()
    xc, dyc = x.detach().cpu(), dy.cpu()
    assert rel_fro(y, xc.float() @ w + orc.lora_forward(xc, A, B, 2.0)) <= REL_TOL
    dx_l, dA, dB = orc.lora_backward(xc, dyc, A, B, 2.0)
    assert rel_fro(x.grad, dyc.float() @ w.t() + dx_l) <= REL_TOL
    assert rel_fro(m.lora_A["default"].weight.grad, dA) <= 5e-3
    assert rel_fro(m.lora_B["default"].weight.grad, dB) <= 5e-3


@pytest.mark.parametrize("M,K,I,act", [(300, 512, 256, False), (1024, 4096, 11008, False), (2048, 1024, 1408, True), (64, 256, 128, False), (520, 5120, 13824, False)])
def test_gate_up_product_with_swiglu_in_the_epilogue(M, K, I, act):
    """q4_gemm_fwd_swiglu on a fused [gate | up] layer against q4_gemm_fwd followed by the element-wise SwiGLU
    kernel (the same roundings: equal up to the order in which shared tiles add their partial sums) and against
    silu(gate) * up of the oracle's products; with and without bias, both tile heights."""
    from alpaca_lora_4bit_b200 import fused_ops
    layer = synth.make_layer(K, 2 * I, 128, act, seed=K + I).to(DEV)
    x = synth.make_acts(M, K, seed=M).to(DEV)
    bias = (torch.randn(2 * I, generator=torch.Generator().manual_seed(1)) * 0.1).half().to(DEV)
    w = orc.recons_v2(layer.qweight.cpu(), layer.scales.cpu(), layer.qzeros.cpu(), layer.g_idx.cpu()).to(DEV).float()
    for b in (None, bias):
        full = torch.empty(M, 2 * I, dtype=torch.float16, device=DEV)
        quant_cuda.gemm(x, layer.qweight, full, layer.scales, layer.qzeros, layer.g_idx, bias=b)
        want = fused_ops.swiglu(full[:, :I], full[:, I:])
        exact = x.float() @ w + (0 if b is None else b.float())
        exact = torch.nn.functional.silu(exact[:, :I]) * exact[:, I:]
        for variant in (0, 2, 3):
            quant_cuda.gemm_set_variant(variant)
            try:
                got = torch.full((M, I), 9.0, dtype=torch.float16, device=DEV)
                quant_cuda.gemm_swiglu(x, layer.qweight, got, layer.scales, layer.qzeros, layer.g_idx, bias=b)
            finally:
                quant_cuda.gemm_set_variant(0)
            assert rel_fro(got, want) <= 1e-3, (variant, rel_fro(got, want))
            assert rel_fro(got, exact) <= 3e-3
            assert float((got == want).float().mean()) >= 0.98              # the same roundings: almost every element equal
            if not act:                        # sequential groups: kept table and promise by default; same bits without either
                for cached, promise in ((False, False), (True, False)):
                    quant_cuda.gemm_set_variant(variant)
                    quant_cuda.cache_zero_terms, quant_cuda.promise_sequential_groups = cached, promise
                    try:
                        other = torch.empty_like(got)
                        quant_cuda.gemm_swiglu(x, layer.qweight, other, layer.scales, layer.qzeros, layer.g_idx, bias=b)
                    finally:
                        quant_cuda.gemm_set_variant(0)
                        quant_cuda.cache_zero_terms, quant_cuda.promise_sequential_groups = True, True
                    if variant:                # a fixed tile height: the same schedule, so the same sums
                        assert torch.equal(other, got), (variant, cached, promise)
                    else:
                        assert rel_fro(other, got) <= 1e-3
    assert quant_cuda.device_status() == 0


def test_backward_with_cached_zero_terms_is_the_same_product():
    """quant_cuda.gemm keeps rn(s (z + 1)) [G, N] of a layer after its first backward (q4_zero_term_table,
    q4_gemm_bwd_table) instead of deriving it into the workspace ahead of every call: same bits either way, one
    table per layer, dropped with the layer's tensors."""
    import gc
    layer = synth.make_layer(1024, 768, 128, True, seed=5).to(DEV)
    dy = synth.make_acts(300, 768, seed=6).to(DEV)
    outs = []
    for cached in (False, True, True):
        quant_cuda.cache_zero_terms = cached
        try:
            dx = torch.empty(300, 1024, dtype=torch.float16, device=DEV)
            quant_cuda.gemm(dy, layer.qweight, dx, layer.scales, layer.qzeros, layer.g_idx, transpose=True)
            outs.append(dx)
        finally:
            quant_cuda.cache_zero_terms = True
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])
    key = id(layer.qzeros)
    assert key in quant_cuda._zero_term_tables
    table = quant_cuda._zero_term_tables[key][0]
    z1 = (((layer.qzeros.cpu().view(-1, 96, 1) >> (4 * torch.arange(8).view(1, 1, 8))) & 0xF) + 1).reshape(8, 768).half()
    assert torch.equal(table.cpu(), layer.scales.cpu() * z1)              # rn(s * (z + 1)), as the reconstruct rounds it
    del layer, table
    gc.collect()
    assert key not in quant_cuda._zero_term_tables


@pytest.mark.parametrize("M,K,N,g", [(300, 1024, 768, 128), (129, 1024, 256, -1), (520, 2048, 512, 32), (70, 11008, 256, 128),
                                     (40, 11008, 256, -1), (260, 1536, 512, 8)])
def test_forward_with_sequential_groups_promised_is_the_same_product(M, K, N, g):
    """Layers without act-order: quant_cuda.gemm hands the forward the kept zero-term table and the word that
    group = row / groupsize (``sequential_groupsize`` of q4_gemm_fwd_residual), and the kernel fetches scales and
    zero terms with a task's packed words instead of building tables per tile.  Same bits as the kernel with its
    shared-memory tables and as the kept table read through g_idx (no promise; q4_gemm_fwd_table), for group sizes
    down to the 8 rows of a task, one group over all rows (a power of two, or 11008 rows where no shift exists and
    the promise is dropped by the library) and in the 512-row form."""
    from alpaca_lora_4bit_b200 import _lib
    layer = synth.make_layer(K, N, g, False, seed=K + N).to(DEV)
    x = synth.make_acts(M, K, seed=M).to(DEV)
    outs = {}
    tables_fit = layer.scales.shape[0] <= 128      # 192 groups of tables leave the CTA-pair kernel no stage: the kept table is what admits it
    for variant in (2, 3):
        try:
            for mode, cached, promise in (("smem", False, False), ("table", True, False), ("promised", True, True)):
                quant_cuda.gemm_set_variant(variant if (cached or tables_fit) else 0)
                quant_cuda.cache_zero_terms, quant_cuda.promise_sequential_groups = cached, promise
                y = torch.empty(M, N, dtype=torch.float16, device=DEV)
                quant_cuda.gemm(x, layer.qweight, y, layer.scales, layer.qzeros, layer.g_idx)
                outs[variant, mode] = y
            table = quant_cuda._zero_term_tables[id(layer.qzeros)][0]
            y = torch.empty(M, N, dtype=torch.float16, device=DEV)
            st = torch.cuda.current_stream().cuda_stream
            ws = _lib.gemm_workspace_for(x.device, st, int(_lib.lib().q4_gemm_workspace_bytes(K, N, layer.scales.shape[0])))
            rc = _lib.lib().q4_gemm_fwd_table(x.data_ptr(), layer.qweight.data_ptr(), y.data_ptr(), layer.scales.data_ptr(),
                                              layer.qzeros.data_ptr(), table.data_ptr(), layer.g_idx.data_ptr(), None, None, None, 0,
                                              M, K, N, layer.scales.shape[0], ws.data_ptr(), ws.numel(), st)
            assert rc == 0
            outs[variant, "abi"] = y
        finally:
            quant_cuda.gemm_set_variant(0)
            quant_cuda.cache_zero_terms, quant_cuda.promise_sequential_groups = True, True
        for mode in ("table", "promised", "abi"):
            assert torch.equal(outs[variant, mode], outs[variant, "smem"]), (variant, mode)
    assert quant_cuda.device_status() == 0
    host = layer.to("cpu")
    want = orc.matmul4bit_ref(x.cpu(), host.qweight, host.scales, host.qzeros, host.g_idx)
    assert rel_fro(outs[2, "promised"], want) <= REL_TOL


@pytest.mark.parametrize("M,K,N,g", [(128, 128, 256, 128), (300, 1024, 768, 128), (256, 512, 512, 64), (77, 2048, 256, -1),
                                     (513, 1024, 512, 128), (1000, 4096, 1024, 128)])
def test_forward_with_weights_in_tensor_memory(M, K, N, g):
    """q4_gemm3_kernel (variant 4: the dequantised weights are the A operand in TMEM, a thread per output column):
    within tolerance of the oracle, and bit-identical to the CTA-pair kernel where that takes whole tiles (the same
    fp16 operands, the same order of accumulation along K), plain and with bias, skip-path add and low-rank term;
    rows that are not a multiple of 128, groups from the 64 rows of a stage up to all of K."""
    layer = synth.make_layer(K, N, g, False, seed=K + N).to(DEV)
    x = synth.make_acts(M, K, seed=M).to(DEV)
    gen = torch.Generator(device=DEV).manual_seed(M)
    bias = (torch.randn(N, generator=gen, device=DEV) * 0.1).half()
    res = torch.randn(M, N, generator=gen, device=DEV).half()
    r = 8
    u = torch.zeros(M, 64, device=DEV, dtype=torch.float16)
    u[:, :r] = torch.randn(M, r, generator=gen, device=DEV).half()
    lw = (torch.randn(N, r, generator=gen, device=DEV) * 0.1).half()

    def run(variant, **kw):
        quant_cuda.gemm_set_variant(variant)
        try:
            y = torch.full((M + 2, N), -9.0, dtype=torch.float16, device=DEV)
            quant_cuda.gemm(x, layer.qweight, y[1:M + 1], layer.scales, layer.qzeros, layer.g_idx, **kw)
        finally:
            quant_cuda.gemm_set_variant(0)
        assert bool((y[0] == -9.0).all()) and bool((y[M + 1] == -9.0).all())        # rows around the output untouched
        return y[1:M + 1]

    def same(a, b):                  # long contractions on few tiles: the pair kernel deals K out to several pairs and adds in another order
        return torch.equal(a, b) if K <= 2048 else rel_fro(a, b) <= 1e-3

    plain = run(4)
    assert same(plain, run(2))
    full = run(4, bias=bias, residual=res, lora_u=u, lora_w=lw)
    assert same(full, run(2, bias=bias, residual=res, lora_u=u, lora_w=lw))
    assert torch.equal(run(4, residual=res), plain + res)
    host = layer.to("cpu")
    want = orc.matmul4bit_ref(x.cpu(), host.qweight, host.scales, host.qzeros, host.g_idx)
    assert rel_fro(plain, want) <= REL_TOL
    assert quant_cuda.device_status() == 0


def test_tensor_memory_kernel_is_chosen_and_refused_where_it_should_be():
    """Default choice: the forward of a sequential layer whose 256 x 256 tiles fit one round goes to the
    weights-in-TMEM kernel even where the pair kernel would have taken 512-row tiles (the activation boxes must
    then be those of 128 rows: 1024 x 11008 x 4096 is the down projection of LLaMA-7B in the finetune step) -
    same product as without it; act-order layers, groups below 64 rows and the backward are refused by variant 4."""
    layer = synth.make_layer(11008, 4096, 128, False, seed=2).to(DEV)
    x = synth.make_acts(1024, 11008, seed=3).to(DEV)
    outs = []
    for variant in (5, 0, 4):
        quant_cuda.gemm_set_variant(variant)
        try:
            y = torch.empty(1024, 4096, dtype=torch.float16, device=DEV)
            quant_cuda.gemm(x, layer.qweight, y, layer.scales, layer.qzeros, layer.g_idx)
            outs.append(y)
        finally:
            quant_cuda.gemm_set_variant(0)
    assert torch.equal(outs[1], outs[2])                    # the default took the same kernel as variant 4
    assert rel_fro(outs[1], outs[0]) <= 1e-3                # the pair kernel adds the halves of K in another order
    assert quant_cuda.device_status() == 0
    act = synth.make_layer(512, 512, 128, True, seed=4).to(DEV)
    small = synth.make_layer(512, 512, 32, False, seed=5).to(DEV)
    seq = synth.make_layer(512, 512, 128, False, seed=6).to(DEV)
    xa = synth.make_acts(64, 512, seed=7).to(DEV)
    quant_cuda.gemm_set_variant(4)
    try:
        for bad, tr in ((act, False), (small, False), (seq, True)):
            with pytest.raises(RuntimeError):
                quant_cuda.gemm(xa, bad.qweight, torch.empty(64, 512, dtype=torch.float16, device=DEV), bad.scales, bad.qzeros, bad.g_idx,
                                transpose=tr)
    finally:
        quant_cuda.gemm_set_variant(0)


@pytest.mark.parametrize("M,K,N", [(1024, 4096, 11008), (700, 2048, 20480), (64, 4096, 1024), (40, 11008, 4096), (300, 8192, 2048)])
def test_tensor_memory_kernel_with_runs_dealt_across_pairs(M, K, N):
    """More 256 x 256 tiles than CTA pairs and a last round that would leave most pairs idle: the weights-in-TMEM
    kernel deals tiles x stages as one sequence (stream-K), shared tiles meet in the workspace.  Same product as the
    pair kernel (which adds K in another order: tolerance), plain and with bias, skip-path add and a rank-16 term
    (the low-rank stage goes with the run that reaches the end of a tile); twice in a row (the counters are left
    zero); the workspace status stays clean.  The short-prompt cases have few tiles and a long contraction: every
    tile is cut between several whole pairs."""
    layer = synth.make_layer(K, N, 128, False, seed=K + N).to(DEV)
    x = synth.make_acts(M, K, seed=M).to(DEV)
    gen = torch.Generator(device=DEV).manual_seed(M)
    bias = (torch.randn(N, generator=gen, device=DEV) * 0.1).half()
    res = torch.randn(M, N, generator=gen, device=DEV).half()
    r = 16
    u = torch.zeros(M, 64, device=DEV, dtype=torch.float16)
    u[:, :r] = torch.randn(M, r, generator=gen, device=DEV).half()
    lw = (torch.randn(N, r, generator=gen, device=DEV) * 0.1).half()

    def run(variant, **kw):
        quant_cuda.gemm_set_variant(variant)
        try:
            y = torch.empty(M, N, dtype=torch.float16, device=DEV)
            quant_cuda.gemm(x, layer.qweight, y, layer.scales, layer.qzeros, layer.g_idx, **kw)
        finally:
            quant_cuda.gemm_set_variant(0)
        return y

    for kw in ({}, dict(bias=bias, residual=res, lora_u=u, lora_w=lw)):
        a, b, c = run(4, **kw), run(4, **kw), run(5, **kw)
        assert torch.equal(a, b)                                   # deterministic: partial sums are added in pair order
        assert rel_fro(a, c) <= 1e-3
    assert quant_cuda.device_status() == 0
