"""Host-side logic of the operator surface on the CPU, kernels replaced by the oracle
(tests/fake_backend.py): routing, autograd wiring, LoRA layer, module surgery, state-dict names."""
import math

import pytest
import torch
import torch.nn as nn

from alpaca_lora_4bit_b200 import autograd_4bit as a4, matmul_utils_4bit as mm4b, models, synth
from alpaca_lora_4bit_b200 import model_attn_mlp_patch as patch
from oracle import q4_oracle as orc
from tests import fake_backend


def make_module(K, N, g=128, act=False, seed=0, cls=a4.Autograd4bitQuantLinear, **kw):
    layer = synth.make_layer(K, N, g, act, seed)
    m = cls(K, N, groupsize=g, **kw) if cls is a4.Autograd4bitQuantLinear else cls("default", K, N, groupsize=g, **kw)
    m.qweight, m.qzeros, m.scales, m.g_idx = layer.qweight, layer.qzeros, layer.scales, layer.g_idx
    m.bias = torch.zeros(N, dtype=torch.float16)
    return m, layer


def test_state_dict_names_and_shapes():
    m = a4.Autograd4bitQuantLinear(256, 128, groupsize=64)
    sd = m.state_dict()
    assert set(sd) == {"qzeros", "scales", "g_idx", "bias", "qweight"}
    assert sd["qweight"].shape == (32, 128) and sd["qweight"].dtype == torch.int32
    assert sd["qzeros"].shape == (4, 16) and sd["scales"].shape == (4, 128) and sd["g_idx"].shape == (256,)
    assert torch.equal(sd["g_idx"], (torch.arange(256) // 64).int())
    v1 = a4.Autograd4bitQuantLinear(256, 128, is_v1_model=True)
    assert set(v1.state_dict()) == {"zeros", "scales", "bias", "qweight"} and v1.g_idx is None
    assert v1.groupsize == 256 and v1.zeros.shape == (128, 1)
    two = a4.Autograd4bitQuantLinear(256, 128, groupsize=64, bits=2)
    assert two.qweight.shape == (16, 128) and two.qzeros.shape == (4, 8) and two.maxq == 3


def test_dispatch_threshold_and_formats():
    layer = synth.make_layer(256, 64, 64, False, 1)
    x = synth.make_acts(20, 256, 2)
    want = orc.matmul4bit_ref(x, layer.qweight, layer.scales, layer.qzeros, layer.g_idx)
    calls = []
    with fake_backend.installed():
        real_gemv, real_rec = fake_backend.gemv, fake_backend.vecquant4recons_v2
        try:
            fake_backend.gemv = lambda *a, **k: (calls.append("gemv"), real_gemv(*a, **k))[1]
            fake_backend.vecquant4recons_v2 = lambda *a, **k: (calls.append("recons"), real_rec(*a, **k))[1]
            y_small = mm4b.matmul4bit(x[:8], layer.qweight, layer.scales, layer.qzeros, layer.g_idx, 64)
            y_big = mm4b.matmul4bit(x, layer.qweight, layer.scales, layer.qzeros, layer.g_idx, 64)
        finally:
            fake_backend.gemv, fake_backend.vecquant4recons_v2 = real_gemv, real_rec
    assert calls == ["gemv", "recons"]                     # 8 rows: decode kernel, 20 rows: large-M path
    assert torch.allclose(y_small.float(), want[:8], atol=2e-2, rtol=1e-2)
    assert torch.allclose(y_big.float(), want, atol=2e-2, rtol=1e-2)
    assert y_big.shape == (20, 64) and y_small.dtype == torch.float16


def test_empty_inputs_launch_nothing():
    """Zero rows in, zero rows out (as ``torch.matmul`` on the reference's dense buffer gives), without a kernel call."""
    layer = synth.make_layer(256, 64, 64, False, 1)
    calls = []
    with fake_backend.installed():
        real_gemv, real_gemm = fake_backend.gemv, fake_backend.gemm
        try:
            fake_backend.gemv = lambda *a, **k: calls.append("gemv")
            fake_backend.gemm = lambda *a, **k: calls.append("gemm")
            y = mm4b.matmul4bit(torch.empty((0, 256), dtype=torch.float16), layer.qweight, layer.scales, layer.qzeros, layer.g_idx, 64)
            y3 = mm4b.matmul4bit(torch.empty((2, 0, 256), dtype=torch.float16), layer.qweight, layer.scales, layer.qzeros, layer.g_idx, 64)
            dx = mm4b._matmul4bit_v2_recons(torch.empty((0, 64), dtype=torch.float16), layer.qweight, layer.scales, layer.qzeros,
                                            layer.g_idx, transpose=True)
        finally:
            fake_backend.gemv, fake_backend.gemm = real_gemv, real_gemm
    assert calls == []
    assert y.shape == (0, 64) and y3.shape == (2, 0, 64) and dx.shape == (0, 256)


def test_autograd_forward_backward_matches_dense():
    m, layer = make_module(256, 128, 64, act=True, seed=3)
    w = orc.recons_v2(layer.qweight, layer.scales, layer.qzeros, layer.g_idx).float()
    x2 = synth.make_acts(24, 256, 4).requires_grad_(True)
    with fake_backend.installed():
        y = m(x2)
        dy = torch.randn_like(y)
        y.backward(dy)
    ref_y = x2.detach().float() @ w
    ref_dx = dy.float() @ w.t()
    assert torch.allclose(y.float(), ref_y, atol=3e-2, rtol=1e-2)
    assert torch.allclose(x2.grad.float(), ref_dx, atol=3e-2, rtol=1e-2)
    assert all(not t.requires_grad for t in (m.qweight, m.scales, m.qzeros, m.g_idx))


def test_backward_without_input_grad_returns_none():
    m, _ = make_module(128, 64, 64, seed=5)
    m2 = nn.Linear(64, 4).half()
    x = synth.make_acts(12, 128, 6)                         # needs no grad
    with fake_backend.installed():
        out = m2(m(x)).float().sum()
        out.backward()                                      # the reference raises here (unbound `grad`)
    assert m2.weight.grad is not None


def test_no_grad_path_and_bias():
    m, layer = make_module(128, 64, 64, seed=7)
    m.bias = torch.randn(64).half()
    x = synth.make_acts(4, 128, 8)
    want = orc.matmul4bit_ref(x, layer.qweight, layer.scales, layer.qzeros, layer.g_idx) + m.bias.float()
    with fake_backend.installed(), torch.no_grad():
        y = m(x)
    assert torch.allclose(y.float(), want, atol=2e-2, rtol=1e-2)
    m.disable_bias = True
    with fake_backend.installed(), torch.no_grad():
        y2 = m(x)
    assert torch.allclose(y2.float(), want - m.bias.float(), atol=2e-2, rtol=1e-2)


def test_make_quant_and_model_to_half_float():
    net = nn.Sequential()
    net.add_module("a", nn.Linear(128, 64))
    net.add_module("blk", nn.Sequential(nn.Linear(64, 64), nn.ReLU()))
    net.add_module("lm_head", nn.Linear(64, 32))
    layers = a4.find_layers(net)
    assert set(layers) == {"a", "blk.0", "lm_head"}
    del layers["lm_head"]
    a4.make_quant_for_4bit_autograd(net, layers, groupsize=64)
    assert isinstance(net.a, a4.Autograd4bitQuantLinear) and isinstance(net.blk[0], a4.Autograd4bitQuantLinear)
    assert isinstance(net.lm_head, nn.Linear)
    assert net.a.scales.dtype == torch.float32
    a4.model_to_half(net)
    assert net.a.scales.dtype == torch.float16 and net.a.bias.dtype == torch.float16 and net.a.qweight.dtype == torch.int32
    a4.model_to_float(net)
    assert net.a.scales.dtype == torch.float32


def test_backend_switch():
    assert a4.backend == "cuda" and a4.is_gptq_backend_available() and not a4.is_triton_backend_available()
    a4.switch_backend_to("cuda")
    with pytest.raises(ValueError):
        a4.switch_backend_to("triton")
    with pytest.raises(ValueError):
        a4.switch_backend_to("rocm")


def test_linear4bitlt_matches_unfused_formula_and_grads():
    m, layer = make_module(256, 128, 64, act=True, seed=9, cls=models.Linear4bitLt, r=8, lora_alpha=16, lora_dropout=0.0)
    A, B = synth.make_lora(256, 128, 8, seed=10, dtype=torch.float32)
    m.lora_A["default"].weight.data.copy_(A)
    m.lora_B["default"].weight.data.copy_(B)
    assert m.scaling["default"] == 2.0 and m.active_adapters == ["default"]
    assert [n for n, p in m.named_parameters() if p.requires_grad] == ["lora_A.default.weight", "lora_B.default.weight"]
    x = synth.make_acts(24, 256, 11).requires_grad_(True)
    w = orc.recons_v2(layer.qweight, layer.scales, layer.qzeros, layer.g_idx).float()
    with fake_backend.installed():
        y = m(x)
        dy = torch.randn_like(y)
        y.backward(dy)
    ref = x.detach().float() @ w + orc.lora_forward(x.detach(), A, B, 2.0)
    assert y.dtype == torch.float16 and torch.allclose(y.float(), ref, atol=3e-2, rtol=1e-2)
    dx_l, dA, dB = orc.lora_backward(x.detach(), dy, A, B, 2.0)
    assert torch.allclose(x.grad.float(), dy.float() @ w.t() + dx_l, atol=3e-2, rtol=1e-2)
    assert torch.allclose(m.lora_A["default"].weight.grad, dA, atol=2e-2, rtol=2e-2)
    assert torch.allclose(m.lora_B["default"].weight.grad, dB, atol=2e-2, rtol=2e-2)
    m._disable_adapters = True
    with fake_backend.installed():
        y0 = m(x.detach())
    assert torch.allclose(y0.float(), x.detach().float() @ w, atol=3e-2, rtol=1e-2)


def test_wrap_with_lora_aliases_buffers():
    net = nn.Sequential()
    q, _ = make_module(128, 64, 64, seed=12)
    net.add_module("q_proj", q)
    net.add_module("other", nn.Linear(64, 64))
    models.wrap_with_lora(net, ["q_proj"], r=4, lora_alpha=8)
    assert isinstance(net.q_proj, models.Linear4bitLt)
    assert net.q_proj.qweight.data_ptr() == q.qweight.data_ptr()           # aliased, not copied
    assert not net.other.weight.requires_grad
    assert sum(p.numel() for p in net.parameters() if p.requires_grad) == 4 * 128 + 64 * 4
    assert torch.count_nonzero(net.q_proj.lora_B["default"].weight) == 0   # PEFT default init: B = 0


def test_fused_qkv_equals_separate_outputs():
    mods = [make_module(128, n, 64, seed=20 + i)[0] for i, n in enumerate((64, 32, 32))]    # GQA widths
    x = synth.make_acts(12, 128, 30)
    with fake_backend.installed(), torch.no_grad():
        sep = torch.cat([m(x) for m in mods], dim=-1)
        fused = patch.fuse_quant_linears(mods)
        y = fused(x)
    assert fused.out_features == 128 and fused.qweight.shape == (16, 128) and fused.qzeros.shape == (2, 16)
    assert torch.equal(y, sep)
    assert "qweight" not in mods[0]._buffers                                # sources were emptied


def test_fuse_refuses_mismatched_act_order():
    a, _ = make_module(128, 64, 64, act=True, seed=40)
    b, _ = make_module(128, 64, 64, act=True, seed=41)
    with pytest.raises(ValueError, match="g_idx"):
        patch.fuse_quant_linears([a, b])


def test_merged_lora_injection_adds_q_and_v_slices():
    qkv, _ = make_module(128, 192, 64, seed=50)
    A = torch.randn(2, 4, 128).half() * 0.1
    B = torch.randn(2, 64, 4).half() * 0.1
    lora = patch.CustomLoraLayerMerged(A, B)
    x = synth.make_acts(6, 128, 51).reshape(2, 3, 128)
    with fake_backend.installed(), torch.no_grad():
        base = qkv(x).clone()
        patch.LoraInjectionWrapper(qkv, lora).apply()
        y = qkv(x)
    dq = (x.float() @ A[0].float().t()) @ B[0].float().t()
    dv = (x.float() @ A[1].float().t()) @ B[1].float().t()
    assert torch.allclose((y - base)[..., :64].float(), dq, atol=2e-2)
    assert torch.allclose((y - base)[..., -64:].float(), dv, atol=2e-2)
    assert torch.count_nonzero((y - base)[..., 64:128]) == 0


def test_llama_patches_on_tiny_model():
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=64, max_position_embeddings=64)
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg).half().eval()
    layers = a4.find_layers(model)
    layers.pop("lm_head")
    assert len(layers) == 14
    a4.make_quant_for_4bit_autograd(model, layers, groupsize=64)
    gen = torch.Generator().manual_seed(1)
    for name, mod in model.named_modules():
        if isinstance(mod, a4.Autograd4bitQuantLinear):
            l = synth.make_layer(mod.in_features, mod.out_features, 64, False, gen=gen)
            mod.qweight, mod.qzeros, mod.scales = l.qweight, l.qzeros, (l.scales.float() * 0.2).half()
            mod.bias = torch.zeros(mod.out_features, dtype=torch.float16)
    ids = torch.randint(0, 64, (2, 16), generator=gen)
    with fake_backend.installed(), torch.no_grad():
        ref = model(ids).logits
        patch.make_quant_attn(model)
        patch.make_fused_mlp(model)
        out = model(ids).logits
    mm4b.cache_buffer = True
    assert isinstance(model.model.layers[0].self_attn, patch.QuantLlamaAttention)
    assert isinstance(model.model.layers[0].mlp, patch.QuantLlamaMLP)
    assert model.model.layers[0].self_attn.qkv_proj.out_features == 128 + 64 + 64
    assert torch.allclose(out.float(), ref.float(), atol=5e-2, rtol=5e-2)
