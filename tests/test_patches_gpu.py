"""The fused inference patches (one quantised qkv projection, one gate_up projection, merged q / v LoRA) and
the small-M routing on the real kernels: a patched model must compute what the unpatched one does."""
import json
import os

import pytest
import torch

from alpaca_lora_4bit_b200 import autograd_4bit as a4, finetune_step as fs, matmul_utils_4bit as mm4b, models, synth
from alpaca_lora_4bit_b200 import model_attn_mlp_patch as patch
from oracle import q4_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rel(a, b):
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return float((a - b).norm() / b.norm())


def small_llama(kv_heads, seed):
    shape = fs.LlamaShape(hidden_size=1024, intermediate_size=2816, num_hidden_layers=2, num_attention_heads=8,
                          num_key_value_heads=kv_heads, vocab_size=512, max_position_embeddings=512)
    return fs.build_quant_llama(shape, DEV, groupsize=128, seed=seed).eval()


@pytest.mark.parametrize("epilogue_rows", [1024, 9])          # SwiGLU as its own kernel, and in the gate_up GEMM's epilogue
@pytest.mark.parametrize("kv_heads", [8, 2])                  # multi-head, and grouped-query (narrower k / v)
def test_fused_attention_and_mlp_match_the_unpatched_model(kv_heads, epilogue_rows):
    ids = torch.randint(0, 512, (2, 160), generator=torch.Generator().manual_seed(1)).to(DEV)
    one = ids[:, :1]
    keep_rows = patch.swiglu_epilogue_rows
    patch.swiglu_epilogue_rows = epilogue_rows
    try:
        with torch.no_grad():
            plain = small_llama(kv_heads, seed=11)
            want = plain(ids).logits                             # prefill: 320 rows through the fused GEMM kernels
            out = plain(ids, use_cache=True)
            want_next = plain(ids[:, -1:] * 0 + 7, past_key_values=out.past_key_values, use_cache=True).logits   # one decode step
            fused = small_llama(kv_heads, seed=11)
            patch.make_quant_attn(fused)
            patch.make_fused_mlp(fused)
            got = fused(ids).logits
            out2 = fused(ids, use_cache=True)
            got_next = fused(ids[:, -1:] * 0 + 7, past_key_values=out2.past_key_values, use_cache=True).logits
    finally:
        mm4b.cache_buffer = True
        patch.swiglu_epilogue_rows = keep_rows
    layer0 = fused.model.layers[0]
    assert isinstance(layer0.self_attn, patch.QuantLlamaAttention) and isinstance(layer0.mlp, patch.QuantLlamaMLP)
    assert layer0.self_attn.qkv_proj.out_features == 1024 + 2 * 128 * kv_heads
    assert layer0.mlp.gate_up_proj.out_features == 2 * 2816
    assert rel(got, want) <= 2e-3
    assert rel(got_next, want_next) <= 2e-3
    assert got_next.shape == (2, 1, 512) and one.shape == (2, 1)


def test_injected_adapter_matches_lora_layers_on_gqa(tmp_path):
    r, alpha = 8, 16
    model = small_llama(2, seed=21)
    models.wrap_with_lora(model, ["q_proj", "v_proj"], r=r, lora_alpha=alpha)
    gen = torch.Generator().manual_seed(5)
    adapter = {}
    for name, mod in model.named_modules():
        if isinstance(mod, models.Linear4bitLt):
            for fac in ("lora_A", "lora_B"):
                w = getattr(mod, fac)["default"].weight
                w.data = (torch.randn(w.shape, generator=gen) * 0.03).to(DEV)
                adapter[f"base_model.model.{name}.{fac}.weight"] = w.data.cpu().clone()
    ids = torch.randint(0, 512, (2, 96), generator=gen).to(DEV)
    with torch.no_grad():
        want = model(ids).logits
    with open(os.path.join(tmp_path, "adapter_config.json"), "w") as f:
        json.dump({"r": r, "lora_alpha": alpha, "target_modules": ["q_proj", "v_proj"], "peft_type": "LORA"}, f)
    torch.save(adapter, os.path.join(tmp_path, "adapter_model.bin"))
    base = small_llama(2, seed=21)
    try:
        with torch.no_grad():
            patch.make_quant_attn(base)
            patch.make_fused_mlp(base)
            wrappers = patch.inject_lora_layers(base, str(tmp_path), device=DEV, dtype=torch.float16)
            got = base(ids).logits
    finally:
        mm4b.cache_buffer = True
    assert (wrappers[0].q_size, wrappers[0].v_size) == (1024, 256)
    assert rel(got, want) <= 3e-3


@pytest.mark.parametrize("rows", [1, 9, 16])
@pytest.mark.parametrize("grad", [True, False])
def test_act_order_layer_with_few_rows_honours_g_idx(rows, grad):
    """A handful of rows on an act-order layer, module flags at their defaults: the reconstruct path of the
    reference always reads g_idx (matmul_utils_4bit.py:121), so must every route here - with grad enabled
    (autograd function) and without (matmul4bit above the switch threshold)."""
    layer = synth.make_layer(1024, 768, 128, act_order=True, seed=31)
    m = a4.Autograd4bitQuantLinear(1024, 768, groupsize=128).to(DEV)
    L = layer.to(DEV)
    m.qweight, m.qzeros, m.scales, m.g_idx = L.qweight, L.qzeros, L.scales, L.g_idx
    m.bias = torch.zeros(768, dtype=torch.float16, device=DEV)
    x = synth.make_acts(rows, 1024, seed=rows)
    want = orc.matmul4bit_ref(x, layer.qweight, layer.scales, layer.qzeros, layer.g_idx)
    assert not mm4b.act_order
    xd = x.to(DEV).requires_grad_(grad)
    with torch.set_grad_enabled(grad):
        y = m(xd)
    if rows > 8 or grad:                      # <= 8 rows without grad: the decode entry, which takes sequential groups by contract
        assert rel(y, want) <= 2e-3
    if grad:
        dy = synth.make_acts(rows, 768, seed=3).to(DEV)
        y.backward(dy)
        want_dx = orc.matmul4bit_ref(dy.cpu(), layer.qweight, layer.scales, layer.qzeros, layer.g_idx, transpose=True)
        assert rel(xd.grad, want_dx) <= 2e-3


def test_two_bit_autograd_function_forward_backward():
    layer = synth.make_layer(1024, 512, 128, True, seed=41, bits=2)
    L = layer.to(DEV)
    x = synth.make_acts(40, 1024, seed=1).to(DEV).requires_grad_(True)
    dy = synth.make_acts(40, 512, seed=2).to(DEV)
    y = a4.AutogradMatmul2bit.apply(x, L.qweight, L.scales, L.qzeros, L.g_idx, 2, 3)
    y.backward(dy)
    w = orc.recons2_v2(layer.qweight, layer.scales, layer.qzeros, layer.g_idx).float()
    assert rel(y, x.detach().cpu().float() @ w) <= 2e-3
    assert rel(x.grad, dy.cpu().float() @ w.t()) <= 2e-3
    m = a4.Autograd4bitQuantLinear(1024, 512, groupsize=128, bits=2).to(DEV)
    m.qweight, m.qzeros, m.scales, m.g_idx = L.qweight, L.qzeros, L.scales, L.g_idx
    m.bias = torch.zeros(512, dtype=torch.float16, device=DEV)
    with torch.no_grad():
        assert rel(m(x.detach()), x.detach().cpu().float() @ w) <= 2e-3
