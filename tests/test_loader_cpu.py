"""Checkpoint round trips on the CPU (kernels replaced by the oracle, tests/fake_backend.py): a tiny synthetic
GPTQ checkpoint written as ``.safetensors`` + ``config.json`` must come back through
``load_llama_model_4bit_low_ram`` with the logits of the model it was saved from, and a LoRA adapter saved in
PEFT's file layout must give, injected into the fused qkv projection, what ``Linear4bitLt`` layers give."""
import json
import os

import pytest
import torch

from alpaca_lora_4bit_b200 import autograd_4bit as a4, matmul_utils_4bit as mm4b, models, synth
from alpaca_lora_4bit_b200 import model_attn_mlp_patch as patch
from tests import fake_backend


def tiny_quant_llama(kv_heads=2, seed=0, groupsize=64):
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=kv_heads, vocab_size=64, max_position_embeddings=64)
    torch.manual_seed(seed)
    model = LlamaForCausalLM(cfg).half().eval()
    layers = a4.find_layers(model)
    layers.pop("lm_head")
    a4.make_quant_for_4bit_autograd(model, layers, groupsize=groupsize)
    gen = torch.Generator().manual_seed(seed + 1)
    for _, mod in model.named_modules():
        if isinstance(mod, a4.Autograd4bitQuantLinear):
            l = synth.make_layer(mod.in_features, mod.out_features, groupsize, False, gen=gen)
            mod.qweight, mod.qzeros, mod.scales = l.qweight, l.qzeros, (l.scales.float() * 0.2).half()
            mod.bias = torch.zeros(mod.out_features, dtype=torch.float16)
    return cfg, model


def test_safetensors_round_trip_through_the_loader(tmp_path):
    from safetensors.torch import save_file
    cfg, model = tiny_quant_llama()
    cfg.save_pretrained(tmp_path)
    ckpt = os.path.join(tmp_path, "tiny-4bit-64g.safetensors")
    save_file({k: v.contiguous() for k, v in model.state_dict().items()}, ckpt)
    ids = torch.randint(0, 64, (2, 12), generator=torch.Generator().manual_seed(5))
    with fake_backend.installed(), torch.no_grad():
        want = model(ids).logits
    loaded, _tokenizer = a4.load_llama_model_4bit_low_ram(str(tmp_path), ckpt, groupsize=64, half=True, device_map={"": "cpu"})
    assert not loaded.training and loaded.seqlen == 2048
    q = loaded.model.layers[1].self_attn.q_proj
    assert isinstance(q, a4.Autograd4bitQuantLinear) and isinstance(loaded.lm_head, torch.nn.Linear)
    assert q.scales.dtype == torch.float16 and q.qweight.dtype == torch.int32 and q.g_idx.dtype == torch.int32
    assert torch.equal(q.qweight, model.model.layers[1].self_attn.q_proj.qweight)
    # the rotary tables are not in any checkpoint: they must have been recomputed, not left as allocated
    assert torch.allclose(loaded.model.rotary_emb.inv_freq, model.model.rotary_emb.inv_freq)
    with fake_backend.installed(), torch.no_grad():
        got = loaded(ids).logits
    assert torch.equal(got, want)
    # without half=True floating-point entries take the dtype the freshly built module has (fp32), as
    # accelerate's loader does for the reference
    full, _ = a4.load_llama_model_4bit_low_ram(str(tmp_path), ckpt, groupsize=64, half=False, device_map={"": "cpu"})
    assert full.model.layers[0].mlp.down_proj.scales.dtype == torch.float32
    assert full.lm_head.weight.dtype == torch.float32


def test_loader_refuses_a_checkpoint_of_another_shape(tmp_path):
    from safetensors.torch import save_file
    cfg, model = tiny_quant_llama()
    cfg.save_pretrained(tmp_path)
    ckpt = os.path.join(tmp_path, "m.safetensors")
    save_file({k: v.contiguous() for k, v in model.state_dict().items()}, ckpt)
    with pytest.raises(ValueError, match="shape"):
        a4.load_llama_model_4bit_low_ram(str(tmp_path), ckpt, groupsize=32, device_map={"": "cpu"})


@pytest.mark.parametrize("kv_heads", [4, 2])                # multi-head, and grouped-query (narrower k / v)
def test_adapter_files_injected_into_fused_qkv_match_lora_layers(tmp_path, kv_heads):
    _, model = tiny_quant_llama(kv_heads=kv_heads, seed=3)
    r, alpha = 4, 8
    models.wrap_with_lora(model, ["q_proj", "v_proj"], r=r, lora_alpha=alpha)
    gen = torch.Generator().manual_seed(11)
    adapter = {}
    for name, mod in model.named_modules():
        if isinstance(mod, models.Linear4bitLt):
            for fac in ("lora_A", "lora_B"):
                w = getattr(mod, fac)["default"].weight
                w.data = torch.randn(w.shape, generator=gen) * 0.05
                adapter[f"base_model.model.{name}.{fac}.weight"] = w.data.clone()
    ids = torch.randint(0, 64, (2, 10), generator=gen)
    with fake_backend.installed(), torch.no_grad():
        want = model(ids).logits
    # the adapter as PEFT writes it
    with open(os.path.join(tmp_path, "adapter_config.json"), "w") as f:
        json.dump({"r": r, "lora_alpha": alpha, "target_modules": ["q_proj", "v_proj"], "peft_type": "LORA"}, f)
    torch.save(adapter, os.path.join(tmp_path, "adapter_model.bin"))
    # a fresh copy of the base model, fused, with the adapter injected on the fused projection
    _, base = tiny_quant_llama(kv_heads=kv_heads, seed=3)
    try:
        with fake_backend.installed(), torch.no_grad():
            patch.make_quant_attn(base)
            patch.make_fused_mlp(base)
            wrappers = patch.inject_lora_layers(base, str(tmp_path), device="cpu", dtype=torch.float16)
            got = base(ids).logits
    finally:
        mm4b.cache_buffer = True
    assert len(wrappers) == 2
    q_width, v_width = 128, 128 * kv_heads // 4
    assert (wrappers[0].q_size, wrappers[0].v_size) == (q_width, v_width)
    assert torch.allclose(got.float(), want.float(), atol=3e-2, rtol=3e-2)
    # and the injection changed something: without it the fused model differs from the LoRA model
    for w in wrappers:
        w.module.forward = w.module.forward_before_lora
    with fake_backend.installed(), torch.no_grad():
        plain = base(ids).logits
    assert (plain.float() - want.float()).abs().max() > (got.float() - want.float()).abs().max()


def test_lora_state_dict_save_and_load_gives_identical_outputs(tmp_path):
    _, model = tiny_quant_llama(seed=7)
    models.wrap_with_lora(model, ["q_proj", "v_proj"], r=4, lora_alpha=8)
    gen = torch.Generator().manual_seed(2)
    for p in model.parameters():
        if p.requires_grad:
            p.data = torch.randn(p.shape, generator=gen) * 0.05
    lora_state = {k: v for k, v in model.state_dict().items() if "lora_" in k}
    assert len(lora_state) == 2 * 2 * 2                     # two layers x (q, v) x (A, B)
    torch.save(lora_state, os.path.join(tmp_path, "lora.bin"))
    ids = torch.randint(0, 64, (1, 9), generator=gen)
    with fake_backend.installed(), torch.no_grad():
        want = model(ids).logits
    _, other = tiny_quant_llama(seed=7)
    models.wrap_with_lora(other, ["q_proj", "v_proj"], r=4, lora_alpha=8)
    missing, unexpected = other.load_state_dict(torch.load(os.path.join(tmp_path, "lora.bin")), strict=False)
    assert not unexpected and all("lora_" not in k for k in missing)
    with fake_backend.installed(), torch.no_grad():
        got = other(ids).logits
    assert torch.equal(got, want)
