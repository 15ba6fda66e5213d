"""The fused element-wise kernels (RMSNorm, SwiGLU, rotary embedding) against the stock transformers
computation they replace: operator by operator, forward and backward, and on a whole two-layer quantised
LLaMA (loss and LoRA gradients of the patched model against the unpatched one)."""
import copy

import pytest
import torch

from alpaca_lora_4bit_b200 import finetune_step as fs, fused_ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rel(a, b):
    a, b = a.double(), b.double()
    return float((a.detach() - b.detach()).norm() / b.detach().norm())


@pytest.mark.parametrize("rows,H", [(1024, 4096), (7, 8192), (33, 200)])
def test_rmsnorm_matches_stock(rows, H):
    g = torch.Generator(device=DEV).manual_seed(rows + H)
    x = (torch.randn((rows, H), generator=g, device=DEV) * 3).half().requires_grad_(True)
    w = (1 + 0.1 * torch.randn(H, generator=g, device=DEV)).half()
    dy = torch.randn((rows, H), generator=g, device=DEV).half()
    y = fused_ops.rms_norm(x, w, 1e-5)
    y.backward(dy)
    got_dx = x.grad.clone(); x.grad = None
    h = x.to(torch.float32)
    ref = w * (h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5)).to(torch.float16)
    ref.backward(dy)
    assert rel(y, ref) <= 1e-3 and float((y.detach().float() - ref.detach().float()).abs().max()) <= 2e-2      # same two roundings; the sums differ in order
    assert rel(got_dx, x.grad) <= 2e-3
    # fp64 calculus as the arbiter: the fused backward is at least as close as the stock one
    x64 = x.detach().double().requires_grad_(True)
    y64 = w.double() * (x64 * torch.rsqrt(x64.pow(2).mean(-1, keepdim=True) + 1e-5))
    y64.backward(dy.double())
    assert rel(got_dx, x64.grad) <= 1.05 * rel(x.grad, x64.grad) + 1e-5


@pytest.mark.parametrize("rows,I,fused_input", [(1024, 11008, False), (5, 256, False), (300, 1024, True)])
def test_swiglu_matches_stock(rows, I, fused_input):
    g = torch.Generator(device=DEV).manual_seed(rows + I)
    if fused_input:                                              # the two halves of one gate_up output
        gu = (torch.randn((rows, 2 * I), generator=g, device=DEV) * 2).half().requires_grad_(True)
        gate, up = torch.split(gu, I, dim=-1)
    else:
        gate = (torch.randn((rows, I), generator=g, device=DEV) * 2).half().requires_grad_(True)
        up = torch.randn((rows, I), generator=g, device=DEV).half().requires_grad_(True)
    d = torch.randn((rows, I), generator=g, device=DEV).half()
    out = fused_ops.swiglu(gate, up)
    ref = torch.nn.functional.silu(gate) * up
    assert rel(out, ref) <= 1e-3
    leaves = [gu] if fused_input else [gate, up]
    got = torch.autograd.grad(out, leaves, d)
    want = torch.autograd.grad(ref, leaves, d)
    for a, b in zip(got, want):
        assert rel(a, b) <= 3e-3


@pytest.mark.parametrize("B,T,H,KV,D,TB", [(4, 256, 32, 32, 128, 1), (1, 77, 8, 2, 64, 1), (3, 40, 4, 4, 32, 3)])
def test_rope_matches_stock(B, T, H, KV, D, TB):
    """TB: batch of the cos / sin tables (1 = the tables of one sequence, broadcast over the batch, as the model passes them)."""
    g = torch.Generator(device=DEV).manual_seed(T + D)
    q = torch.randn((B, T, H * D), generator=g, device=DEV).half().requires_grad_(True)
    k = torch.randn((B, T, KV * D), generator=g, device=DEV).half().requires_grad_(True)
    ang = torch.rand((TB, T, D // 2), generator=g, device=DEV) * 6.28
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1).half(), torch.cat([ang.sin(), ang.sin()], -1).half()
    qv, kv = q.view(B, T, H, D).transpose(1, 2), k.view(B, T, KV, D).transpose(1, 2)
    qe, ke = fused_ops.apply_rotary_pos_emb(qv, kv, cos, sin)
    c, s = cos.unsqueeze(1), sin.unsqueeze(1)
    qr, kr = qv * c + fused_ops._rotate_half(qv) * s, kv * c + fused_ops._rotate_half(kv) * s
    assert qe.shape == qr.shape and rel(qe, qr) <= 1e-3 and rel(ke, kr) <= 1e-3
    dq, dk = torch.randn_like(qr), torch.randn_like(kr)
    got = torch.autograd.grad([qe, ke], [q, k], [dq, dk])
    want = torch.autograd.grad([qr, kr], [q, k], [dq, dk])
    assert rel(got[0], want[0]) <= 2e-3 and rel(got[1], want[1]) <= 2e-3


def test_patched_llama_step_matches_stock():
    shape = fs.LlamaShape(hidden_size=512, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=8,
                          num_key_value_heads=4, vocab_size=1000, max_position_embeddings=256)

    def build(patched):
        model = fs.build_quant_llama(shape, DEV, groupsize=128, seed=3)
        fs.add_lora(model, ["q_proj", "v_proj"], r=8, alpha=16, seed=4)
        if patched:
            fused_ops.patch_llama(model)
        fs.apply_gradient_checkpointing(model)
        model.train()
        return fs.LoraFinetuner(model, lr=0.0, loss_scale=64.0, dynamic_scale=False)

    ids = torch.randint(0, 1000, (2, 64), generator=torch.Generator().manual_seed(9)).to(DEV)
    from transformers.models.llama import modeling_llama as ml
    stock_rope = ml.apply_rotary_pos_emb
    try:
        a = build(False)
        la = float(a.step(ids)); ga = a.flat.buffer.clone()
        b = build(True)
        lb = float(b.step(ids)); gb = b.flat.buffer.clone()
    finally:
        ml.apply_rotary_pos_emb = stock_rope
    assert abs(la - lb) <= 2e-3 * abs(la)
    assert rel(gb, ga) <= 2e-2


def test_skip_path_adds_in_the_projection_epilogues():
    """patch_llama hands the two residual adds of every decoder layer to o_proj / down_proj
    (``q4_gemm_fwd_residual``): same logits and same LoRA gradients as the model with the stock layer forward,
    where the adds are torch kernels; the product itself (quant_cuda.gemm with a residual) equals product + add to the bit."""
    from alpaca_lora_4bit_b200 import quant_cuda, synth
    layer = synth.make_layer(1024, 768, 128, False, seed=3).to(DEV)
    x = synth.make_acts(300, 1024, seed=4).to(DEV)
    res = synth.make_acts(300, 768, seed=5).to(DEV)
    bias = (torch.randn(768, generator=torch.Generator().manual_seed(6)) * 0.1).half().to(DEV)
    for variant in (0, 1, 2, 3):
        quant_cuda.gemm_set_variant(variant)
        try:
            plain = torch.empty(300, 768, dtype=torch.float16, device=DEV)
            quant_cuda.gemm(x, layer.qweight, plain, layer.scales, layer.qzeros, layer.g_idx, bias=bias)
            fused = torch.empty_like(plain)
            quant_cuda.gemm(x, layer.qweight, fused, layer.scales, layer.qzeros, layer.g_idx, bias=bias, residual=res)
        finally:
            quant_cuda.gemm_set_variant(0)
        assert torch.equal(fused, plain + res), variant

    ids = torch.randint(0, 256, (2, 96), generator=torch.Generator().manual_seed(8)).to(DEV)
    shape = fs.LlamaShape(hidden_size=512, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=8,
                          num_key_value_heads=4, vocab_size=256, max_position_embeddings=256)

    def run(patch_layers):
        model = fs.build_quant_llama(shape, DEV, groupsize=128, seed=2)
        fs.add_lora(model, ["q_proj", "v_proj", "o_proj", "down_proj"], r=8, alpha=16, seed=3)
        if patch_layers:
            fused_ops.patch_llama(model)
            assert "forward" in model.model.layers[0].__dict__
        fs.apply_gradient_checkpointing(model)
        model.train()
        ft = fs.LoraFinetuner(model, lr=0.0, loss_scale=64.0, dynamic_scale=False)
        loss = float(ft.step(ids))
        torch.cuda.synchronize()
        for layer_ in model.model.layers:                       # nothing is left behind on the projections
            assert "_q4_residual" not in layer_.self_attn.o_proj.__dict__ and "_q4_residual" not in layer_.mlp.down_proj.__dict__
        return loss, ft.flat.buffer.clone()

    stock_rope = __import__("transformers.models.llama.modeling_llama", fromlist=["x"]).apply_rotary_pos_emb
    try:
        loss_p, g_p = run(True)
    finally:
        __import__("transformers.models.llama.modeling_llama", fromlist=["x"]).apply_rotary_pos_emb = stock_rope
    loss_s, g_s = run(False)
    assert abs(loss_p - loss_s) <= 2e-3 * abs(loss_s)
    assert float((g_p - g_s).norm() / g_s.norm()) <= 2e-2


def test_fused_gate_up_trains_like_two_layers():
    """patch_llama(fuse_gate_up=True) replaces the MLPs (no adapter on gate / up) by the fused-gate/up module: same
    loss and same LoRA gradients as the model with two layers, through checkpointing and the whole finetune step;
    an MLP with an adapter on gate_proj is left alone."""
    from alpaca_lora_4bit_b200 import model_attn_mlp_patch as patch
    ids = torch.randint(0, 256, (2, 96), generator=torch.Generator().manual_seed(8)).to(DEV)
    shape = fs.LlamaShape(hidden_size=512, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=8,
                          num_key_value_heads=4, vocab_size=256, max_position_embeddings=256)

    def run(fuse, targets):
        model = fs.build_quant_llama(shape, DEV, groupsize=128, seed=2)
        fs.add_lora(model, targets, r=8, alpha=16, seed=3)
        fused_ops.patch_llama(model, fuse_gate_up=fuse)
        n_fused = sum(isinstance(m, patch.QuantLlamaMLP) for m in model.modules())
        fs.apply_gradient_checkpointing(model)
        model.train()
        ft = fs.LoraFinetuner(model, lr=0.0, loss_scale=64.0, dynamic_scale=False)
        loss = float(ft.step(ids))
        torch.cuda.synchronize()
        return loss, ft.flat.buffer.clone(), n_fused

    stock_rope = __import__("transformers.models.llama.modeling_llama", fromlist=["x"]).apply_rotary_pos_emb
    try:
        loss_f, g_f, n_f = run(True, ["q_proj", "v_proj", "down_proj"])
        loss_s, g_s, n_s = run(False, ["q_proj", "v_proj", "down_proj"])
        _, _, n_adapter = run(True, ["q_proj", "gate_proj"])
    finally:
        __import__("transformers.models.llama.modeling_llama", fromlist=["x"]).apply_rotary_pos_emb = stock_rope
    assert n_f == 2 and n_s == 0 and n_adapter == 0
    assert abs(loss_f - loss_s) <= 2e-3 * abs(loss_s)
    assert float((g_f - g_s).norm() / g_s.norm()) <= 2e-2


@pytest.mark.parametrize("rows,I", [(300, 1024), (1024, 11008), (5, 8)])
def test_swiglu_on_a_fused_gate_up_tensor(rows, I):
    """swiglu_fused takes [gate | up] as one tensor and returns one gradient tensor for it: same values as the
    two-tensor form (and as the stock expression), no concatenation in the backward."""
    g = torch.Generator(device=DEV).manual_seed(rows + I)
    gu = (torch.randn((2, rows, 2 * I), generator=g, device=DEV) * 2).half().requires_grad_(True)
    d = torch.randn((2, rows, I), generator=g, device=DEV).half()
    out = fused_ops.swiglu_fused(gu)
    gate, up = torch.split(gu, I, dim=-1)
    assert torch.equal(out, fused_ops.swiglu(gate, up))
    ref = torch.nn.functional.silu(gate) * up
    assert rel(out, ref) <= 1e-3
    (got,) = torch.autograd.grad(out, [gu], d)
    (two,) = torch.autograd.grad(fused_ops.swiglu(gate, up), [gu], d)
    (want,) = torch.autograd.grad(ref, [gu], d)
    assert torch.equal(got, two) and rel(got, want) <= 3e-3
