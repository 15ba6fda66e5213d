"""The LoRA finetune step on the GPU with the real kernels: the fused tensor-core path and the
reference composition (reconstruct + library GEMM, LoRA as separate small GEMMs) must agree on loss
and gradients, the step must learn, and the CUDA-graph replay must reproduce the eager step."""
import pytest
import torch

from alpaca_lora_4bit_b200 import finetune_step as fs, matmul_utils_4bit as mm4b, models, quant_cuda

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SMALL = fs.LlamaShape(hidden_size=512, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=8,
                      num_key_value_heads=4, vocab_size=256, max_position_embeddings=128)


def build(act_order, seed=0):
    model = fs.build_quant_llama(SMALL, torch.device(DEV), groupsize=128, act_order=act_order, seed=seed)
    fs.add_lora(model, ["q_proj", "v_proj"], r=8, alpha=16, seed=seed + 1)
    fs.apply_gradient_checkpointing(model)
    model.train()
    return model


def one_step_grads(fused, act_order):
    mm4b.fused_gemm = fused
    models.fused_lora = fused
    try:
        model = build(act_order)
        ft = fs.LoraFinetuner(model, lr=0.0, loss_scale=64.0, dynamic_scale=False)
        ids = torch.randint(0, 256, (4, 96), generator=torch.Generator().manual_seed(5)).to(DEV)
        loss = float(ft.step(ids))
        torch.cuda.synchronize()
        assert quant_cuda.device_status() == 0
        return loss, ft.flat.buffer.clone()
    finally:
        mm4b.fused_gemm = True
        models.fused_lora = True


@pytest.mark.parametrize("act_order", [False, True])
def test_fused_step_matches_reconstruct_and_library_gemm(act_order):
    """384 token rows per quant linear: forward, checkpoint recompute and backward all take the fused
    dequant-GEMM (with the LoRA stage on q_proj / v_proj); the same step with the kernels switched to
    the reference's composition gives the same loss and LoRA gradients."""
    loss_f, g_f = one_step_grads(True, act_order)
    loss_r, g_r = one_step_grads(False, act_order)
    assert loss_f == loss_f and abs(loss_f - loss_r) <= 2e-3 * abs(loss_r)
    assert float(g_r.abs().max()) > 0
    rel = float((g_f - g_r).norm() / g_r.norm())
    assert rel <= 2e-2, rel                     # fp16 activations end to end: two roundings of every layer output differ


def test_step_learns_and_graph_replay_matches_eager():
    torch.manual_seed(0)
    ids = torch.randint(0, 256, (4, 64), generator=torch.Generator().manual_seed(9)).to(DEV)
    eager = fs.LoraFinetuner(build(False), lr=5e-3, loss_scale=64.0, dynamic_scale=False)
    graphed = fs.LoraFinetuner(build(False), lr=5e-3, loss_scale=64.0, dynamic_scale=False)
    assert graphed.capture(ids, warmup=2)       # two eager steps on a side stream, then the capture (which runs nothing)
    le = [float(eager.step(ids)) for _ in range(6)]
    lg = [float(graphed.step(ids)) for _ in range(4)]
    torch.cuda.synchronize()
    assert quant_cuda.device_status() == 0
    assert all(v == v for v in le) and le[-1] < le[0]
    for a, b in zip(le[2:], lg):                # replay k continues where the two warm-up steps left off
        assert abs(a - b) <= 1e-3 * abs(a)


def test_gqa_act_order_all_projections_bf16_autocast():
    """The shape of the large configuration in small: grouped-query attention, act-order g_idx, LoRA r=16 on all
    seven projections, bf16 autocast (the quant linears and the LoRA products still compute in fp16, hence the
    static loss scale), with the fused element-wise kernels routed in.  Fused kernels against the reference's
    composition: same loss, same LoRA gradients; finite everywhere."""
    from alpaca_lora_4bit_b200 import fused_ops
    from transformers.models.llama import modeling_llama as ml
    shape = fs.LlamaShape(hidden_size=1024, intermediate_size=3584, num_hidden_layers=2, num_attention_heads=8,
                          num_key_value_heads=1, vocab_size=512, max_position_embeddings=512)
    targets = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]
    ids = torch.randint(0, 512, (1, 256), generator=torch.Generator().manual_seed(3)).to(DEV)
    stock_rope = ml.apply_rotary_pos_emb

    def run(fused):
        mm4b.fused_gemm = fused
        models.fused_lora = fused
        try:
            model = fs.build_quant_llama(shape, torch.device(DEV), groupsize=128, act_order=True, seed=4, gain=0.5)
            fs.add_lora(model, targets, r=16, alpha=32, seed=5)
            if fused:
                fused_ops.patch_llama(model)
            fs.apply_gradient_checkpointing(model)
            model.train()
            ft = fs.LoraFinetuner(model, lr=0.0, loss_scale=256.0, autocast_dtype=torch.bfloat16)
            loss = float(ft.step(ids))
            torch.cuda.synchronize()
            assert quant_cuda.device_status() == 0
            return loss, ft.flat.buffer.clone()
        finally:
            mm4b.fused_gemm = True
            models.fused_lora = True
            ml.apply_rotary_pos_emb = stock_rope

    loss_f, g_f = run(True)
    loss_r, g_r = run(False)
    assert loss_f == loss_f and bool(torch.isfinite(g_f).all()) and float(g_f.abs().max()) > 0
    assert abs(loss_f - loss_r) <= 5e-3 * abs(loss_r)
    rel = float((g_f - g_r).norm() / g_r.norm())
    assert rel <= 3e-2, rel
