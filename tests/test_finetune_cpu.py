"""The finetune step and its data-parallel gradient exchange on the CPU (kernels replaced by the
oracle): loss goes down, flat gradient buffer aliases every .grad, and two gloo ranks with
different micro-batches end up with the gradients of the one-process global batch."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from alpaca_lora_4bit_b200 import finetune_step as fs
from tests import fake_backend

TINY = fs.LlamaShape(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                     num_key_value_heads=2, vocab_size=64, max_position_embeddings=64)


def build(seed=0):
    model = fs.build_quant_llama(TINY, "cpu", groupsize=64, act_order=True, seed=seed)
    fs.add_lora(model, ["q_proj", "v_proj"], r=4, alpha=8, seed=seed + 1)
    fs.apply_gradient_checkpointing(model)
    return model


def test_structure_and_flat_grads():
    model = build()
    assert fs.quant_linear_params(model) == 2 * (128 * 128 * 2 + 128 * 64 * 2 + 3 * 128 * 256)
    assert fs.lora_param_count(model) == 2 * (4 * 128 + 128 * 4 + 4 * 128 + 64 * 4)
    ft = fs.LoraFinetuner(model, lr=1e-2, loss_scale=1.0, autocast=False)
    assert all(p.grad.data_ptr() >= ft.flat.buffer.data_ptr() for p in ft.params)
    assert sum(p.numel() for p in ft.params) == ft.flat.buffer.numel()


def test_step_learns_on_cpu():
    torch.manual_seed(0)
    model = build().float()
    ft = fs.LoraFinetuner(model, lr=2e-2, loss_scale=1.0, autocast=False)
    ids = torch.randint(0, 64, (2, 16), generator=torch.Generator().manual_seed(1))
    with fake_backend.installed():
        losses = [float(ft.step(ids)) for _ in range(6)]
    assert all(l == l for l in losses)
    assert losses[-1] < losses[0]
    assert float(ft.flat.buffer.abs().sum()) > 0


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _dp_worker(rank, world, port, out):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    model = build().float()
    ft = fs.LoraFinetuner(model, lr=0.0, loss_scale=1.0, autocast=False)
    ids = torch.randint(0, 64, (4, 16), generator=torch.Generator().manual_seed(7))      # global batch of 4
    with fake_backend.installed():
        ft.step(ids[2 * rank:2 * rank + 2])                                               # 2 sequences per rank
    torch.save(ft.flat.buffer.clone(), os.path.join(out, f"g{rank}.pt"))
    dist.destroy_process_group()


def test_two_rank_gradients_equal_global_batch(tmp_path):
    port = _free_port()
    mp.spawn(_dp_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    g0, g1 = torch.load(tmp_path / "g0.pt"), torch.load(tmp_path / "g1.pt")
    assert torch.equal(g0, g1)                                       # identical on every rank after the all-reduce
    model = build().float()
    ft = fs.LoraFinetuner(model, lr=0.0, loss_scale=1.0, autocast=False)
    ids = torch.randint(0, 64, (4, 16), generator=torch.Generator().manual_seed(7))
    with fake_backend.installed():
        ft.step(ids)
    assert torch.allclose(g0, ft.flat.buffer, rtol=2e-3, atol=1e-6)  # mean of rank means = global mean
