"""q4_adamw_flat (AdamW with loss-scale handling over flat buffers, three launches per step) against
torch.optim.AdamW under torch.amp.GradScaler, which is what the reference's trainer runs
(finetune.py:150-170 of the reference: optim="adamw_torch", fp16=True)."""
import pytest
import torch

from alpaca_lora_4bit_b200 import finetune_step as fs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _params(seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    shapes = [(8, 256), (512, 8), (16, 1000), (3,), (1001, 7)]
    return [torch.nn.Parameter(torch.randn(s, generator=g, device=DEV)) for s in shapes]


@pytest.mark.parametrize("dynamic", [True, False])
def test_matches_torch_adamw_under_gradscaler(dynamic):
    ours, ref = _params(1), _params(1)
    flat = fs.FlatGrads(ours)
    opt = fs.FlatAdamW(ours, flat, lr=3e-3, init_scale=1024.0, dynamic=dynamic, growth_interval=3)
    ropt = torch.optim.AdamW(ref, lr=3e-3)
    # a static scale is compared with a scaler that never gets to grow and sees no overflow
    scaler = torch.amp.GradScaler("cuda", init_scale=1024.0, growth_interval=3 if dynamic else 10 ** 9)
    scaler.scale(torch.zeros(1, device=DEV))                                   # creates its device-side state
    bad_steps = (2, 6) if dynamic else ()
    g = torch.Generator(device=DEV).manual_seed(2)
    taken = 0
    for step in range(9):
        grads = [torch.randn(p.shape, generator=g, device=DEV) for p in ref]
        if step in bad_steps:
            grads[1][5, 3] = float("inf") if step == 2 else float("nan")       # a step the scaler must skip
        scale = float(scaler.get_scale())
        assert opt.loss_scale == scale
        flat.zero()
        for p, q, gr in zip(ours, ref, grads):
            p.grad.copy_(gr * scale)                                           # what backward of the scaled loss leaves
            q.grad = gr * scale
        opt.step()
        scaler.step(ropt)
        scaler.update()
        taken += step not in bad_steps
        assert opt.steps_taken == taken
        for p, q in zip(ours, ref):
            assert torch.allclose(p, q, rtol=2e-6, atol=2e-7), (step, float((p - q).abs().max()))
    assert opt.loss_scale == float(scaler.get_scale())


def test_gradients_summed_over_ranks_are_divided():
    ours, ref = _params(3), _params(3)
    flat = fs.FlatGrads(ours)
    opt = fs.FlatAdamW(ours, flat, lr=1e-2, init_scale=8.0, dynamic=False)
    ropt = torch.optim.AdamW(ref, lr=1e-2)
    g = torch.Generator(device=DEV).manual_seed(4)
    grads = [torch.randn(p.shape, generator=g, device=DEV) for p in ref]
    for p, q, gr in zip(ours, ref, grads):
        p.grad.copy_(gr * 8.0 * 4.0)                                           # four ranks' scaled gradients, summed
        q.grad = gr.clone()
    opt.step(grad_div=4.0)
    ropt.step()
    for p, q in zip(ours, ref):
        assert torch.allclose(p, q, rtol=2e-6, atol=2e-7)
    # the parameters are views of one buffer, in order
    assert ours[0].data_ptr() == opt.param.data_ptr()
    assert ours[1].data_ptr() == opt.param.data_ptr() + 4 * ours[0].numel()


def test_half_copies_follow_the_parameters():
    """The optimiser kernel keeps an fp16 copy of every parameter for the LoRA kernels (``_q4_half``); an in-place
    write to a parameter makes ``models._half_of`` cast again until ``refresh_half``."""
    from alpaca_lora_4bit_b200 import models
    ps = _params(7)
    flat = fs.FlatGrads(ps)
    opt = fs.FlatAdamW(ps, flat, lr=1e-2, init_scale=1.0, dynamic=False)
    for p in ps:
        assert torch.equal(p._q4_half, p.detach().half()) and models._half_of(p) is p._q4_half
    for p in ps:
        p.grad.copy_(torch.randn(p.shape, device=DEV))
    opt.step()
    for p in ps:
        assert torch.equal(p._q4_half, p.detach().half()) and models._half_of(p) is p._q4_half
    with torch.no_grad():
        ps[0].mul_(2.0)
    assert models._half_of(ps[0]) is not ps[0]._q4_half and torch.equal(models._half_of(ps[0]), ps[0].detach().half())
    opt.refresh_half()
    assert models._half_of(ps[0]) is ps[0]._q4_half and torch.equal(ps[0]._q4_half, ps[0].detach().half())
