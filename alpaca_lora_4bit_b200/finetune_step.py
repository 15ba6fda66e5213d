"""One LoRA finetune step over a 4-bit LLaMA, single GPU or data parallel.

This is the caller whose step the benchmark times: what the reference's ``finetune.py`` sets up
around the quant linears (finetune.py:36-188) without the HF Trainer: every ``nn.Linear`` but
``lm_head`` becomes an ``Autograd4bitQuantLinear`` (autograd_4bit.py:266-272), the target
projections get ``Linear4bitLt`` LoRA layers (models.py:13-76), every decoder layer runs under
``torch.utils.checkpoint`` with the embedding output as a grad-requiring leaf
(gradient_checkpointing.py:19-65), fp16 autocast with loss scaling, AdamW on the LoRA factors.
Data parallelism follows the reference's DDP use (Finetune4bConfig.py:83-88, finetune.py:166):
every rank holds the whole int4 base and its own micro-batch; the only exchange is one
all-reduce of the LoRA gradients, here over a single flat fp32 buffer that all ``.grad`` fields
alias, so one collective per step moves everything.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Iterable, List, Optional

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from .autograd_4bit import Autograd4bitQuantLinear, find_layers, make_quant_for_4bit_autograd, reset_rotary_buffers
from .models import Linear4bitLt, wrap_with_lora


@dataclass
class LlamaShape:
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    vocab_size: int = 32000
    max_position_embeddings: int = 2048

    @staticmethod
    def llama_7b() -> "LlamaShape":
        return LlamaShape()

    @staticmethod
    def llama2_70b() -> "LlamaShape":
        return LlamaShape(8192, 28672, 80, 64, 8, 32000, 4096)


def fill_random_quant(mod: Autograd4bitQuantLinear, gen: torch.Generator, act_order: bool, scale_mul: float = 1.0):
    """Random GPTQ v2 contents on the module's device: uniform levels, zero points 0..14, fp16 scales
    uniform in [0.002, 0.02] * scale_mul, sequential or permuted ``g_idx``."""
    dev = mod.qweight.device
    K, N, g = mod.in_features, mod.out_features, mod.groupsize
    G = math.ceil(K / g)
    mod.qweight = torch.randint(-2 ** 31, 2 ** 31 - 1, (K // 8, N), generator=gen, device=dev, dtype=torch.int64).to(torch.int32)
    zl = torch.randint(0, 15, (G, N), generator=gen, device=dev, dtype=torch.int64)
    sh = torch.arange(8, device=dev, dtype=torch.int64) * 4
    zw = (zl.reshape(G, N // 8, 8) << sh).sum(-1)
    mod.qzeros = torch.where(zw >= 2 ** 31, zw - 2 ** 32, zw).to(torch.int32)
    mod.scales = ((torch.rand((G, N), generator=gen, device=dev) * 0.018 + 0.002) * scale_mul).half()
    if act_order:
        mod.g_idx = (torch.randperm(K, generator=gen, device=dev) // g).to(torch.int32)
    else:
        mod.g_idx = (torch.arange(K, device=dev) // g).to(torch.int32)
    mod.bias = torch.zeros(N, dtype=torch.float16, device=dev)


def build_quant_llama(shape: LlamaShape, device, groupsize: int = 128, act_order: bool = False, seed: int = 0,
                      attn_implementation: str = "sdpa", gain: float = 1.0) -> nn.Module:
    """Random-init LLaMA of the given shape with every linear but ``lm_head`` quantised (4-bit, v2).

    Built on the meta device so the dense fp16 weights of the replaced linears never exist.  ``gain`` scales
    every quantised layer (1.0 = unit gain); deep stacks of random layers want less."""
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=shape.hidden_size, intermediate_size=shape.intermediate_size,
                      num_hidden_layers=shape.num_hidden_layers, num_attention_heads=shape.num_attention_heads,
                      num_key_value_heads=shape.num_key_value_heads, vocab_size=shape.vocab_size,
                      max_position_embeddings=shape.max_position_embeddings, attn_implementation=attn_implementation)
    with torch.device("meta"):
        model = LlamaForCausalLM(cfg)
    model = model.half()
    layers = find_layers(model)
    layers.pop("lm_head", None)
    make_quant_for_4bit_autograd(model, layers, groupsize=groupsize)
    model = model.to_empty(device=device)
    gen = torch.Generator(device=device).manual_seed(seed)
    for name, mod in model.named_modules():
        if isinstance(mod, Autograd4bitQuantLinear):
            # random levels minus random zero points have a standard deviation of about 6.3 levels and the
            # base scales average 0.011; shrink them so that every layer has unit gain (std(W) = 1/sqrt(K)),
            # as trained checkpoints roughly do - otherwise 32 random layers overflow fp16
            fill_random_quant(mod, gen, act_order, scale_mul=gain / (6.3 * 0.011 * math.sqrt(mod.in_features)))
    with torch.no_grad():
        for name, prm in model.named_parameters():
            if prm.dim() >= 2:
                prm.copy_((torch.randn(prm.shape, generator=gen, device=device) * 0.02).to(prm.dtype))
            else:
                prm.fill_(1.0)                                     # RMSNorm weights
    reset_rotary_buffers(model, cfg, device)       # non-persistent buffers, created on the meta device
    model.config.use_cache = False
    return model


def add_lora(model: nn.Module, targets: Iterable[str], r: int, alpha: int, std_a: float = 0.02, std_b: float = 0.01,
             seed: int = 1) -> nn.Module:
    """LoRA on the named projections: fp32 factors (as fresh PEFT adapters are), A ~ N(0, std_a), B ~ N(0, std_b)."""
    wrap_with_lora(model, list(targets), r=r, lora_alpha=alpha, lora_dropout=0.0)
    dev = next(model.parameters()).device
    gen = torch.Generator(device=dev).manual_seed(seed)
    for mod in model.modules():
        if isinstance(mod, Linear4bitLt):
            for name in mod.lora_A.keys():
                a, b = mod.lora_A[name].weight, mod.lora_B[name].weight
                a.data = (torch.randn(a.shape, generator=gen, device=dev) * std_a).float()
                b.data = (torch.randn(b.shape, generator=gen, device=dev) * std_b).float()
    return model


def apply_gradient_checkpointing(model: nn.Module) -> None:
    """Recompute every decoder layer in the backward (gradient_checkpointing.py:47-65)."""
    for layer in model.model.layers:
        inner = layer.forward

        def wrapped(*args, _inner=inner, **kwargs):
            # no dropout anywhere in the step, so there is no RNG state to save and restore
            return checkpoint(_inner, *args, use_reentrant=False, preserve_rng_state=False, **kwargs)

        layer.forward = wrapped
    # the embedding output must carry a gradient or the checkpointed segments have nothing to differentiate
    model.get_input_embeddings().register_forward_hook(lambda m, i, o: o.requires_grad_(True))


class FlatGrads:
    """All trainable gradients as views of one contiguous fp32 buffer (one collective per step)."""

    def __init__(self, params: List[nn.Parameter]):
        self.params = params
        total = sum(p.numel() for p in params)
        self.buffer = torch.zeros(total, dtype=torch.float32, device=params[0].device)
        off = 0
        for p in params:
            p.grad = self.buffer[off:off + p.numel()].view_as(p)
            off += p.numel()

    def zero(self):
        self.buffer.zero_()

    def all_reduce_sum(self, group=None) -> int:
        """Sums the buffer over the ranks; returns the number of ranks (the divisor the optimiser applies)."""
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(self.buffer, op=dist.ReduceOp.SUM, group=group)
            return dist.get_world_size(group)
        return 1

    def all_reduce_mean(self, group=None):
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(self.buffer, op=dist.ReduceOp.SUM, group=group)
            self.buffer.div_(dist.get_world_size(group))


class FlatAdamW:
    """AdamW with loss-scale handling over flat buffers: the trainable factors become views of one fp32
    buffer (as their gradients are views of ``FlatGrads.buffer``) and a step is one ``q4_adamw_flat`` call,
    three launches whatever the number of adapters, with the step count and the loss scale kept on the device
    so that the step can be captured.  Same arithmetic as ``torch.optim.AdamW`` under ``torch.amp.GradScaler``
    (what the reference's trainer runs, finetune.py:150-170)."""

    def __init__(self, params: List[nn.Parameter], flat: "FlatGrads", lr: float, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, init_scale: float = 65536.0, dynamic: bool = True, growth_factor: float = 2.0,
                 backoff_factor: float = 0.5, growth_interval: int = 2000):
        dev = params[0].device
        total = flat.buffer.numel()
        self.params = params
        self.param = torch.empty(total, dtype=torch.float32, device=dev)
        off = 0
        for p in params:
            n = p.numel()
            self.param[off:off + n].copy_(p.data.reshape(-1))
            p.data = self.param[off:off + n].view_as(p)
            off += n
        # fp16 copy of the parameters, refreshed by the optimiser kernel: the LoRA kernels compute in fp16 and would
        # otherwise cast every factor on every use (three times per step under checkpointing)
        self.param_h = self.param.to(torch.float16)
        off = 0
        for p in params:
            n = p.numel()
            p._q4_half = self.param_h[off:off + n].view_as(p)
            p._q4_half_version = p._version            # an in-place write to the parameter invalidates the copy (see refresh_half)
            off += n
        self.grad = flat.buffer
        self.exp_avg = torch.zeros_like(self.param)
        self.exp_avg_sq = torch.zeros_like(self.param)
        self.state = torch.tensor([0.0, float(init_scale), 0.0, 0.0], dtype=torch.float32, device=dev)
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.growth_factor, self.backoff_factor = growth_factor, backoff_factor
        self.growth_interval = growth_interval if dynamic else 0

    def scale(self, loss: torch.Tensor) -> torch.Tensor:
        return loss.float() * self.state[1]

    def refresh_half(self) -> None:
        """Re-derive the fp16 copies after the parameters were written by anything but ``step`` (a loaded adapter,
        a manual edit): the kernels read the copies, and a captured step reads them without asking."""
        self.param_h.copy_(self.param)
        for p in self.params:
            p._q4_half_version = p._version

    def step(self, grad_div: float = 1.0) -> None:
        from . import _lib
        with _lib.on_device(self.param.device):
            _lib.check(_lib.lib().q4_adamw_flat(self.param.data_ptr(), self.grad.data_ptr(), self.exp_avg.data_ptr(),
                                                self.exp_avg_sq.data_ptr(), self.param.numel(), self.lr, self.betas[0], self.betas[1],
                                                self.eps, self.weight_decay, float(grad_div), self.state.data_ptr(),
                                                self.growth_factor, self.backoff_factor, self.growth_interval,
                                                self.param_h.data_ptr(), _lib.stream_of(self.param)), "adamw_flat")

    @property
    def steps_taken(self) -> int:
        return int(self.state[0].item())

    @property
    def loss_scale(self) -> float:
        return float(self.state[1].item())


class LoraFinetuner:
    """Owns the optimizer state and runs one step: forward, backward, gradient all-reduce, AdamW."""

    def __init__(self, model: nn.Module, lr: float = 3e-4, loss_scale: float = 1024.0, autocast: bool = True,
                 group=None, dynamic_scale: Optional[bool] = None, autocast_dtype: torch.dtype = torch.float16):
        self.model = model
        self.params = [p for p in model.parameters() if p.requires_grad]
        if not self.params:
            raise ValueError("model has no trainable parameters (wrap it with add_lora first)")
        self.flat = FlatGrads(self.params)
        on_gpu = self.params[0].is_cuda
        self._graph = None
        self._static_ids = None
        self._static_loss = None
        self.loss_scale = loss_scale
        self.autocast = autocast
        self.autocast_dtype = autocast_dtype
        self.group = group
        # fp16 training as the HF Trainer does it: dynamic loss scale, steps with non-finite gradients skipped
        if dynamic_scale is None:
            dynamic_scale = self.params[0].is_cuda and autocast and autocast_dtype == torch.float16
        if on_gpu:
            # one flat optimiser kernel; a static scale is a dynamic one that never moves
            self.opt = FlatAdamW(self.params, self.flat, lr=lr, init_scale=loss_scale, dynamic=bool(dynamic_scale))
            self.scaler = None
        else:
            self.opt = torch.optim.AdamW(self.params, lr=lr)
            self.scaler = None

    def capture(self, example_ids: torch.Tensor, warmup: int = 3) -> bool:
        """Record the whole step (forward, backward, gradient all-reduce, AdamW) as one CUDA graph for
        batches shaped like ``example_ids``; later ``step`` calls of that shape replay it.  The ~700
        kernel launches of the quant linears and the thousands of small framework kernels around them
        are otherwise issued one by one from Python, which is what bounds the step time.  Returns False
        (and stays on the eager path) if the step cannot be captured."""
        if not example_ids.is_cuda:
            return False
        try:
            if isinstance(self.opt, FlatAdamW):
                self.opt.refresh_half()            # the captured kernels read the fp16 copies as they are replayed
            self._static_ids = example_ids.clone()
            side = torch.cuda.Stream(device=example_ids.device)
            side.wait_stream(torch.cuda.current_stream(example_ids.device))
            with torch.cuda.stream(side):
                for _ in range(warmup):
                    self._eager_step(self._static_ids)
            torch.cuda.current_stream(example_ids.device).wait_stream(side)
            torch.cuda.synchronize(example_ids.device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self._static_loss = self._eager_step(self._static_ids)
            self._graph = graph
            return True
        except Exception as exc:                                   # capture is an optimisation, never a requirement
            print(f"finetune_step: CUDA-graph capture not possible ({type(exc).__name__}: {exc}); running eagerly")
            self._graph = None
            torch.cuda.synchronize(example_ids.device)
            return False

    def step(self, input_ids: torch.Tensor) -> torch.Tensor:
        """One optimisation step on a batch of token ids ``[B, T]`` (labels = inputs, shifted inside
        the model).  Returns the detached loss (a device scalar)."""
        if self._graph is not None and input_ids.shape == self._static_ids.shape:
            self._static_ids.copy_(input_ids, non_blocking=True)
            self._graph.replay()
            return self._static_loss
        return self._eager_step(input_ids)

    def _eager_step(self, input_ids: torch.Tensor) -> torch.Tensor:
        self.flat.zero()
        dev_type = input_ids.device.type
        with torch.autocast(device_type=dev_type, dtype=self.autocast_dtype, enabled=self.autocast and dev_type == "cuda"):
            loss = self.model(input_ids=input_ids, labels=input_ids, use_cache=False).loss
        if isinstance(self.opt, FlatAdamW):
            # fp16 training as the HF Trainer does it: dynamic loss scale, steps with non-finite gradients skipped.
            # The quant linears and the LoRA products compute in fp16 whatever the autocast dtype is, so a
            # (static) scale is applied under bf16 autocast as well.
            self.opt.scale(loss).backward()
            world = self.flat.all_reduce_sum(self.group)   # scaled gradients; an overflow on any rank reaches all
            self.opt.step(grad_div=world)                  # unscales, divides by the ranks, skips the update on inf/nan
        else:
            # The quant linears and the LoRA products compute in fp16 whatever the autocast dtype is (their
            # autograd functions cast their inputs to fp16, as the reference's do), so the gradients that
            # flow back through them want the static loss scale under bf16 autocast as well.
            scale = self.loss_scale
            (loss.float() * scale).backward()
            self.flat.buffer.div_(scale)
            self.flat.all_reduce_mean(self.group)
            self.opt.step()
        return loss.detach()


def lora_param_count(model: nn.Module) -> int:
    return sum(p.numel() for p in model.parameters() if p.requires_grad)


def quant_linear_params(model: nn.Module) -> int:
    return sum(m.in_features * m.out_features for m in model.modules() if isinstance(m, Autograd4bitQuantLinear))
