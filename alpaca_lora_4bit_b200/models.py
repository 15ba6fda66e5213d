"""LoRA on top of the quantised linear: ``Linear4bitLt`` and the PEFT hooks, with the names of
the reference's ``models.py`` (models.py:13-163).

``Linear4bitLt(adapter_name, in_features, out_features, groupsize, is_v1_model, r, lora_alpha,
lora_dropout)`` computes ``base(x) + lora_B(lora_A(dropout(x))) * (lora_alpha / r)`` per active
adapter (models.py:51-69) and exposes PEFT 0.6's ``LoraLayer`` attributes (``lora_A``, ``lora_B``,
``lora_dropout``, ``scaling``, ``r``, ``lora_alpha``, ``active_adapters``, ``disable_adapters``,
``update_layer``, ``set_adapter``).  When ``peft`` is importable the class derives from its
``LoraLayer``; otherwise from a small structural twin with the same attributes, so the layer
works (and is tested) without PEFT installed.  ``GPTQLoraModel`` needs PEFT and is resolved
lazily on attribute access.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.amp import custom_bwd, custom_fwd

from . import _lib
from . import matmul_utils_4bit as mm4b
from . import quant_cuda
from .autograd_4bit import Autograd4bitQuantLinear

fused_lora = True      # base product and LoRA term in one kernel when the layer and input allow it

try:  # PEFT is optional
    from peft.tuners.lora import LoraLayer as _PeftLoraLayer  # type: ignore
    _HAVE_PEFT = True
except Exception:  # pragma: no cover - depends on the environment
    _PeftLoraLayer = None
    _HAVE_PEFT = False


class LoraLayerTwin:
    """Attribute-compatible stand-in for ``peft.tuners.lora.LoraLayer`` (PEFT 0.6)."""

    def __init__(self, in_features: int, out_features: int, **kwargs):
        self.r = {}
        self.lora_alpha = {}
        self.scaling = {}
        self.lora_dropout = nn.ModuleDict({})
        self.lora_A = nn.ModuleDict({})
        self.lora_B = nn.ModuleDict({})
        self._disable_adapters = False
        self._active_adapter = []
        self.merged_adapters = []
        self.in_features = in_features
        self.out_features = out_features

    @property
    def disable_adapters(self) -> bool:
        return self._disable_adapters

    @property
    def active_adapters(self):
        a = self._active_adapter
        return [a] if isinstance(a, str) else list(a)

    @property
    def active_adapter(self):
        return self._active_adapter

    def update_layer(self, adapter_name, r, lora_alpha, lora_dropout, init_lora_weights):
        if r <= 0:
            raise ValueError(f"`r` should be a positive integer value but the value passed is {r}")
        self.r[adapter_name] = r
        self.lora_alpha[adapter_name] = lora_alpha
        self.lora_dropout[adapter_name] = nn.Dropout(p=lora_dropout) if lora_dropout > 0.0 else nn.Identity()
        self.lora_A[adapter_name] = nn.Linear(self.in_features, r, bias=False)
        self.lora_B[adapter_name] = nn.Linear(r, self.out_features, bias=False)
        self.scaling[adapter_name] = lora_alpha / r
        if init_lora_weights:
            nn.init.kaiming_uniform_(self.lora_A[adapter_name].weight, a=math.sqrt(5))
            nn.init.zeros_(self.lora_B[adapter_name].weight)

    def set_adapter(self, adapter_names):
        if isinstance(adapter_names, str):
            adapter_names = [adapter_names]
        for name, layer in list(self.lora_A.items()) + list(self.lora_B.items()):
            layer.requires_grad_(name in adapter_names)
        self._active_adapter = list(adapter_names)

    def enable_adapters(self, enabled: bool):
        self._disable_adapters = not enabled
        for name, layer in list(self.lora_A.items()) + list(self.lora_B.items()):
            layer.requires_grad_(enabled and name in self.active_adapters)


_LoraBase = _PeftLoraLayer if _HAVE_PEFT else LoraLayerTwin


def _lora_project(x2: torch.Tensor, w: torch.Tensor, scaling: float) -> torch.Tensor:
    """``scaling * x2 @ w.T`` as the zero-padded fp16 ``[M, 64]`` operand of the fused GEMM's LoRA stage
    (``x2`` fp16 ``[M, C]``, ``w`` fp16 ``[r, C]``, both contiguous)."""
    out = torch.empty((x2.shape[0], 64), dtype=torch.float16, device=x2.device)
    with _lib.on_device(x2.device):
        _lib.check(_lib.lib().q4_lora_project(x2.data_ptr(), w.data_ptr(), out.data_ptr(), x2.shape[0], x2.shape[1], w.shape[0],
                                              float(scaling), _lib.stream_of(x2)), "lora_project")
    return out


def _half_of(p: torch.Tensor) -> torch.Tensor:
    """fp16 contiguous copy of a LoRA factor: the copy its optimiser keeps beside it (``_q4_half``, refreshed by the
    flat AdamW kernel) when there is one, else a cast."""
    h = getattr(p, "_q4_half", None)
    if h is not None and h.shape == p.shape and h.device == p.device and getattr(p, "_q4_half_version", -1) == p._version:
        return h
    return p.detach().to(torch.float16).contiguous()


class LoraMatmul4bit(torch.autograd.Function):
    """``y = x @ W + bias + scaling * (x @ A^T) @ B^T`` over a 4-bit v2 layer in one fused kernel, with
    the matching backward ``dx = dy @ W^T + scaling * (dy @ B) @ A`` (also one kernel) and the LoRA
    gradients ``dA = (scaling * dy @ B)^T @ x``, ``dB = dy^T @ (scaling * x @ A^T)``.

    Same mathematics as ``Autograd4bitQuantLinear.forward`` followed by the adapter update of
    ``Linear4bitLt.forward`` (models.py:51-69).  The rank-r activations ``u = scaling * x A^T`` and
    ``v = scaling * dy B`` come from ``q4_lora_project`` (one read of x or dy, written in the padded form
    the GEMM kernels take), everything N- or K-wide runs inside the dequant-GEMM kernels, and one
    ``q4_lora_grads`` launch produces both gradients in the factors' own dtype (fp32 for fresh PEFT
    adapters) instead of fp16 products cast back by autograd."""

    @staticmethod
    @custom_fwd(device_type="cuda")
    def forward(ctx, x, lora_a, lora_b, scaling, qweight, scales, qzeros, g_idx, bias, residual=None):
        K, N = qweight.shape[0] * 8, qweight.shape[1]
        x2 = x.reshape(-1, K)
        if x2.dtype != torch.float16 or not x2.is_contiguous():
            x2 = x2.to(torch.float16).contiguous()
        a_h, b_h = _half_of(lora_a), _half_of(lora_b)                            # [r, K], [N, r]
        u = _lora_project(x2, a_h, scaling)                                      # [M, 64], scaling folded in
        y = torch.empty((x2.shape[0], N), dtype=torch.float16, device=x.device)
        res2 = None
        if residual is not None and residual.dtype == torch.float16 and residual.numel() == y.numel():
            res2 = residual.reshape(y.shape)
            res2 = res2 if res2.is_contiguous() else None
        quant_cuda.gemm(x2, qweight, y, scales.half(), qzeros, g_idx, bias=None if bias is None else bias.half(),
                        lora_u=u, lora_w=b_h, residual=res2)
        if residual is not None and res2 is None:
            y = y + residual.reshape(y.shape).to(y.dtype)
        ctx.save_for_backward(x2, u, lora_a, lora_b, qweight, scales, qzeros, g_idx)
        ctx.scaling = scaling
        ctx.x_shape = x.shape
        ctx.x_dtype = x.dtype
        return y.reshape(x.shape[:-1] + (N,))

    @staticmethod
    @custom_bwd(device_type="cuda")
    def backward(ctx, grad_output):
        x2, u, lora_a, lora_b, qweight, scales, qzeros, g_idx = ctx.saved_tensors
        K, N = qweight.shape[0] * 8, qweight.shape[1]
        r = lora_a.shape[0]
        dy = grad_output.reshape(-1, N)
        if dy.dtype != torch.float16 or not dy.is_contiguous():
            dy = dy.to(torch.float16).contiguous()
        M = dy.shape[0]
        # v = scaling * dy @ B: the projection kernel wants its small operand as [r, N]
        bt_h = _half_of(lora_b).t().contiguous()
        v = _lora_project(dy, bt_h, ctx.scaling)
        dx = d_a = d_b = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty((M, K), dtype=torch.float16, device=dy.device)
            quant_cuda.gemm(dy, qweight, dx, scales.half(), qzeros, g_idx, transpose=True,
                            lora_u=v, lora_w=_half_of(lora_a))
            dx = dx.reshape(ctx.x_shape).to(ctx.x_dtype)
        want_a, want_b = ctx.needs_input_grad[1], ctx.needs_input_grad[2]
        if want_a or want_b:
            ga = torch.empty((r, K), dtype=torch.float32, device=dy.device) if want_a else None
            gb = torch.empty((N, r), dtype=torch.float32, device=dy.device) if want_b else None
            with _lib.on_device(dy.device):
                _lib.check(_lib.lib().q4_lora_grads(v.data_ptr(), x2.data_ptr(), ga.data_ptr() if want_a else None, K,
                                                    dy.data_ptr(), u.data_ptr(), gb.data_ptr() if want_b else None, N,
                                                    M, r, _lib.stream_of(dy)), "lora_grads")
            d_a = ga.to(lora_a.dtype) if want_a else None
            d_b = gb.to(lora_b.dtype) if want_b else None
        d_res = grad_output if (len(ctx.needs_input_grad) > 9 and ctx.needs_input_grad[9]) else None
        return (dx, d_a, d_b, None, None, None, None, None, None, d_res)[:max(len(ctx.needs_input_grad), 9)]


class Linear4bitLt(Autograd4bitQuantLinear, _LoraBase):
    """LoRA implemented on a 4-bit quantised dense layer (models.py:13-76)."""

    def __init__(self, adapter_name, in_features, out_features, groupsize: int = -1, is_v1_model: bool = False,
                 r: int = 0, lora_alpha: int = 1, lora_dropout: float = 0.0, **kwargs):
        Autograd4bitQuantLinear.__init__(self, in_features, out_features, groupsize, is_v1_model)
        _LoraBase.__init__(self, in_features=in_features, out_features=out_features)
        # the packed base weight is frozen; only the LoRA factors train
        for t in (self.qweight, self.scales, self.bias):
            t.requires_grad = False
        if self.is_v1_model:
            self.zeros.requires_grad = False
        else:
            self.qzeros.requires_grad = False
            self.g_idx.requires_grad = False
        init_lora_weights = kwargs.pop("init_lora_weights", True)
        self.update_layer(adapter_name, r, lora_alpha, lora_dropout, init_lora_weights)
        self.set_adapter([adapter_name])

    def _fused_adapter(self, x: torch.Tensor):
        """Name of the one adapter the fused kernel can serve for this call, else None."""
        if not (fused_lora and mm4b.fused_gemm) or self.disable_adapters or self.is_v1_model or self.bits != 4:
            return None
        active = [n for n in self.active_adapters if n in self.lora_A.keys()]
        if len(active) != 1 or not x.is_cuda or not torch.is_grad_enabled():
            return None
        name = active[0]
        drop = self.lora_dropout[name]
        if isinstance(drop, nn.Dropout) and drop.p > 0 and self.training:
            return None                                   # the LoRA branch would see a different x
        rows = x.numel() // x.shape[-1]
        if rows <= mm4b.auto_switch_thd or self.r[name] > 64:
            return None
        if not quant_cuda.gemm_supported(self.in_features, self.out_features, self.scales.shape[0], False):
            return None
        return name

    def forward(self, x: torch.Tensor):
        residual = self.take_residual()                   # left by a patched decoder layer: this call returns projection + residual
        name = self._fused_adapter(x)
        if name is not None:
            bias = None if (self.disable_bias or self.bias is None) else self.bias
            return LoraMatmul4bit.apply(x, self.lora_A[name].weight, self.lora_B[name].weight, self.scaling[name],
                                        self.qweight, self.scales, self.qzeros, self.g_idx, bias, residual)
        result = Autograd4bitQuantLinear._forward(self, x, None)
        if residual is not None:
            result = result + residual.to(result.dtype)
        if self.disable_adapters:
            return result
        previous_dtype = result.dtype
        for name in self.active_adapters:
            if name not in self.lora_A.keys():
                continue
            a, b = self.lora_A[name], self.lora_B[name]
            xa = self.lora_dropout[name](x.to(a.weight.dtype))
            result = result + b(a(xa)) * self.scaling[name]
        return result.to(previous_dtype)

    @property
    def weight(self):
        """PEFT probes ``.weight.device`` / ``.dtype``; answer with the packed tensor's."""
        class _WeightInfo:
            device = self.qweight.device
            dtype = self.qweight.dtype
        return _WeightInfo()


def _gptq_lora_model():
    """Build ``GPTQLoraModel`` (needs PEFT): a ``LoraModel`` whose module factory wraps quant linears
    in ``Linear4bitLt`` and re-points the packed buffers instead of copying (models.py:79-137)."""
    from peft.tuners import lora
    from peft.tuners.lora import Linear

    class GPTQLoraModel(lora.LoraModel):
        @staticmethod
        def _create_new_module(lora_config, adapter_name, target, **kwargs):
            bias = kwargs.pop("bias", False)
            if isinstance(target, Autograd4bitQuantLinear):
                return Linear4bitLt(adapter_name, target.in_features, target.out_features, target.groupsize,
                                    target.is_v1_model, bias=bias, **kwargs)
            if isinstance(target, torch.nn.Linear):
                if kwargs.get("fan_in_fan_out"):
                    kwargs["fan_in_fan_out"] = lora_config.fan_in_fan_out = False
                return Linear(adapter_name, target.in_features, target.out_features, bias=bias, **kwargs)
            raise ValueError(f"Target module {target} is not supported.")

        @staticmethod
        def _replace_module(parent, child_name, new_module, child):
            setattr(parent, child_name, new_module)
            if isinstance(child, Autograd4bitQuantLinear) and isinstance(new_module, Linear4bitLt):
                adopt_packed_buffers(new_module, child)
                device = child.qweight.device
            else:
                child = getattr(child, "base_layer", child)
                if not hasattr(new_module, "base_layer"):
                    new_module.weight = child.weight
                    if hasattr(child, "bias"):
                        new_module.bias = child.bias
                device = child.weight.device
            for name, module in new_module.named_modules():
                if "lora_" in name or "ranknum" in name:
                    module.to(device)

    return GPTQLoraModel


def adopt_packed_buffers(new_module: Linear4bitLt, child: Autograd4bitQuantLinear) -> None:
    """Alias (not copy) the packed tensors of ``child`` into ``new_module`` (models.py:117-129)."""
    new_module.qweight = child.qweight
    new_module.scales = child.scales
    if child.is_v1_model:
        new_module.zeros = child.zeros
    else:
        new_module.qzeros = child.qzeros
        new_module.g_idx = child.g_idx
    new_module.bias = child.bias
    device = child.qweight.device
    for name, module in new_module.named_modules():
        if "lora_" in name:
            module.to(device)


def wrap_with_lora(model: nn.Module, target_modules, r: int, lora_alpha: int, lora_dropout: float = 0.0,
                   adapter_name: str = "default", init_lora_weights: bool = True) -> nn.Module:
    """PEFT-free equivalent of ``get_peft_model(model, LoraConfig(target_modules=...))`` for quant
    linears: every ``Autograd4bitQuantLinear`` whose name ends with one of ``target_modules`` becomes a
    ``Linear4bitLt`` sharing its packed buffers; all other parameters are frozen."""
    for p in model.parameters():
        p.requires_grad_(False)
    for name, mod in list(model.named_modules()):
        if isinstance(mod, Autograd4bitQuantLinear) and not isinstance(mod, Linear4bitLt) \
                and any(name == t or name.endswith("." + t) for t in target_modules):
            new = Linear4bitLt(adapter_name, mod.in_features, mod.out_features, mod.groupsize, mod.is_v1_model,
                               r=r, lora_alpha=lora_alpha, lora_dropout=lora_dropout,
                               init_lora_weights=init_lora_weights)
            adopt_packed_buffers(new, mod)
            parent_name, _, leaf = name.rpartition(".")
            parent = model.get_submodule(parent_name) if parent_name else model
            setattr(parent, leaf, new)
    return model


def __getattr__(name):
    if name == "GPTQLoraModel":
        return _gptq_lora_model()
    raise AttributeError(name)
