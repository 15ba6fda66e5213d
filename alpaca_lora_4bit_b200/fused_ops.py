"""Fused element-wise operators of a LLaMA decoder layer on the sm_100a library, with autograd: RMSNorm,
the SwiGLU product and the rotary embedding, each one kernel forward and one backward instead of the
half-dozen framework kernels of the stock modules (``LlamaRMSNorm.forward``, ``LlamaMLP.forward``,
``apply_rotary_pos_emb`` of transformers, which the reference's finetune step runs unchanged around its
quant linears, finetune.py:150-175).

``patch_llama(model)`` re-routes the three in a transformers LLaMA.  Every operator takes the fused path
only for fp16 CUDA tensors of a supported shape and otherwise falls back to the stock computation, so a
patched model still runs (and is tested) on the CPU.  The norm weight and the rotary tables are treated as
constants in the backward: in a LoRA finetune only the LoRA factors train.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib


def _fusable(*tensors) -> bool:
    return all(t.is_cuda and t.dtype == torch.float16 for t in tensors)


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows, H = x2.shape
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        with _lib.on_device(x.device):
            _lib.check(_lib.lib().q4_rmsnorm_fwd(x2.data_ptr(), weight.data_ptr(), y.data_ptr(), rstd.data_ptr(), rows, H, float(eps),
                                                 _lib.stream_of(x2)), "rmsnorm")
        ctx.save_for_backward(x2, weight, rstd)
        ctx.shape = x.shape
        return y.reshape(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, weight, rstd = ctx.saved_tensors
        rows, H = x2.shape
        g = dy.reshape(rows, H)
        if g.dtype != torch.float16 or not g.is_contiguous():
            g = g.half().contiguous()
        dx = torch.empty_like(x2)
        with _lib.on_device(x2.device):
            _lib.check(_lib.lib().q4_rmsnorm_bwd(g.data_ptr(), x2.data_ptr(), weight.data_ptr(), rstd.data_ptr(), dx.data_ptr(), rows, H,
                                                 _lib.stream_of(x2)), "rmsnorm_bwd")
        return dx.reshape(ctx.shape), None, None


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``weight * (x * rsqrt(mean(x^2) + eps)).to(x.dtype)`` as ``LlamaRMSNorm.forward`` computes it."""
    H = x.shape[-1]
    if _fusable(x, weight) and not weight.requires_grad and H % 8 == 0 and H <= 8192 and x.numel() > 0:
        return _RMSNorm.apply(x, weight if weight.is_contiguous() else weight.contiguous(), eps)
    h = x.to(torch.float32)
    h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)
    return weight * h.to(x.dtype)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up):
        I = gate.shape[-1]
        g2, u2 = gate.reshape(-1, I), up.reshape(-1, I)
        pitch = g2.stride(0)
        out = torch.empty((g2.shape[0], I), dtype=torch.float16, device=gate.device)
        with _lib.on_device(gate.device):
            _lib.check(_lib.lib().q4_swiglu_fwd(g2.data_ptr(), u2.data_ptr(), out.data_ptr(), g2.shape[0], I, pitch, _lib.stream_of(gate)),
                       "swiglu")
        ctx.save_for_backward(g2, u2)
        ctx.shape = gate.shape
        return out.reshape(gate.shape)

    @staticmethod
    def backward(ctx, dout):
        g2, u2 = ctx.saved_tensors
        rows, I = g2.shape
        d = dout.reshape(rows, I)
        if d.dtype != torch.float16 or not d.is_contiguous():
            d = d.half().contiguous()
        dg, du = torch.empty((rows, I), dtype=torch.float16, device=d.device), torch.empty((rows, I), dtype=torch.float16, device=d.device)
        with _lib.on_device(d.device):
            _lib.check(_lib.lib().q4_swiglu_bwd(d.data_ptr(), g2.data_ptr(), u2.data_ptr(), dg.data_ptr(), du.data_ptr(), rows, I,
                                                g2.stride(0), I, _lib.stream_of(d)), "swiglu_bwd")
        return dg.reshape(ctx.shape), du.reshape(ctx.shape)


class _SwiGLUFused(torch.autograd.Function):
    """``silu(gu[..., :I]) * gu[..., I:]`` on one fused gate_up output: the backward writes both halves of one
    gradient tensor, so nothing concatenates them afterwards."""

    @staticmethod
    def forward(ctx, gu):
        I = gu.shape[-1] // 2
        g2 = gu.reshape(-1, 2 * I)
        out = torch.empty((g2.shape[0], I), dtype=torch.float16, device=gu.device)
        with _lib.on_device(gu.device):
            _lib.check(_lib.lib().q4_swiglu_fwd(g2.data_ptr(), g2.data_ptr() + 2 * I, out.data_ptr(), g2.shape[0], I, 2 * I,
                                                _lib.stream_of(gu)), "swiglu")
        ctx.save_for_backward(g2)
        ctx.shape = gu.shape
        return out.reshape(gu.shape[:-1] + (I,))

    @staticmethod
    def backward(ctx, dout):
        (g2,) = ctx.saved_tensors
        rows, I = g2.shape[0], g2.shape[1] // 2
        d = dout.reshape(rows, I)
        if d.dtype != torch.float16 or not d.is_contiguous():
            d = d.half().contiguous()
        dgu = torch.empty((rows, 2 * I), dtype=torch.float16, device=d.device)
        with _lib.on_device(d.device):
            _lib.check(_lib.lib().q4_swiglu_bwd(d.data_ptr(), g2.data_ptr(), g2.data_ptr() + 2 * I, dgu.data_ptr(), dgu.data_ptr() + 2 * I,
                                                rows, I, 2 * I, 2 * I, _lib.stream_of(d)), "swiglu_bwd")
        return dgu.reshape(ctx.shape)


def swiglu_fused(gu: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for ``gu = [gate | up]`` along the last dimension (the output of a fused gate_up
    projection); falls back to ``swiglu`` on the two halves where the kernel does not apply."""
    I = gu.shape[-1] // 2
    if _fusable(gu) and gu.shape[-1] == 2 * I and I % 8 == 0 and gu.numel() > 0 and gu.is_contiguous() and gu.data_ptr() % 16 == 0:
        return _SwiGLUFused.apply(gu)
    gate, up = torch.split(gu, I, dim=-1)
    return swiglu(gate, up)


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` (the product inside ``LlamaMLP.forward``); ``gate`` and ``up`` may be the two halves of
    one fused gate_up output (rows of a common pitch)."""
    I = gate.shape[-1]
    ok = (_fusable(gate, up) and gate.shape == up.shape and I % 8 == 0 and gate.numel() > 0 and gate.stride(-1) == 1 and up.stride(-1) == 1)
    if ok:
        g2, u2 = gate.reshape(-1, I), up.reshape(-1, I)             # views for the halves of a fused output
        ok = g2.stride(0) == u2.stride(0) and g2.stride(0) % 8 == 0 and g2.data_ptr() % 16 == 0 and u2.data_ptr() % 16 == 0
    if ok:
        return _SwiGLU.apply(gate, up)
    return F.silu(gate) * up


class _Rope(torch.autograd.Function):
    """Rotary embedding of a ``[B, heads, T, D]`` view of a projection output ``[B, T, heads * D]``."""

    @staticmethod
    def forward(ctx, t, cos, sin):
        B, Hh, T, D = t.shape
        src = t.transpose(1, 2)                                   # [B, T, heads, D], the memory order of the projection
        if not src.is_contiguous():
            src = src.contiguous()
        out = torch.empty((B, T, Hh, D), dtype=torch.float16, device=t.device)
        with _lib.on_device(t.device):
            _lib.check(_lib.lib().q4_rope(src.data_ptr(), cos.data_ptr(), sin.data_ptr(), out.data_ptr(), B * T, Hh, D, Hh * D, cos.shape[0] * cos.shape[1], 0,
                                          _lib.stream_of(t)), "rope")
        ctx.save_for_backward(cos, sin)
        return out.transpose(1, 2)

    @staticmethod
    def backward(ctx, g):
        cos, sin = ctx.saved_tensors
        B, Hh, T, D = g.shape
        src = g.transpose(1, 2)
        if src.dtype != torch.float16 or not src.is_contiguous():
            src = src.half().contiguous()
        out = torch.empty((B, T, Hh, D), dtype=torch.float16, device=g.device)
        with _lib.on_device(g.device):
            _lib.check(_lib.lib().q4_rope(src.data_ptr(), cos.data_ptr(), sin.data_ptr(), out.data_ptr(), B * T, Hh, D, Hh * D, cos.shape[0] * cos.shape[1], 1,
                                          _lib.stream_of(g)), "rope_bwd")
        return out.transpose(1, 2), None, None


def _rotate_half(x):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def apply_rotary_pos_emb(q, k, cos, sin, unsqueeze_dim=1):
    """Drop-in for transformers' ``apply_rotary_pos_emb`` (``q``, ``k`` ``[B, heads, T, D]``, ``cos`` / ``sin``
    ``[B, T, D]``)."""
    D = q.shape[-1]
    if (unsqueeze_dim == 1 and q.dim() == 4 and _fusable(q, k, cos, sin) and cos.dim() == 3 and cos.shape[0] in (1, q.shape[0])
            and cos.shape[1] == q.shape[2] and cos.shape[2] == D and sin.shape == cos.shape and D % 16 == 0 and not cos.requires_grad and q.numel() > 0):
        c = cos if cos.is_contiguous() else cos.contiguous()
        s = sin if sin.is_contiguous() else sin.contiguous()
        return _Rope.apply(q, c, s), _Rope.apply(k, c, s)
    cos = cos.unsqueeze(unsqueeze_dim)
    sin = sin.unsqueeze(unsqueeze_dim)
    return (q * cos) + (_rotate_half(q) * sin), (k * cos) + (_rotate_half(k) * sin)


def _decoder_layer_forward(layer):
    """``LlamaDecoderLayer.forward`` with the two skip-path adds handed to the projections that end the blocks
    (``o_proj``, ``down_proj``): a quant linear that was offered the residual returns ``projection + residual``,
    from its GEMM's epilogue where the fused kernel runs.  A projection that is not a quant linear, or a block that
    never called it, leaves the add here."""
    from .autograd_4bit import Autograd4bitQuantLinear

    def closing(block, name):
        proj = getattr(block, name, None)
        return proj if isinstance(proj, Autograd4bitQuantLinear) else None

    def forward(hidden_states, attention_mask=None, position_ids=None, past_key_values=None, use_cache=False,
                position_embeddings=None, **kwargs):
        residual = hidden_states
        hidden_states = layer.input_layernorm(hidden_states)
        proj = closing(layer.self_attn, "o_proj")
        if proj is not None:
            proj.offer_residual(residual)
        hidden_states, _ = layer.self_attn(hidden_states=hidden_states, attention_mask=attention_mask, position_ids=position_ids,
                                           past_key_values=past_key_values, use_cache=use_cache,
                                           position_embeddings=position_embeddings, **kwargs)
        if proj is None or proj.take_residual() is not None:          # not taken: the add is still owed
            hidden_states = residual + hidden_states
        residual = hidden_states
        hidden_states = layer.post_attention_layernorm(hidden_states)
        proj = closing(layer.mlp, "down_proj")
        if proj is not None:
            proj.offer_residual(residual)
        hidden_states = layer.mlp(hidden_states)
        if proj is None or proj.take_residual() is not None:
            hidden_states = residual + hidden_states
        return hidden_states

    return forward


def _fuse_gate_up(model: nn.Module) -> int:
    """Replace every ``LlamaMLP`` whose gate and up projections are plain 4-bit quant linears with the same group
    layout (no adapters on them) by ``QuantLlamaMLP`` - the reference's fused inference MLP
    (model_attn_mlp_patch.py:165-247), which trains as well: one product of 2 I columns forward, one product over a
    contraction of 2 I backward (the sum of the two input gradients happens in the accumulator), the SwiGLU kernel
    reading and writing the halves of the fused tensor in place.  Returns the number of MLPs replaced."""
    from transformers.models.llama import modeling_llama as ml
    from .autograd_4bit import Autograd4bitQuantLinear
    from . import model_attn_mlp_patch as patch
    done = 0
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            if not isinstance(child, ml.LlamaMLP):
                continue
            g, u = getattr(child, "gate_proj", None), getattr(child, "up_proj", None)
            if type(g) is not Autograd4bitQuantLinear or type(u) is not Autograd4bitQuantLinear:
                continue
            if g.is_v1_model or u.is_v1_model or g.bits != 4 or u.bits != 4 or g.groupsize != u.groupsize or not torch.equal(g.g_idx, u.g_idx):
                continue
            setattr(parent, name, patch.QuantLlamaMLP(child))
            done += 1
    return done


def patch_llama(model: nn.Module, fuse_gate_up: bool = False) -> nn.Module:
    """Route the RMSNorms, the SwiGLU products, the rotary embedding and the skip-path adds of a transformers LLaMA
    through the fused operators above.  The norm, MLP and decoder-layer modules are patched per instance; the rotary
    function is a module-level name of ``transformers.models.llama.modeling_llama`` and is replaced there (the
    replacement computes exactly the stock expression whenever the fused path does not apply).  Call it before
    anything wraps the layers' ``forward`` (gradient checkpointing).  ``fuse_gate_up`` also concatenates the gate
    and up projections of every MLP that carries no adapter on them (``_fuse_gate_up``; the packed tensors of the
    two layers are copied into one and the sources freed)."""
    from transformers.models.llama import modeling_llama as ml
    if fuse_gate_up:
        _fuse_gate_up(model)
    for mod in model.modules():
        if isinstance(mod, ml.LlamaDecoderLayer) and "forward" not in mod.__dict__:
            mod.forward = _decoder_layer_forward(mod)
    for mod in model.modules():
        if isinstance(mod, ml.LlamaRMSNorm):
            mod.forward = (lambda h, _m=mod: rms_norm(h, _m.weight, _m.variance_epsilon))
        elif isinstance(mod, ml.LlamaMLP) and type(getattr(mod, "act_fn", None)).__name__ in ("SiLU", "SiLUActivation"):
            mod.forward = (lambda x, _m=mod: _m.down_proj(swiglu(_m.gate_proj(x), _m.up_proj(x))))
    ml.apply_rotary_pos_emb = apply_rotary_pos_emb
    return model
