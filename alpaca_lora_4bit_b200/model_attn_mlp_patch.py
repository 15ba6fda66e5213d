"""Fused projection patches for LLaMA, with the names of the reference's ``model_attn_mlp_patch``
(model_attn_mlp_patch.py:14-335), retargeted at the installed transformers (5.x attention API).

* ``make_quant_attn`` concatenates the packed q/k/v tensors along the output dimension into one
  quant linear (one launch instead of three) and swaps every ``LlamaAttention`` for
  ``QuantLlamaAttention`` (model_attn_mlp_patch.py:73-162).  Unlike the reference the split is
  GQA-safe (q, k and v may have different widths), and fusing is refused when the three layers
  do not share ``g_idx`` (act-order checkpoints), because one fused layer has one ``g_idx``.
* ``make_fused_mlp`` does the same for gate/up (``QuantLlamaMLP``, model_attn_mlp_patch.py:165-247).
* ``inject_lora_layers`` adds a merged q/v LoRA on top of the fused qkv output
  (model_attn_mlp_patch.py:250-335); q and v updates may have different widths (grouped-query attention).
"""
from __future__ import annotations

import json
import re

import torch
import torch.nn as nn
from torch.nn import functional as F

from . import fused_ops, matmul_utils_4bit, quant_cuda
from .autograd_4bit import Autograd4bitQuantLinear


def fuse_quant_linears(layers, is_v1_model=False):
    """One ``Autograd4bitQuantLinear`` computing the concatenation of the outputs of ``layers``
    (same input width, same group size).  Packed tensors are concatenated along N and the
    sources are emptied (model_attn_mlp_patch.py:88-119,173-199)."""
    first = layers[0]
    if any(l.in_features != first.in_features or l.groupsize != first.groupsize for l in layers):
        raise ValueError("layers to fuse must share in_features and groupsize")
    out_features = sum(l.out_features for l in layers)
    fused = Autograd4bitQuantLinear(first.in_features, out_features,
                                    groupsize=-1 if is_v1_model else first.groupsize, is_v1_model=is_v1_model,
                                    bits=first.bits)
    fused.qweight = torch.cat([l.qweight for l in layers], dim=1)
    if is_v1_model:
        fused.zeros = torch.cat([l.zeros for l in layers], dim=0)
        fused.scales = torch.cat([l.scales for l in layers], dim=0)
    else:
        for l in layers[1:]:
            if not torch.equal(l.g_idx, first.g_idx):
                raise ValueError("cannot fuse layers with different g_idx (act-order): the fused layer has one g_idx")
        fused.qzeros = torch.cat([l.qzeros for l in layers], dim=1)
        fused.scales = torch.cat([l.scales for l in layers], dim=1)
        fused.g_idx = first.g_idx
    have_bias = all(l.bias is not None for l in layers)
    fused.bias = torch.cat([l.bias for l in layers], dim=0) if have_bias else None
    for l in layers:                          # free the sources
        for name in ("qweight", "qzeros", "zeros", "scales", "g_idx", "bias"):
            if name in l._buffers:
                del l._buffers[name]
    if fused.qweight.is_cuda:
        torch.cuda.empty_cache()
    return fused


class QuantLlamaAttention(nn.Module):
    """Multi-headed attention with one fused quantised qkv projection (model_attn_mlp_patch.py:14-70).

    Call signature of transformers 5.x ``LlamaAttention.forward``: rotary cos/sin arrive as
    ``position_embeddings`` and the KV cache as ``past_key_values``.
    """

    def __init__(self, config, layer_idx, qkv_proj, o_proj, q_size, kv_size):
        super().__init__()
        self.config = config
        self.layer_idx = layer_idx
        self.head_dim = getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads
        self.num_heads = config.num_attention_heads
        self.num_key_value_heads = config.num_key_value_heads
        self.num_key_value_groups = self.num_heads // self.num_key_value_heads
        self.hidden_size = config.hidden_size
        self.scaling = self.head_dim ** -0.5
        self.attention_dropout = getattr(config, "attention_dropout", 0.0)
        self.is_causal = True
        self.q_size, self.kv_size = q_size, kv_size
        self.qkv_proj = qkv_proj
        self.o_proj = o_proj

    def forward(self, hidden_states, position_embeddings=None, attention_mask=None, past_key_values=None, **kwargs):
        from transformers.models.llama.modeling_llama import apply_rotary_pos_emb
        bsz, q_len, _ = hidden_states.size()
        qkv = self.qkv_proj(hidden_states)
        q, k, v = torch.split(qkv, [self.q_size, self.kv_size, self.kv_size], dim=2)
        q = q.view(bsz, q_len, self.num_heads, self.head_dim).transpose(1, 2)
        k = k.view(bsz, q_len, self.num_key_value_heads, self.head_dim).transpose(1, 2)
        v = v.view(bsz, q_len, self.num_key_value_heads, self.head_dim).transpose(1, 2)
        cos, sin = position_embeddings
        q, k = apply_rotary_pos_emb(q, k, cos, sin)
        if past_key_values is not None:
            k, v = past_key_values.update(k, v, self.layer_idx)
        causal = attention_mask is None and q_len > 1 and k.shape[2] == q_len
        mask = attention_mask
        if mask is not None and mask.dim() == 4:
            mask = mask[:, :, :, : k.shape[2]]
        attn = F.scaled_dot_product_attention(q, k, v, attn_mask=mask, is_causal=causal, scale=self.scaling,
                                              enable_gqa=self.num_key_value_groups > 1)
        attn = attn.transpose(1, 2).reshape(bsz, q_len, -1)
        return self.o_proj(attn), None


def _replace(model, name, new):
    parent_name, _, leaf = name.rpartition('.')
    parent = model.get_submodule(parent_name) if parent_name else model
    setattr(parent, leaf, new)


def make_quant_attn(model, is_v1_model=False):
    """Replace all LlamaAttention modules with QuantLlamaAttention, fusing the q, k, v projections."""
    from transformers.models.llama.modeling_llama import LlamaAttention
    print('Turning off matmul cache ...')
    matmul_utils_4bit.cache_buffer = False
    for name, m in list(model.named_modules()):
        if not isinstance(m, LlamaAttention):
            continue
        q_size, kv_size = m.q_proj.out_features, m.k_proj.out_features
        qkv = fuse_quant_linears([m.q_proj, m.k_proj, m.v_proj], is_v1_model=is_v1_model)
        _replace(model, name, QuantLlamaAttention(m.config, m.layer_idx, qkv, m.o_proj, q_size, kv_size))


swiglu_epilogue_rows = 2048        # rows from which QuantLlamaMLP takes the SwiGLU product in the GEMM epilogue


class QuantLlamaMLP(nn.Module):
    """SwiGLU MLP with one fused quantised gate/up projection (model_attn_mlp_patch.py:165-232)."""

    def __init__(self, old_module, is_v1_model=False):
        super().__init__()
        self.intermediate_size = old_module.gate_proj.out_features
        self.gate_up_proj = fuse_quant_linears([old_module.gate_proj, old_module.up_proj], is_v1_model=is_v1_model)
        self.down_proj = old_module.down_proj
        self.act_fn = old_module.act_fn

    def _fused_product(self, x):
        """The gate/up projection with the SwiGLU product in its epilogue, where that kernel applies and pays:
        inference on ``swiglu_epilogue_rows`` rows or more (measured on LLaMA-7B/13B shapes: level with the product
        followed by the element-wise kernel at 2048 rows and without the ``[M, 2 I]`` tensor, 4 % ahead at 4096 rows,
        10 % behind at 512 rows,
        where a tile's epilogue - four warps doing the SiLU of 32768 sums - is a larger share of the tile), a 4-bit
        v2 layer, SiLU."""
        gu = self.gate_up_proj
        rows = x.numel() // x.shape[-1]
        if (torch.is_grad_enabled() and x.requires_grad) or not x.is_cuda or rows < swiglu_epilogue_rows or not matmul_utils_4bit.fused_gemm:
            return None
        if gu.is_v1_model or gu.bits != 4 or type(self.act_fn).__name__ not in ("SiLU", "SiLUActivation"):
            return None
        if not quant_cuda.gemm_swiglu_supported(gu.in_features, gu.out_features, gu.scales.shape[0]):
            return None
        x2 = x.reshape(rows, gu.in_features)
        if x2.dtype != torch.float16 or not x2.is_contiguous():
            x2 = x2.to(torch.float16).contiguous()
        out = torch.empty((rows, self.intermediate_size), dtype=torch.float16, device=x.device)
        bias = None if (gu.disable_bias or gu.bias is None) else gu.bias.half()
        quant_cuda.gemm_swiglu(x2, gu.qweight, out, gu.scales.half(), gu.qzeros, gu.g_idx, bias=bias)
        return out.reshape(x.shape[:-1] + (self.intermediate_size,)).to(x.dtype)

    def forward(self, x):
        h = self._fused_product(x)
        if h is not None:
            return self.down_proj(h)
        gu = self.gate_up_proj(x)
        if type(self.act_fn).__name__ in ("SiLU", "SiLUActivation"):
            # one kernel reads the two halves of the fused output where they lie and writes the product (and, in the
            # backward, the two halves of one gradient tensor)
            return self.down_proj(fused_ops.swiglu_fused(gu))
        gate, up = torch.split(gu, self.intermediate_size, dim=-1)
        return self.down_proj(self.act_fn(gate) * up)


def make_fused_mlp(m, parent_name='', is_v1_model=False):
    """Replace all LlamaMLP modules with QuantLlamaMLP modules (model_attn_mlp_patch.py:235-247)."""
    from transformers.models.llama.modeling_llama import LlamaMLP
    if isinstance(m, LlamaMLP):
        return QuantLlamaMLP(m, is_v1_model=is_v1_model)
    for name, child in list(m.named_children()):
        new = make_fused_mlp(child, parent_name=f"{parent_name}.{name}", is_v1_model=is_v1_model)
        if isinstance(new, QuantLlamaMLP):
            setattr(m, name, new)
    return m


class CustomLoraLayerMerged(torch.nn.Module):
    """q and v LoRA factors of one layer: ``lora_A [2, r, K]`` (pre-scaled by alpha / r) and ``lora_B``,
    stacked as ``[2, N, r]`` when q and v have the same width (model_attn_mlp_patch.py:250-259).  Under
    grouped-query attention the v projection is narrower than q: ``lora_B`` is then the pair
    ``(B_q [N_q, r], B_v [N_v, r])`` and the two products run separately.  ``forward`` returns the pair
    of updates ``(q update, v update)`` either way."""

    def __init__(self, lora_A, lora_B):
        super().__init__()
        self.lora_A = torch.nn.Parameter(lora_A, requires_grad=False)
        self.stacked = torch.is_tensor(lora_B)
        if self.stacked:
            self.lora_B = torch.nn.Parameter(lora_B, requires_grad=False)
        else:
            self.lora_B_q = torch.nn.Parameter(lora_B[0], requires_grad=False)
            self.lora_B_v = torch.nn.Parameter(lora_B[1], requires_grad=False)

    @property
    def widths(self):
        """(q width, v width) of the update."""
        return (self.lora_B.shape[1], self.lora_B.shape[1]) if self.stacked else (self.lora_B_q.shape[0], self.lora_B_v.shape[0])

    def forward(self, x):
        if self.stacked:
            return torch.einsum('bjm,ndm,nkd->nbjk', x, self.lora_A, self.lora_B)
        u = torch.einsum('bjm,ndm->nbjd', x, self.lora_A)
        return u[0] @ self.lora_B_q.t(), u[1] @ self.lora_B_v.t()


class LoraInjectionWrapper:
    """Adds the merged q/v LoRA onto the q slice (the first ``q_size`` columns) and the v slice (the last
    ``v_size`` columns) of a fused qkv output (model_attn_mlp_patch.py:262-280).  The slice widths default
    to the widths of the LoRA update itself, which is a third of the output each for multi-head attention
    and follows the narrower k/v projections under grouped-query attention."""

    def __init__(self, module, lora_layer, q_size=None, v_size=None):
        self.module = module
        self.lora_layer = lora_layer
        widths = lora_layer.widths if hasattr(lora_layer, 'widths') else (module.out_features // 3,) * 2
        self.q_size = q_size if q_size is not None else widths[0]
        self.v_size = v_size if v_size is not None else widths[1]

    def apply(self):
        self.module.forward_before_lora = self.module.forward
        self.module.forward = self.forward_with_lora
        self.module.is_lora_injected = True

    def forward_with_lora(self, x):
        result = self.module.forward_before_lora(x)
        lora_out = self.lora_layer(x)
        result[:, :, :self.q_size] += lora_out[0]
        result[:, :, -self.v_size:] += lora_out[1]
        return result


def _read_adapter_weights(lora_path):
    """``adapter_model.bin`` (PEFT <= 0.6, what the reference reads) or ``adapter_model.safetensors``."""
    import os
    bin_path = os.path.join(lora_path, 'adapter_model.bin')
    if os.path.exists(bin_path):
        return torch.load(bin_path, map_location='cpu')
    from safetensors.torch import load_file
    return load_file(os.path.join(lora_path, 'adapter_model.safetensors'))


def inject_lora_layers(model, lora_path, device='cuda', dtype=torch.float16):
    """Load a PEFT adapter (``adapter_config.json`` + ``adapter_model.bin``) and inject its q/v LoRA
    into every fused ``qkv_proj`` (model_attn_mlp_patch.py:283-335)."""
    print('Device: {}, dtype: {}'.format(device, dtype))
    with open(lora_path + '/adapter_config.json', 'r') as file:
        lora_config = json.load(file)
    scaling = lora_config['lora_alpha'] / lora_config['r']
    per_layer = {}
    for key, value in _read_adapter_weights(lora_path).items():
        key = key.replace('base_model.model.', '').replace('.default.weight', '.weight')
        prefix = re.findall(r'^model\.layers\.\d+\.', key)[0]
        per_layer.setdefault(prefix, {})[key.replace(prefix, '')] = value
    lora_layers = {}
    for prefix, w in per_layer.items():
        a = torch.stack([w['self_attn.q_proj.lora_A.weight'], w['self_attn.v_proj.lora_A.weight']]).to(device=device, dtype=dtype)
        bq = w['self_attn.q_proj.lora_B.weight'].to(device=device, dtype=dtype)
        bv = w['self_attn.v_proj.lora_B.weight'].to(device=device, dtype=dtype)
        b = torch.stack([bq, bv]) if bq.shape == bv.shape else (bq, bv)       # unequal under grouped-query attention
        lora_layers[prefix] = CustomLoraLayerMerged(a * scaling, b).to(device=device, dtype=dtype)
    wrappers = []
    for n, m in model.named_modules():
        if 'qkv_proj' in n and isinstance(m, Autograd4bitQuantLinear):
            if getattr(m, 'is_lora_injected', False):
                m.forward = m.forward_before_lora
            prefix = re.findall(r'^model\.layers\.\d+\.', n)[0]
            q_size, v_size = lora_layers[prefix].widths
            wrapper = LoraInjectionWrapper(m, lora_layers[prefix], q_size=q_size, v_size=v_size)
            wrapper.apply()
            wrappers.append(wrapper)
    print('Lora Injected.')
    return wrappers
