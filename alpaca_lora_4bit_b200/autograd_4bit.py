"""Quantised linear module and its autograd functions, with the public names of the reference's
``autograd_4bit`` (autograd_4bit.py:32-255).

``Autograd4bitQuantLinear`` holds the packed GPTQ buffers under the reference's state-dict names
(``qweight``, ``qzeros``/``zeros``, ``scales``, ``g_idx``, ``bias``) and routes like the reference
(autograd_4bit.py:192-208): with grad enabled through ``AutogradMatmul4bit`` (forward ``x @ W``,
backward ``dy @ W.T``, nothing but the four packed tensors saved), otherwise through
``matmul4bit_with_backend``.  There is one backend, the sm_100a library: ``switch_backend_to('cuda')``
is accepted, ``'triton'`` is refused.
"""
from __future__ import annotations

import logging
import math
import time

import torch
import torch.nn as nn
from torch.amp import custom_bwd, custom_fwd

from . import matmul_utils_4bit as mm4b

gptq_backend_loaded = True
triton_backend_loaded = False


class AutogradMatmul4bitNotImplemented(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, qweight, scales, zeros, g_idx, bits, maxq):
        raise NotImplementedError()

    @staticmethod
    def backward(ctx, grad_output):
        raise NotImplementedError()


class AutogradMatmul4bitCuda(torch.autograd.Function):
    """``y = x @ W`` over a 4-bit layer; ``g_idx is None`` marks a v1 layer (autograd_4bit.py:32-54).

    Inputs are cast to fp16 under autocast exactly as the reference's ``custom_fwd`` does.
    Unlike the reference, ``backward`` returns ``None`` for ``x`` when it needs no gradient
    instead of failing on an unbound name (autograd_4bit.py:49-54).
    """

    @staticmethod
    @custom_fwd(device_type="cuda", cast_inputs=torch.float16)
    def forward(ctx, x, qweight, scales, zeros, g_idx, bits, maxq):
        ctx.save_for_backward(qweight, scales, zeros, g_idx)
        if g_idx is None:
            return mm4b._matmul4bit_v1_recons(x, qweight, scales, zeros)
        return mm4b._matmul4bit_v2_recons(x, qweight, scales, zeros, g_idx)

    @staticmethod
    @custom_bwd(device_type="cuda")
    def backward(ctx, grad_output):
        qweight, scales, zeros, g_idx = ctx.saved_tensors
        grad = None
        if ctx.needs_input_grad[0]:
            if g_idx is None:
                grad = mm4b._matmul4bit_v1_recons(grad_output, qweight, scales, zeros, transpose=True)
            else:
                grad = mm4b._matmul4bit_v2_recons(grad_output, qweight, scales, zeros, g_idx, transpose=True)
        return grad, None, None, None, None, None, None


class AutogradMatmul2bitCuda(torch.autograd.Function):
    """2-bit twin (autograd_4bit.py:56-72)."""

    @staticmethod
    @custom_fwd(device_type="cuda", cast_inputs=torch.float16)
    def forward(ctx, x, qweight, scales, zeros, g_idx, bits, maxq):
        ctx.save_for_backward(qweight, scales, zeros, g_idx)
        return mm4b._matmul2bit_v2_recons(x, qweight, scales, zeros, g_idx)

    @staticmethod
    @custom_bwd(device_type="cuda")
    def backward(ctx, grad_output):
        qweight, scales, zeros, g_idx = ctx.saved_tensors
        grad = None
        if ctx.needs_input_grad[0]:
            grad = mm4b._matmul2bit_v2_recons(grad_output, qweight, scales, zeros, g_idx, transpose=True)
        return grad, None, None, None, None, None, None


def is_triton_backend_available():
    return False


def is_gptq_backend_available():
    return True


AutogradMatmul4bit = AutogradMatmul4bitCuda
AutogradMatmul2bit = AutogradMatmul2bitCuda
backend = 'cuda'


def switch_backend_to(to_backend):
    """Kept for source compatibility (autograd_4bit.py:133-150); only ``'cuda'`` exists here."""
    global AutogradMatmul4bit, backend
    if to_backend == 'cuda':
        AutogradMatmul4bit = AutogradMatmul4bitCuda
        backend = 'cuda'
        print('Using CUDA implementation.')
    elif to_backend == 'triton':
        raise ValueError('Triton backend is not part of this build; the sm_100a CUDA library is the only backend.')
    else:
        raise ValueError('Backend not supported.')


def matmul4bit_with_backend(x, qweight, scales, qzeros, g_idx, bits, maxq, groupsize=None):
    if backend == 'cuda':
        return mm4b.matmul4bit(x, qweight, scales, qzeros, g_idx, groupsize)
    raise ValueError('Backend not supported.')


# Assumes layer is perfectly divisible into 256 * 256 blocks
class Autograd4bitQuantLinear(nn.Module):

    def __init__(self, in_features, out_features, groupsize=-1, is_v1_model=False, bits=4):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.bits = bits
        self.maxq = 2 ** self.bits - 1
        groupsize = groupsize if groupsize != -1 else in_features
        self.groupsize = groupsize
        self.is_v1_model = is_v1_model
        self.disable_bias = False
        per_word = 32 // bits
        if is_v1_model:
            self.register_buffer('zeros', torch.empty((out_features, 1)))
            self.register_buffer('scales', torch.empty((out_features, 1)))
            self.g_idx = None
        else:
            groups = math.ceil(in_features / groupsize)
            self.register_buffer('qzeros', torch.empty((groups, out_features // per_word), dtype=torch.int32))
            self.register_buffer('scales', torch.empty((groups, out_features)))
            self.register_buffer('g_idx', (torch.arange(in_features) // groupsize).to(torch.int32))
        self.register_buffer('bias', torch.zeros(out_features))
        self.register_buffer('qweight', torch.empty((in_features // per_word, out_features), dtype=torch.int32))

    def forward(self, x):
        zeros = self.zeros if self.is_v1_model else self.qzeros
        if self.bits == 4:
            if torch.is_grad_enabled():
                out = AutogradMatmul4bit.apply(x, self.qweight, self.scales, zeros, self.g_idx, self.bits, self.maxq)
            else:
                out = matmul4bit_with_backend(x, self.qweight, self.scales, zeros, self.g_idx, self.bits, self.maxq,
                                              self.groupsize)
        elif self.bits == 2:
            out = AutogradMatmul2bit.apply(x, self.qweight, self.scales, self.qzeros, self.g_idx, self.bits, self.maxq)
        else:
            raise ValueError('Unsupported bitwidth.')
        if not self.disable_bias and self.bias is not None:
            out = out + self.bias.to(out.dtype)
        return out


def make_quant_for_4bit_autograd(module, names, name='', groupsize=-1, is_v1_model=False, bits=4):
    """Swap every submodule whose dotted name is in ``names`` for a quant linear of the same shape
    (autograd_4bit.py:211-222)."""
    if isinstance(module, Autograd4bitQuantLinear):
        return
    for child_name, child in list(module.named_children()):
        full = name + '.' + child_name if name != '' else child_name
        if full in names:
            setattr(module, child_name,
                    Autograd4bitQuantLinear(child.in_features, child.out_features, groupsize=groupsize,
                                            is_v1_model=is_v1_model, bits=bits))
        else:
            make_quant_for_4bit_autograd(child, names, full, groupsize=groupsize, is_v1_model=is_v1_model, bits=bits)


def _cast_quant_buffers(model, dtype):
    for _, m in model.named_modules():
        if isinstance(m, Autograd4bitQuantLinear):
            if m.is_v1_model:
                m.zeros = m.zeros.to(dtype)
            m.scales = m.scales.to(dtype)
            if m.bias is not None:
                m.bias = m.bias.to(dtype)


def model_to_half(model):
    """``model.half()`` plus fp16 scales / zeros / bias on every quant linear (autograd_4bit.py:225-233)."""
    model.half()
    _cast_quant_buffers(model, torch.float16)
    print('Converted as Half.')


def model_to_float(model):
    """Inverse of :func:`model_to_half` (autograd_4bit.py:236-244)."""
    model.float()
    _cast_quant_buffers(model, torch.float32)
    print('Converted as Float.')


def find_layers(module, layers=(nn.Conv2d, nn.Linear), name=''):
    """Dotted name -> module for every leaf of the given types (autograd_4bit.py:247-255)."""
    if type(module) in tuple(layers):
        return {name: module}
    res = {}
    for child_name, child in module.named_children():
        res.update(find_layers(child, layers=layers, name=name + '.' + child_name if name != '' else child_name))
    return res


def _load_state(model, model_path):
    """Fill the quant buffers by name from a ``.safetensors`` / torch checkpoint, without accelerate."""
    if str(model_path).endswith('.safetensors'):
        from safetensors.torch import load_file
        state = load_file(model_path)
    else:
        state = torch.load(model_path, map_location='cpu')
    own = dict(model.named_parameters())
    own.update(dict(model.named_buffers()))
    missing = [k for k in own if k not in state and not k.endswith('rotary_emb.inv_freq')]
    for key, value in state.items():
        if key not in own:
            continue
        mod_name, _, leaf = key.rpartition('.')
        mod = model.get_submodule(mod_name) if mod_name else model
        cur = getattr(mod, leaf)
        if isinstance(cur, nn.Parameter):
            setattr(mod, leaf, nn.Parameter(value.to(cur.dtype), requires_grad=False))
        else:
            setattr(mod, leaf, value)
    if missing:
        logging.warning('checkpoint has no entry for: %s', ', '.join(missing[:8]))
    return model


def load_llama_model_4bit_low_ram(config_path, model_path, groupsize=-1, half=False, device_map="auto", seqlen=2048,
                                  is_v1_model=False, bits=4):
    """Build an HF LLaMA, swap every linear but ``lm_head`` for a quant linear and load a GPTQ
    checkpoint into it (autograd_4bit.py:258-294).  The reference places weights with accelerate;
    this loader reads the checkpoint directly and moves the model to one device (``device_map`` of the
    form ``{'': device}`` or ``"auto"`` = current CUDA device)."""
    from transformers import AutoTokenizer, LlamaConfig, LlamaForCausalLM
    t0 = time.time()
    config = LlamaConfig.from_pretrained(config_path)
    saved = torch.get_default_dtype()
    torch.set_default_dtype(torch.float16)
    try:
        with torch.device('meta'):
            model = LlamaForCausalLM(config)
    finally:
        torch.set_default_dtype(saved)
    model = model.to_empty(device='cpu')
    layers = find_layers(model)
    layers.pop('lm_head', None)
    make_quant_for_4bit_autograd(model, layers, groupsize=groupsize, is_v1_model=is_v1_model, bits=bits)
    _load_state(model, model_path)
    device = device_map.get('', 'cuda') if isinstance(device_map, dict) else 'cuda'
    model = model.to(device)
    model.seqlen = seqlen
    if half:
        model_to_half(model)
    tokenizer = AutoTokenizer.from_pretrained(config_path)
    tokenizer.truncation_side = 'left'
    print(f"Loaded the model in {(time.time() - t0):.2f} seconds.")
    return model, tokenizer
