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
    def forward(ctx, x, qweight, scales, zeros, g_idx, bits, maxq, bias=None, residual=None):
        """``bias`` (not an argument of the reference's function, whose module adds the bias in a kernel of
        its own, autograd_4bit.py:204-206) and ``residual`` (the skip path a decoder layer adds after the
        projection): added in the epilogue of the fused product where that runs."""
        ctx.save_for_backward(qweight, scales, zeros, g_idx)
        if g_idx is None:
            out = mm4b._matmul4bit_v1_recons(x, qweight, scales, zeros)
            out = out if bias is None else out + bias.to(out.dtype)
            return out if residual is None else out + residual.to(out.dtype)
        return mm4b._matmul4bit_v2_recons(x, qweight, scales, zeros, g_idx, bias=bias, residual=residual)

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
        res_grad = grad_output if (len(ctx.needs_input_grad) > 8 and ctx.needs_input_grad[8]) else None
        return (grad, None, None, None, None, None, None, None, res_grad)[:max(len(ctx.needs_input_grad), 7)]


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

    def take_residual(self):
        """The skip-path tensor a patched decoder layer left for this call (``offer_residual``), or None: whoever
        computes this module's output adds it, in the product's epilogue where that is possible."""
        return self.__dict__.pop("_q4_residual", None)

    def offer_residual(self, residual) -> None:
        """Called by a decoder layer patched by ``fused_ops.patch_llama`` right before the block that ends in this
        projection: the next ``forward`` returns ``projection + residual``."""
        self.__dict__["_q4_residual"] = residual

    def forward(self, x):
        residual = self.take_residual()
        out = self._forward(x, residual)
        return out

    def _forward(self, x, residual=None):
        zeros = self.zeros if self.is_v1_model else self.qzeros
        if self.bits == 4:
            if torch.is_grad_enabled():
                if AutogradMatmul4bit is AutogradMatmul4bitCuda:
                    # bias and residual ride in the product's epilogue instead of further passes over the output
                    bias = None if (self.disable_bias or self.bias is None) else self.bias
                    if residual is not None and residual.dtype != torch.float16:
                        out = AutogradMatmul4bit.apply(x, self.qweight, self.scales, zeros, self.g_idx, self.bits, self.maxq, bias)
                        return out + residual.to(out.dtype)
                    return AutogradMatmul4bit.apply(x, self.qweight, self.scales, zeros, self.g_idx, self.bits, self.maxq, bias, residual)
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
        if residual is not None:
            out = out + residual.to(out.dtype)
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


def _read_checkpoint(model_path):
    if str(model_path).endswith('.safetensors'):
        from safetensors.torch import load_file
        return load_file(str(model_path))
    return torch.load(model_path, map_location='cpu')


def _load_state(model, model_path):
    """Fill parameters and quant buffers by name from a ``.safetensors`` / torch checkpoint, without
    accelerate.  Like ``accelerate.load_checkpoint_and_dispatch`` with no dtype given (what the reference
    calls, autograd_4bit.py:273-278), a floating-point entry is cast to the dtype the module holds for it
    (so fp16 ``scales`` of a checkpoint become fp32 until ``model_to_half``); integer entries are taken as
    they are.  Every value lands on the device of the tensor it replaces."""
    state = _read_checkpoint(model_path)
    own = dict(model.named_parameters())
    own.update(dict(model.named_buffers()))
    missing = [k for k in own if k not in state and 'rotary_emb' not in k]
    unexpected = [k for k in state if k not in own]
    for key, value in state.items():
        if key not in own:
            continue
        mod_name, _, leaf = key.rpartition('.')
        mod = model.get_submodule(mod_name) if mod_name else model
        cur = getattr(mod, leaf)
        if tuple(value.shape) != tuple(cur.shape):
            raise ValueError(f'checkpoint entry {key} has shape {tuple(value.shape)}, the model expects {tuple(cur.shape)}')
        if cur.is_floating_point() and value.is_floating_point():
            value = value.to(cur.dtype)
        value = value.to(cur.device)
        if isinstance(cur, nn.Parameter):
            setattr(mod, leaf, nn.Parameter(value, requires_grad=False))
        else:
            setattr(mod, leaf, value)
    if missing:
        logging.warning('checkpoint has no entry for: %s', ', '.join(missing[:8]))
    if unexpected:
        logging.warning('checkpoint entries without a place in the model: %s', ', '.join(unexpected[:8]))
    return model


def reset_rotary_buffers(model, config, device):
    """The rotary embedding's ``inv_freq`` / ``original_inv_freq`` are non-persistent buffers: no checkpoint
    holds them, and a model materialised from the meta device has uninitialised memory there.  Recompute
    them from the configuration."""
    for mod in model.modules():
        if hasattr(mod, 'inv_freq') and hasattr(mod, 'compute_default_rope_parameters'):
            inv, scaling = mod.compute_default_rope_parameters(config, device)
            mod.inv_freq = inv
            if hasattr(mod, 'original_inv_freq'):
                mod.original_inv_freq = inv.clone()
            if hasattr(mod, 'attention_scaling'):
                mod.attention_scaling = scaling


def _target_device(device_map):
    if isinstance(device_map, dict):
        return torch.device(device_map.get('', 'cuda'))
    if isinstance(device_map, (str, torch.device)) and str(device_map) not in ('auto', 'balanced', 'sequential'):
        return torch.device(device_map)
    return torch.device('cuda', torch.cuda.current_device()) if torch.cuda.is_available() else torch.device('cpu')


def load_llama_model_4bit_low_ram(config_path, model_path, groupsize=-1, half=False, device_map="auto", seqlen=2048,
                                  is_v1_model=False, bits=4):
    """Build an HF LLaMA, swap every linear but ``lm_head`` for a quant linear and load a GPTQ
    checkpoint into it (autograd_4bit.py:258-294).  The reference places weights with accelerate;
    this loader reads the checkpoint directly onto one device (``device_map`` of the form
    ``{'': device}``, a device, or ``"auto"`` = the current CUDA device).  The model is built on the
    meta device and its linears are swapped there, so the dense weights of the quantised layers never
    exist anywhere.  Returns ``(model, tokenizer)``; the tokenizer is ``None`` when ``config_path``
    holds no tokenizer files."""
    from transformers import LlamaConfig, LlamaForCausalLM
    t0 = time.time()
    config = LlamaConfig.from_pretrained(config_path)
    with torch.device('meta'):
        model = LlamaForCausalLM(config)
        model = model.eval()
        layers = find_layers(model)
        layers.pop('lm_head', None)
        make_quant_for_4bit_autograd(model, layers, groupsize=groupsize, is_v1_model=is_v1_model, bits=bits)
    device = _target_device(device_map)
    model = model.to_empty(device=device)
    for m in model.modules():                       # buffers the constructor computes and no checkpoint carries
        if isinstance(m, Autograd4bitQuantLinear):
            m.bias = torch.zeros(m.out_features, device=device)
            if not m.is_v1_model:
                m.g_idx = (torch.arange(m.in_features, device=device) // m.groupsize).to(torch.int32)
    _load_state(model, model_path)
    reset_rotary_buffers(model, config, device)
    if getattr(config, 'tie_word_embeddings', False):
        model.tie_weights()
    model.seqlen = seqlen
    if half:
        model_to_half(model)
    tokenizer = None
    try:
        from transformers import AutoTokenizer
        tokenizer = AutoTokenizer.from_pretrained(config_path)
        tokenizer.truncation_side = 'left'
    except (OSError, ValueError, KeyError, TypeError) as exc:
        logging.warning('no tokenizer loaded from %s (%s)', config_path, type(exc).__name__)
    print(f"Loaded the model in {(time.time() - t0):.2f} seconds.")
    return model, tokenizer


def load_llama_model_4bit_low_ram_and_offload(config_path, model_path, lora_path=None, groupsize=-1, seqlen=2048,
                                              max_memory=None, is_v1_model=False, bits=4):
    """The reference's variant for GPUs that cannot hold the model spreads layers over GPU and host
    memory with accelerate (autograd_4bit.py:296-362).  A B200 holds every LLaMA this format exists for
    (a 70B int4 checkpoint is 35 GB of 180), so the whole model goes to the current device, in half
    precision as the reference leaves it; ``max_memory`` is accepted and ignored.  With ``lora_path`` the
    PEFT adapter there is applied through the int4 LoRA layers (needs ``peft``)."""
    model, tokenizer = load_llama_model_4bit_low_ram(config_path, model_path, groupsize=groupsize, half=False,
                                                     seqlen=seqlen, is_v1_model=is_v1_model, bits=bits)
    if lora_path is not None:
        from .monkeypatch.peft_tuners_lora_monkey_patch import replace_peft_model_with_int4_lora_model
        replace_peft_model_with_int4_lora_model()
        from peft import PeftModel
        model = PeftModel.from_pretrained(model, lora_path, torch_dtype=torch.float32, is_trainable=True)
        print('{} Lora Applied.'.format(lora_path))
    _cast_quant_buffers(model, torch.float16)
    return model, tokenizer


load_llama_model_4bit_low_ram_and_offload_to_cpu = load_llama_model_4bit_low_ram_and_offload
