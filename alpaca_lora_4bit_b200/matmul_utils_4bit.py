"""Dispatch layer with the names, flags and call signatures of the reference's
``matmul_utils_4bit`` (matmul_utils_4bit.py:12-186), on the sm_100a kernels.

Routing (``matmul4bit``, matmul_utils_4bit.py:146-170): ``zeros.dtype != int32`` means a v1
layer, otherwise v2; ``prod(x.shape[:-1]) > auto_switch_thd`` goes to the large-M path,
anything smaller to the decode kernel.  Module-level switches keep their reference names:

  use_new, auto_switch, auto_switch_thd   as in the reference (threshold default 8; the decode
                                          kernel itself accepts up to 16 rows per launch)
  faster_mode                             'old_faster' | 'faster' | 'disable' — all three run the
                                          same decode kernel; the value only selects whether the
                                          groups come from ``groupsize`` or from ``g_idx``
  act_order                               take the group of every row from ``g_idx``
  cache_buffer / buffer_mat_dic           cache of dense fp16 buffers used by the reconstruct path
  fused_gemm (new)                        True: ``_matmul4bit_v2_recons`` runs the fused dequant-GEMM
                                          kernels (W never written to global memory) whenever the
                                          operands are fp16 and the shape is supported; False, or an
                                          unsupported shape / dtype: reconstruct + ``torch.matmul`` as
                                          in the reference
  debug                                   print which variant ran
"""
from __future__ import annotations

import math

import numpy as np
import torch

from . import _lib, quant_cuda

# Global Buffer
buffer_mat_dic = {}
use_new = True
auto_switch = True
auto_switch_thd = 8
debug = False
faster_mode = 'old_faster'  # set disable to disable it
valid_faster_mode = ('faster', 'old_faster')
act_order = False
cache_buffer = True
fused_gemm = True          # large-M v2 products on the fused tcgen05 kernels instead of reconstruct + library GEMM


def get_buffer(shape_of_qweight, dtype=torch.float16, device='cuda', bits=4):
    """Dense ``[K, N]`` scratch for the reconstruct path, cached per shape (matmul_utils_4bit.py:22-33)."""
    target_shape = (shape_of_qweight[0] * (32 // bits), shape_of_qweight[1])
    if not cache_buffer:
        return torch.empty(target_shape, dtype=dtype, device=device)
    buf = buffer_mat_dic.get(target_shape)
    if buf is None or buf.device != torch.device(device) or buf.dtype != dtype:
        buf = torch.empty(target_shape, dtype=dtype, device=device)
        buffer_mat_dic[target_shape] = buf
    return buf




_groups_are_sequential = quant_cuda.groups_are_sequential


def _decode(x, qweight, scales, zeros, g_idx, groupsize, flags):
    dtype = x.dtype
    x2 = x if x.dim() == 2 else x.reshape(-1, x.shape[-1])
    if x2.shape[0] == 0:                      # no rows: nothing to launch
        return x.new_zeros(x.shape[:-1] + (qweight.shape[1],))
    if dtype != torch.float16:
        x2 = x2.half()
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    y = torch.empty((x2.shape[0], qweight.shape[1]), dtype=torch.float16 if dtype == torch.float16 else torch.float32,
                    device=x.device)
    quant_cuda.gemv(x2, qweight, y, scales if scales.dtype == torch.float16 else scales.half(), zeros, g_idx, groupsize, flags)
    if y.dtype != dtype:
        y = y.to(dtype)
    return y if x.dim() == 2 else y.reshape(x.shape[:-1] + (qweight.shape[1],))


def _matmul4bit_v1(x, qweight, scales, zeros):
    """Decode product on a v1 layer (matmul_utils_4bit.py:36-56): ``x @ (scales*q - zeros)``."""
    if debug:
        print('_matmul4bit_v1')
    assert qweight.shape[0] * 8 == x.shape[-1]
    sh = scales.half().reshape(-1).contiguous()
    zh = zeros.half().reshape(-1).contiguous()
    return _decode(x, qweight, sh, zh, None, x.shape[-1], _lib.GEMV_V1)


def _matmul4bit_v2(x, qweight, scales, zeros, g_idx, groupsize=None):
    """Decode product on a v2 layer (matmul_utils_4bit.py:59-95)."""
    if debug:
        print('_matmul4bit_v2')
    assert qweight.shape[0] * 8 == x.shape[-1]
    if faster_mode not in valid_faster_mode and faster_mode != 'disable':
        raise ValueError('faster_mode should be in {}'.format(valid_faster_mode))
    K = x.shape[-1]
    if groupsize is None or groupsize <= 0:
        groupsize = K // scales.shape[0]
    # 'old_faster' derives the group from the row index (quant_cuda_kernel.cu:1023); the other
    # reference variants read g_idx (matmul_utils_4bit.py:75-83,90-93).  With sequential g_idx both
    # agree, so the per-row lookup is taken for act_order, for a group size the sequential kernel
    # cannot take, and - outside 'old_faster' - for a g_idx that is not sequential.
    by_index = act_order or (groupsize % 32 != 0)
    if not by_index and faster_mode != 'old_faster' and g_idx is not None:
        by_index = not _groups_are_sequential(g_idx, scales.shape[0])
    if by_index and g_idx is None:
        raise ValueError('act_order decode needs g_idx')
    return _decode(x, qweight, scales, zeros, g_idx if by_index else None, groupsize,
                   _lib.GEMV_ACT_ORDER if by_index else 0)


def _dense_matmul(x, buffer, transpose):
    """``x @ W`` or ``x @ W.T`` on a reconstructed dense weight (library GEMM)."""
    return torch.matmul(x, buffer.T if transpose else buffer)


def _check_inner(x, qweight, per_word, transpose):
    inner = qweight.shape[1] if transpose else qweight.shape[0] * per_word
    assert inner == x.shape[-1], f"inner dimension {x.shape[-1]} does not match the layer ({inner})"


def _matmul4bit_v1_recons(x, qweight, scales, zeros, transpose=False):
    """Large-M product on a v1 layer (matmul_utils_4bit.py:98-111)."""
    if debug:
        print('_matmul4bit_v1_recons')
    _check_inner(x, qweight, 8, transpose)
    buffer = get_buffer(qweight.shape, dtype=scales.dtype, device=qweight.device)
    quant_cuda.vecquant4recons_v1(qweight, buffer, scales.reshape(-1), zeros.reshape(-1))
    return _dense_matmul(x, buffer, transpose)


def _with_bias(out, bias):
    return out if bias is None else out + bias.to(out.dtype)


def _plus(out, residual):
    return out if residual is None else out + residual.reshape(out.shape).to(out.dtype)


def _matmul4bit_v2_recons(x, qweight, scales, zeros, g_idx, transpose=False, bias=None, residual=None):
    """Large-M product on a v2 layer (matmul_utils_4bit.py:114-127): ``x @ W`` or, with
    ``transpose``, ``x @ W.T`` (the backward of the layer).  ``bias`` and ``residual`` (forward only; not
    arguments of the reference's function): added to the product - the residual to the rounded product, as a
    separate fp16 add would - inside the kernel where the fused path runs."""
    if debug:
        print('_matmul4bit_v2_recons')
    _check_inner(x, qweight, 8, transpose)
    K, N = qweight.shape[0] * 8, qweight.shape[1]
    rows = math.prod(x.shape[:-1])
    if (not transpose and 0 < rows <= 16 and x.is_cuda and x.dtype == torch.float16 and scales.dtype == torch.float16):
        # a handful of rows above the switch threshold: the streaming decode kernel still ends sooner than a
        # tensor-core launch whose tiles would be almost all padding.  The reconstruct path always honours
        # g_idx (matmul_utils_4bit.py:121), so the sequential-group kernel is taken only for a g_idx that is
        # sequential; any other goes to the decode kernel that looks the group of every row up.
        G = scales.shape[0]
        if not act_order and K % G == 0 and (K // G) % 32 == 0 and _groups_are_sequential(g_idx, G):
            return _plus(_with_bias(_decode(x, qweight, scales, zeros, None, K // G, 0), bias), residual)
        return _plus(_with_bias(_decode(x, qweight, scales, zeros, g_idx, max(K // G, 1), _lib.GEMV_ACT_ORDER), bias), residual)
    if (fused_gemm and x.dtype == torch.float16 and scales.dtype == torch.float16
            and quant_cuda.gemm_supported(K, N, scales.shape[0], transpose)):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        out = torch.empty((x2.shape[0], K if transpose else N), dtype=torch.float16, device=x.device)
        if x2.shape[0] > 0:                   # no rows: nothing to launch
            b16 = None if (bias is None or transpose) else (bias if bias.dtype == torch.float16 else bias.half())
            res2 = None
            if residual is not None and not transpose and residual.dtype == torch.float16 and residual.numel() == out.numel():
                res2 = residual.reshape(out.shape)
                res2 = res2 if res2.is_contiguous() else None
            quant_cuda.gemm(x2, qweight, out, scales, zeros, g_idx, transpose=transpose, bias=b16, residual=res2)
            if residual is not None and res2 is None:
                out = _plus(out, residual)
        elif residual is not None:
            out = _plus(out, residual)
        return out.reshape(x.shape[:-1] + (out.shape[-1],))
    buffer = get_buffer(qweight.shape, dtype=scales.dtype, device=qweight.device)
    quant_cuda.vecquant4recons_v2(qweight, buffer, scales, zeros, g_idx)
    return _plus(_with_bias(_dense_matmul(x, buffer, transpose), None if transpose else bias), None if transpose else residual)


def _matmul2bit_v2_recons(x, qweight, scales, zeros, g_idx, transpose=False):
    """Large-M product on a 2-bit v2 layer (matmul_utils_4bit.py:130-143)."""
    if debug:
        print('_matmul2bit_v2_recons')
    _check_inner(x, qweight, 16, transpose)
    buffer = get_buffer(qweight.shape, dtype=scales.dtype, device=qweight.device, bits=2)
    quant_cuda.vecquant2recons_v2(qweight, buffer, scales, zeros, g_idx)
    return _dense_matmul(x, buffer, transpose)


def matmul4bit(x, qweight, scales, zeros, g_idx=None, groupsize=None):
    """No-grad entry (matmul_utils_4bit.py:146-170): format from ``zeros.dtype``, kernel from M."""
    # the sequential-group kernel serves the default 'old_faster' mode, which derives groups from the row index
    # as the reference's kernel does, and the modes that read g_idx when that g_idx is sequential
    seq_ok = (g_idx is not None and not act_order and not debug and
              (faster_mode == 'old_faster' or ((faster_mode == 'faster' or faster_mode == 'disable') and zeros.dtype == torch.int32
                                               and _groups_are_sequential(g_idx, scales.shape[0]))))
    if seq_ok:
        # a layer the per-token path has served before: its recorded plan, if this call fits it
        y = quant_cuda.decode_planned(x, qweight, scales, zeros, -1 if groupsize is None else groupsize,
                                      min(16, auto_switch_thd) if use_new and auto_switch else 16)
        if y is not None:
            return y
    if (seq_ok and x.dim() == 2 and 1 <= x.shape[0] <= 16 and not (use_new and auto_switch and x.shape[0] > auto_switch_thd)
            and zeros.dtype == torch.int32 and x.dtype == torch.float16 and scales.dtype == torch.float16
            and x.is_cuda and x.is_contiguous()):
        # the per-token call: sequential groups, fp16 in and out - straight to the decode kernel
        gs = groupsize if groupsize is not None and groupsize > 0 else x.shape[1] // scales.shape[0]
        if gs % 32 == 0:
            return quant_cuda.decode_v2(x, qweight, scales, zeros, gs, plan_key=-1 if groupsize is None else groupsize)
    rows = math.prod(x.shape[:-1])
    large = use_new and auto_switch and rows > auto_switch_thd
    if zeros.dtype != torch.int32:            # v1: float zeros
        if large:
            return _matmul4bit_v1_recons(x.half(), qweight, scales.half(), zeros.half())
        return _matmul4bit_v1(x, qweight, scales, zeros)
    if g_idx is None:                         # v2 without g_idx: one group
        g_idx = torch.zeros(qweight.shape[0] * 8, dtype=torch.int32, device=x.device)
    if large:
        return _matmul4bit_v2_recons(x.half(), qweight, scales.half(), zeros, g_idx)
    return _matmul4bit_v2(x, qweight, scales, zeros, g_idx, groupsize)


def v2_to_v1(scales, zeros):
    """Float zero term ``(z + 1) * scales`` of a one-group v2 layer, i.e. its v1 form
    (matmul_utils_4bit.py:173-186; a debugging aid in the reference)."""
    assert zeros.shape[0] == 1
    shifts = torch.arange(0, 32, 4, device=zeros.device, dtype=torch.int32)
    z = ((zeros.reshape(-1, 1) >> shifts) & 0xF).reshape(-1).to(torch.float16)
    return z * scales + scales
