"""Test-only stand-in for ``alpaca_lora_4bit_b200.quant_cuda`` built on the CPU oracle.

The package has no CPU path; to exercise its host-side logic (dispatch, autograd wiring, module
surgery) without a GPU the tests swap the kernel facade for these oracle-backed functions.
Nothing outside ``tests/`` may import this file."""
import contextlib

import torch

from oracle import q4_oracle as orc


def vecquant4recons_v2(mat, res, scales, zeros, g_idx):
    res.copy_(orc.recons_v2(mat, scales, zeros, g_idx))


def vecquant4recons_v1(mat, res, scales, zeros):
    res.copy_(orc.recons_v1(mat, scales, zeros))


def vecquant2recons_v2(mat, res, scales, zeros, g_idx):
    res.copy_(orc.recons2_v2(mat, scales, zeros, g_idx))


def gemv(x, qweight, y, scales, zeros, g_idx, groupsize, flags, bias=None):
    K = x.shape[-1]
    if flags & 4:
        w = orc.recons_v1(qweight, scales.reshape(-1), zeros.reshape(-1))
    else:
        gi = g_idx if (flags & 2) else (torch.arange(K) // groupsize).int()
        w = orc.recons_v2(qweight, scales, zeros, gi)
    out = x.float() @ w.float()
    if bias is not None:
        out = out + bias.float()
    y.copy_((y.float() + out) if (flags & 1) else out)


def decode_planned(x, qweight, scales, zeros, groupsize, max_rows):
    return None                                   # no layer is ever recorded: every call takes the general path


def gemm_supported(K, N, G, transpose):
    return K % 128 == 0 and N % 128 == 0


def gemm(x, qweight, out, scales, zeros, g_idx, transpose=False, bias=None, residual=None):
    w = orc.recons_v2(qweight, scales, zeros, g_idx).float()
    y = x.float() @ (w.t() if transpose else w)
    if bias is not None:
        y = y + bias.float()
    out.copy_(y)
    if residual is not None:
        out.add_(residual)


@contextlib.contextmanager
def installed():
    """Route the dispatch layer to the oracle for the duration of the block."""
    import sys
    from alpaca_lora_4bit_b200 import matmul_utils_4bit as mm4b
    me = sys.modules[__name__]
    saved = mm4b.quant_cuda
    mm4b.quant_cuda = me
    try:
        yield
    finally:
        mm4b.quant_cuda = saved
