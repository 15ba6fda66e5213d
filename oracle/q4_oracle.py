"""CPU oracle for the GPTQ int4 dequant-matmul path.  TEST INFRASTRUCTURE ONLY.

This file restates, on the CPU with torch tensors, the arithmetic of the reference's
``quant_cuda`` kernels and of the Python composition built on them.  Only ``tests/``,
``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline / ``--impl reference`` legs may
import it; the shipped package never does.

Parity status: **pinned against the reference's own kernels.**  The reference has no CPU
implementation of this path and its only tests are whole-model runs that need a checkpoint
download (tests/test_cuda_generation.py:56-73, tests/test_cuda_finetune.py:87), so none of its
test vectors reaches the operator boundary.  Instead its ``quant_cuda`` extension is compiled
unmodified for sm_100a (``oracle/build_ref.py`` -> ``oracle/_ref/``) and
``tests/test_reference_kernels.py`` runs those kernels on the GPU next to this oracle: the
reconstruct kernels (4-bit v2 with fp16 and fp32 scales, v1, 2-bit) agree with the functions below
bit for bit, the decode kernels within the tolerance.  On a machine without a GPU the oracle is
additionally held to an independent scalar re-derivation of the kernel source, element by
element (``tests/golden/make_golden.py``).

Arithmetic notes.  The reference kernels are templated on ``scalar_t``; for ``c10::Half`` every
binary operator converts to float, computes, and rounds back to half, so
``scale * q - zero`` is three separately rounded fp16 operations and never an FMA
(float arithmetic on two halves followed by one rounding to half equals the correctly rounded
half operation because 24 >= 2*11+2).  torch's CPU half kernels round the same way.
"""
from __future__ import annotations

import torch

__all__ = [
    "unpack_rows", "unpack_cols", "recons_v2", "recons_v1", "recons2_v2",
    "matmul_recons", "matmul4bit_ref", "gemv_fp32", "lora_forward", "lora_backward",
]


def unpack_rows(qweight: torch.Tensor, bits: int = 4) -> torch.Tensor:
    """int32 ``[K*bits/32, N]`` -> int32 ``[K, N]`` of quantised levels.

    Row ``k = (32/bits)*r + j`` is field ``j`` (low bits first) of word ``qweight[r, n]``:
    ``(tmp >> shift) & 0xF`` with ``shift = b % 8 * 4`` (quant_cuda_kernel.cu:1148-1151;
    2-bit: ``b % 16 * 2``, ``& 0x3``, :1206-1209).
    """
    per = 32 // bits
    mask = (1 << bits) - 1
    w = qweight.to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(per, dtype=torch.int64) * bits
    q = (w[:, None, :] >> shifts[None, :, None]) & mask          # [R, per, N]
    return q.reshape(qweight.shape[0] * per, qweight.shape[1]).to(torch.int32)


def unpack_cols(qzeros: torch.Tensor, bits: int = 4) -> torch.Tensor:
    """int32 ``[G, N*bits/32]`` -> int32 ``[G, N]`` of stored zero points (without the +1).

    Column ``n`` is field ``n % (32/bits)`` of word ``qzeros[g, n / (32/bits)]``
    (quant_cuda_kernel.cu:1143-1146).
    """
    per = 32 // bits
    mask = (1 << bits) - 1
    z = qzeros.to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(per, dtype=torch.int64) * bits
    out = (z[:, :, None] >> shifts[None, None, :]) & mask         # [G, W, per]
    return out.reshape(qzeros.shape[0], qzeros.shape[1] * per).to(torch.int32)


def _recons_generic(qweight, scales, qzeros, g_idx, bits):
    q = unpack_rows(qweight, bits)                                 # [K, N]
    z1 = unpack_cols(qzeros, bits) + 1                             # [G, N]
    gi = g_idx.to(torch.int64)
    T = scales.dtype
    s = scales[gi]                                                 # [K, N]
    if T == torch.float16:
        zero = s * z1[gi].to(T)                                    # rounded to fp16
        return s * q.to(T) - zero                                  # two more roundings
    # float: nvcc contracts ``scale * q - zero`` into one FMA (zero itself is a rounded product).
    zero = s * z1[gi].to(T)
    prod = s.double() * q.double() - zero.double()                 # exact in double, one rounding
    return prod.to(T)


def recons_v2(qweight, scales, qzeros, g_idx) -> torch.Tensor:
    """VecQuant4ReconsV2Kernel (quant_cuda_kernel.cu:1127-1153).

    ``W[k,n] = scale * T(q) - scale * T(z+1)`` with ``scale = scales[g_idx[k], n]`` and ``z`` the
    nibble ``n%8`` of ``qzeros[g_idx[k], n/8]``; result dtype = ``scales.dtype``.
    """
    return _recons_generic(qweight, scales, qzeros, g_idx, 4)


def recons2_v2(qweight, scales, qzeros, g_idx) -> torch.Tensor:
    """VecQuant2ReconsV2Kernel (quant_cuda_kernel.cu:1185-1211): 16 two-bit fields per word."""
    return _recons_generic(qweight, scales, qzeros, g_idx, 2)


def recons_v1(qweight, scales, zeros) -> torch.Tensor:
    """VecQuant4ReconsV1Kernel (quant_cuda_kernel.cu:1076-1097).

    ``W[k,n] = scales[n] * T(q) - zeros[n]`` (per-column float scale and zero, two roundings).
    """
    q = unpack_rows(qweight, 4)
    T = scales.dtype
    s = scales.reshape(1, -1)
    z = zeros.reshape(1, -1).to(T)
    if T == torch.float16:
        return s * q.to(T) - z
    return (s.double() * q.double() - z.double()).to(T)


def matmul_recons(x, w, transpose: bool = False) -> torch.Tensor:
    """fp32-accumulate matmul on a reconstructed weight: ``x @ W`` or ``x @ W.T``.

    The reference composition is reconstruct-then-``torch.matmul``
    (matmul_utils_4bit.py:121-126); cuBLAS accumulates in fp32, so the oracle multiplies in
    fp32 and leaves the result unrounded for the relative-Frobenius comparison.
    """
    wf = w.float()
    return x.float() @ (wf.t() if transpose else wf)


def matmul4bit_ref(x, qweight, scales, qzeros, g_idx, transpose: bool = False) -> torch.Tensor:
    """``_matmul4bit_v2_recons`` (matmul_utils_4bit.py:114-127) in fp32."""
    return matmul_recons(x, recons_v2(qweight, scales, qzeros, g_idx), transpose)


def gemv_fp32(x, qweight, scales, qzeros, g_idx) -> torch.Tensor:
    """VecQuant4MatMulKernel (quant_cuda_kernel.cu:475-536) in real arithmetic.

    ``y[b,n] = sum_k (s*q - s*(z+1)) * x[b,k]`` with ``s = scales[g_idx[k], n]``, all in fp32 in
    the reference; evaluated here in float64 so that it serves as the exact target for the
    decode kernels (which only have to meet the relative-Frobenius tolerance).
    """
    q = unpack_rows(qweight, 4).double()
    z1 = (unpack_cols(qzeros, 4) + 1).double()
    gi = g_idx.to(torch.int64)
    s = scales.double()[gi]
    w = s * q - s * z1[gi]
    return x.double() @ w


def lora_forward(x, A, B, scaling: float) -> torch.Tensor:
    """``lora_B(lora_A(x)) * scaling`` (models.py:61-66) in fp32: A ``[r,K]``, B ``[N,r]``."""
    return (x.float() @ A.float().t()) @ B.float().t() * scaling


def lora_backward(x, dy, A, B, scaling: float):
    """Gradients of the LoRA branch by plain calculus, fp32: returns ``(dx, dA, dB)``."""
    xf, dyf, Af, Bf = x.float(), dy.float(), A.float(), B.float()
    u = xf @ Af.t()                      # [M, r]
    dB = (dyf.t() @ u) * scaling         # [N, r]
    du = (dyf @ Bf) * scaling            # [M, r]
    dA = du.t() @ xf                     # [r, K]
    dx = du @ Af                         # [M, K]
    return dx, dA, dB
