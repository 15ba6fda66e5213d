"""Seeded synthetic GPTQ layers and activations.

No checkpoint is reachable from a sandbox without network, so the benchmark, the smoke test and
the tests draw layers with the distributions of a real GPTQ v2 checkpoint: every 4-bit level
equally likely, stored zero points 0..14 (the kernels add 1), fp16 scales uniform in
[0.002, 0.02], and either sequential groups (``g_idx[k] = k // groupsize``) or an act-order
permutation (``g_idx[k] = perm[k] // groupsize``).  Everything comes from one CPU
``torch.Generator`` in a fixed draw order, so two callers with the same seed see the same bits.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class QuantLayer:
    """Packed buffers of one quantised linear, named as in Autograd4bitQuantLinear."""
    qweight: torch.Tensor          # int32 [K*bits/32, N]
    qzeros: torch.Tensor           # int32 [G, N*bits/32]
    scales: torch.Tensor           # fp16  [G, N]
    g_idx: torch.Tensor            # int32 [K]
    K: int
    N: int
    groupsize: int
    bits: int = 4

    def to(self, device) -> "QuantLayer":
        return QuantLayer(self.qweight.to(device), self.qzeros.to(device), self.scales.to(device),
                          self.g_idx.to(device), self.K, self.N, self.groupsize, self.bits)


def _rand_words(shape, gen) -> torch.Tensor:
    """Uniform 32-bit patterns as int32."""
    lo = torch.randint(0, 1 << 16, shape, generator=gen, dtype=torch.int64)
    hi = torch.randint(0, 1 << 16, shape, generator=gen, dtype=torch.int64)
    w = (hi << 16) | lo
    w = torch.where(w >= (1 << 31), w - (1 << 32), w)
    return w.to(torch.int32)


def pack_cols(levels: torch.Tensor, bits: int = 4) -> torch.Tensor:
    """int ``[G, N]`` levels -> int32 ``[G, N*bits/32]``, field ``n % per`` of word ``n // per``."""
    per = 32 // bits
    G, N = levels.shape
    v = levels.to(torch.int64).reshape(G, N // per, per)
    shifts = torch.arange(per, dtype=torch.int64) * bits
    w = (v << shifts).sum(-1)
    w = torch.where(w >= (1 << 31), w - (1 << 32), w)
    return w.to(torch.int32)


def pack_rows(levels: torch.Tensor, bits: int = 4) -> torch.Tensor:
    """int ``[K, N]`` levels -> int32 ``[K*bits/32, N]``, field ``k % per`` of word ``k // per``."""
    per = 32 // bits
    K, N = levels.shape
    v = levels.to(torch.int64).reshape(K // per, per, N)
    shifts = (torch.arange(per, dtype=torch.int64) * bits)[None, :, None]
    w = (v << shifts).sum(1)
    w = torch.where(w >= (1 << 31), w - (1 << 32), w)
    return w.to(torch.int32)


def make_layer(K: int, N: int, groupsize: int = 128, act_order: bool = False, seed: int = 0,
               bits: int = 4, gen: Optional[torch.Generator] = None) -> QuantLayer:
    """Draw one layer on the CPU.  Draw order: qweight, zero levels, scales, permutation."""
    if gen is None:
        gen = torch.Generator(device="cpu").manual_seed(seed)
    per = 32 // bits
    if groupsize == -1:
        groupsize = K
    G = math.ceil(K / groupsize)
    qweight = _rand_words((K // per, N), gen)
    zlev = torch.randint(0, (1 << bits) - 1, (G, N), generator=gen, dtype=torch.int64)
    qzeros = pack_cols(zlev, bits)
    scales = (torch.rand((G, N), generator=gen, dtype=torch.float32) * 0.018 + 0.002).half()
    if act_order:
        perm = torch.randperm(K, generator=gen)
        g_idx = (perm // groupsize).to(torch.int32)
    else:
        g_idx = (torch.arange(K) // groupsize).to(torch.int32)
    return QuantLayer(qweight, qzeros, scales, g_idx, K, N, groupsize, bits)


def make_acts(M: int, K: int, seed: int = 1, gen: Optional[torch.Generator] = None,
              dtype=torch.float16) -> torch.Tensor:
    """Activations ``[M, K] ~ N(0, 1)``."""
    if gen is None:
        gen = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn((M, K), generator=gen, dtype=torch.float32).to(dtype)


def make_lora(K: int, N: int, r: int, seed: int = 2, std_a: float = 0.02, std_b: float = 0.02,
              gen: Optional[torch.Generator] = None, dtype=torch.float16):
    """LoRA factors ``A [r, K] ~ N(0, std_a)``, ``B [N, r] ~ N(0, std_b)``."""
    if gen is None:
        gen = torch.Generator(device="cpu").manual_seed(seed)
    A = (torch.randn((r, K), generator=gen, dtype=torch.float32) * std_a).to(dtype)
    B = (torch.randn((N, r), generator=gen, dtype=torch.float32) * std_b).to(dtype)
    return A, B


def gemv_bytes(M: int, K: int, N: int, groupsize: int = 128) -> int:
    """Algorithmic HBM bytes of one decode call: every operand read or written exactly once.

    qweight K*N/2 + qzeros K*N/(2*groupsize) + scales 2*K*N/groupsize + g_idx 4K + x 2MK + y 2MN.
    """
    G = math.ceil(K / groupsize)
    return K * N // 2 + G * N // 2 + 2 * G * N + 4 * K + 2 * M * K + 2 * M * N
