"""Regenerates the golden fixtures in this directory:  python tests/golden/make_golden.py

The reference cannot be imported or built unmodified in a sandbox without its pinned
dependencies, so the fixtures are produced by an independent scalar evaluation of the kernel
formulas, one element at a time in Python floats with ``struct``'s IEEE half rounding (no torch
arithmetic, no vectorisation), following

  * VecQuant4ReconsV2Kernel  quant_cuda_kernel.cu:1127-1153
  * VecQuant4ReconsV1Kernel  quant_cuda_kernel.cu:1076-1097
  * VecQuant2ReconsV2Kernel  quant_cuda_kernel.cu:1185-1211
  * VecQuant4MatMulKernel    quant_cuda_kernel.cu:475-536 (real-valued sum, float64)

The vectorised oracle (oracle/q4_oracle.py) and the CUDA kernels are both tested against these
files.  Inputs are drawn by alpaca_lora_4bit_b200.synth with the seeds written below.
"""
from __future__ import annotations

import os
import struct
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from alpaca_lora_4bit_b200 import synth  # noqa: E402


def h(v: float) -> float:
    """Round a Python float to the nearest IEEE binary16 value (ties to even)."""
    return struct.unpack("e", struct.pack("e", v))[0]


def f32(v: float) -> float:
    return struct.unpack("f", struct.pack("f", v))[0]


def field(word: int, idx: int, bits: int) -> int:
    return ((word & 0xFFFFFFFF) >> (idx * bits)) & ((1 << bits) - 1)


def scalar_recons_v2(layer, bits=4):
    per = 32 // bits
    K, N = layer.K, layer.N
    qw = layer.qweight.tolist()
    qz = layer.qzeros.tolist()
    sc = layer.scales.float().tolist()
    gi = layer.g_idx.tolist()
    out = np.zeros((K, N), dtype=np.float16)
    for k in range(K):
        g = gi[k]
        for n in range(N):
            s = sc[g][n]
            z1 = field(qz[g][n // per], n % per, bits) + 1
            q = field(qw[k // per][n], k % per, bits)
            zero = h(s * z1)
            out[k, n] = h(h(s * q) - zero)
    return out


def scalar_recons_v1(qweight, scales, zeros):
    R, N = qweight.shape
    qw = qweight.tolist()
    sc = scales.float().reshape(-1).tolist()
    ze = zeros.float().reshape(-1).tolist()
    out = np.zeros((R * 8, N), dtype=np.float16)
    for k in range(R * 8):
        for n in range(N):
            out[k, n] = h(h(sc[n] * field(qw[k // 8][n], k % 8, 4)) - ze[n])
    return out


def scalar_gemv(layer, x):
    K, N = layer.K, layer.N
    qw = layer.qweight.tolist()
    qz = layer.qzeros.tolist()
    sc = layer.scales.float().tolist()
    gi = layer.g_idx.tolist()
    xs = x.float().tolist()
    out = np.zeros((len(xs), N), dtype=np.float64)
    for b in range(len(xs)):
        for n in range(N):
            acc = 0.0
            for k in range(K):
                g = gi[k]
                s = sc[g][n]
                z1 = field(qz[g][n // 8], n % 8, 4) + 1
                q = field(qw[k // 8][n], k % 8, 4)
                acc += (s * q - s * z1) * xs[b][k]
            out[b, n] = acc
    return out


def save_layer(prefix, layer, **extra):
    np.savez_compressed(
        os.path.join(HERE, prefix + ".npz"),
        qweight=layer.qweight.numpy(), qzeros=layer.qzeros.numpy(),
        scales=layer.scales.numpy(), g_idx=layer.g_idx.numpy(),
        K=layer.K, N=layer.N, groupsize=layer.groupsize, bits=layer.bits, **extra)


def main():
    # 4-bit v2, sequential groups and act-order, tiny group so several groups are exercised
    for name, K, N, g, act, seed in [
        ("recons_v2_seq_k128_n64_g32", 128, 64, 32, False, 11),
        ("recons_v2_act_k128_n64_g32", 128, 64, 32, True, 12),
        ("recons_v2_act_k256_n32_g128", 256, 32, 128, True, 13),
    ]:
        layer = synth.make_layer(K, N, g, act, seed)
        x = synth.make_acts(3, K, seed + 100)
        save_layer(name, layer, w=scalar_recons_v2(layer), x=x.numpy(), y=scalar_gemv(layer, x))
        print("wrote", name)

    # hand-made corner values: scale extremes incl. subnormal products, all levels, all zeros
    layer = synth.make_layer(64, 32, 32, True, 14)
    sc = layer.scales.clone()
    sc[0, :8] = torch.tensor([6.0e-8, 1.0e-7, 6.1e-5, 6.2e-5, 1e-4, 0.5, 100.0, 2048.0]).half()
    sc[1, :4] = torch.tensor([-0.01, -6.0e-8, 0.0, 65504.0 / 16]).half()
    layer.scales = sc
    save_layer("recons_v2_corner_k64_n32_g32", layer, w=scalar_recons_v2(layer))
    print("wrote corner")

    # 2-bit v2
    layer = synth.make_layer(128, 64, 32, True, 15, bits=2)
    save_layer("recons2_v2_act_k128_n64_g32", layer, w=scalar_recons_v2(layer, bits=2))
    print("wrote 2-bit")

    # v1 (per-column float scale / zero)
    gen = torch.Generator().manual_seed(16)
    base = synth.make_layer(128, 64, 128, False, 16)
    sc1 = (torch.rand((64, 1), generator=gen) * 0.018 + 0.002).half()
    ze1 = (sc1.float() * torch.randint(1, 16, (64, 1), generator=gen)).half()
    np.savez_compressed(os.path.join(HERE, "recons_v1_k128_n64.npz"),
                        qweight=base.qweight.numpy(), scales=sc1.numpy(), zeros=ze1.numpy(),
                        w=scalar_recons_v1(base.qweight, sc1, ze1))
    print("wrote v1")


if __name__ == "__main__":
    main()
