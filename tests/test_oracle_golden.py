"""The vectorised CPU oracle against the scalar golden fixtures (bit-exact) — no GPU."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import q4_oracle as orc

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _load(name):
    d = np.load(os.path.join(GOLD, name))
    return {k: d[k] for k in d.files}


def _bits(t):
    return t.contiguous().view(torch.int16)


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "recons_v2_*.npz"))))
def test_recons_v2_bit_exact(path):
    d = _load(os.path.basename(path))
    w = orc.recons_v2(torch.from_numpy(d["qweight"]), torch.from_numpy(d["scales"]),
                      torch.from_numpy(d["qzeros"]), torch.from_numpy(d["g_idx"]))
    want = torch.from_numpy(d["w"])
    nan = torch.isnan(want)
    assert torch.equal(torch.isnan(w), nan)
    assert torch.equal(_bits(w)[~nan], _bits(want)[~nan])


def test_recons2_v2_bit_exact():
    d = _load("recons2_v2_act_k128_n64_g32.npz")
    w = orc.recons2_v2(torch.from_numpy(d["qweight"]), torch.from_numpy(d["scales"]),
                       torch.from_numpy(d["qzeros"]), torch.from_numpy(d["g_idx"]))
    assert torch.equal(_bits(w), _bits(torch.from_numpy(d["w"])))


def test_recons_v1_bit_exact():
    d = _load("recons_v1_k128_n64.npz")
    w = orc.recons_v1(torch.from_numpy(d["qweight"]), torch.from_numpy(d["scales"]),
                      torch.from_numpy(d["zeros"]))
    assert torch.equal(_bits(w), _bits(torch.from_numpy(d["w"])))


@pytest.mark.parametrize("name", ["recons_v2_seq_k128_n64_g32.npz", "recons_v2_act_k128_n64_g32.npz",
                                  "recons_v2_act_k256_n32_g128.npz"])
def test_gemv_matches_scalar(name):
    d = _load(name)
    y = orc.gemv_fp32(torch.from_numpy(d["x"]), torch.from_numpy(d["qweight"]),
                      torch.from_numpy(d["scales"]), torch.from_numpy(d["qzeros"]),
                      torch.from_numpy(d["g_idx"]))
    want = torch.from_numpy(d["y"])
    assert torch.allclose(y, want, rtol=1e-10, atol=1e-10)


def test_fp32_scales_is_single_fma():
    """float scales: one fused multiply-subtract of a rounded zero term."""
    d = _load("recons_v2_act_k128_n64_g32.npz")
    s = torch.from_numpy(d["scales"]).float() * 1.2345
    w = orc.recons_v2(torch.from_numpy(d["qweight"]), s, torch.from_numpy(d["qzeros"]),
                      torch.from_numpy(d["g_idx"]))
    assert w.dtype == torch.float32
    q = orc.unpack_rows(torch.from_numpy(d["qweight"])).double()
    z1 = (orc.unpack_cols(torch.from_numpy(d["qzeros"])) + 1)
    gi = torch.from_numpy(d["g_idx"]).long()
    zero = (s[gi] * z1[gi].float())
    want = (s[gi].double() * q - zero.double()).float()
    assert torch.equal(w, want)


def test_pack_unpack_roundtrip():
    from alpaca_lora_4bit_b200 import synth
    g = torch.Generator().manual_seed(3)
    lev = torch.randint(0, 16, (64, 48), generator=g)
    assert torch.equal(orc.unpack_rows(synth.pack_rows(lev)), lev.int())
    assert torch.equal(orc.unpack_cols(synth.pack_cols(lev)), lev.int())
    lev2 = torch.randint(0, 4, (64, 48), generator=g)
    assert torch.equal(orc.unpack_rows(synth.pack_rows(lev2, 2), 2), lev2.int())
