"""The PEFT hook (``GPTQLoraModel._create_new_module`` / ``_replace_module`` and
``replace_peft_model_with_int4_lora_model``) run against PEFT's own classes when ``peft`` is installed and
against ``tests/fake_peft`` (the 0.6 signatures of the few classes the hook touches) when it is not."""
import importlib
import os
import sys

import pytest
import torch
import torch.nn as nn

from alpaca_lora_4bit_b200 import autograd_4bit as a4, models, synth
from oracle import q4_oracle as orc
from tests import fake_backend

FAKE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "fake_peft")


@pytest.fixture
def peft_pkg():
    """The real package if there is one, else the stand-in, importable for the duration of the test."""
    try:
        import peft  # noqa: F401
        yield importlib.import_module("peft")
        return
    except ImportError:
        pass
    sys.path.insert(0, FAKE)
    try:
        yield importlib.import_module("peft")
    finally:
        sys.path.remove(FAKE)
        for name in [m for m in sys.modules if m == "peft" or m.startswith("peft.")]:
            del sys.modules[name]


def test_registry_and_factory_hooks_are_replaced(peft_pkg):
    from alpaca_lora_4bit_b200.monkeypatch.peft_tuners_lora_monkey_patch import replace_peft_model_with_int4_lora_model
    from peft.tuners.lora import LoraModel
    stock_create = LoraModel._create_new_module
    replace_peft_model_with_int4_lora_model()
    cls = peft_pkg.peft_model.PEFT_TYPE_TO_MODEL_MAPPING[peft_pkg.PeftType.LORA]
    assert cls.__name__ == "GPTQLoraModel" and issubclass(cls, LoraModel)
    assert LoraModel._create_new_module is not stock_create
    assert models.GPTQLoraModel.__name__ == "GPTQLoraModel"            # resolved lazily through the module attribute


def test_quant_linears_become_lora_layers_with_aliased_buffers(peft_pkg):
    if not hasattr(peft_pkg.tuners.lora, "LoraConfig") or "fake_peft" not in peft_pkg.__file__:
        pytest.skip("runs the model walk of the stand-in; the installed PEFT has its own")
    from alpaca_lora_4bit_b200.monkeypatch.peft_tuners_lora_monkey_patch import replace_peft_model_with_int4_lora_model
    from peft.tuners.lora import Linear as PeftLinear, LoraConfig
    replace_peft_model_with_int4_lora_model()
    cls = peft_pkg.peft_model.PEFT_TYPE_TO_MODEL_MAPPING[peft_pkg.PeftType.LORA]

    layer = synth.make_layer(256, 128, 64, act_order=True, seed=3)
    net = nn.Module()
    net.q_proj = a4.Autograd4bitQuantLinear(256, 128, groupsize=64)
    net.q_proj.qweight, net.q_proj.qzeros, net.q_proj.scales, net.q_proj.g_idx = layer.qweight, layer.qzeros, layer.scales, layer.g_idx
    net.q_proj.bias = torch.zeros(128, dtype=torch.float16)
    net.head = nn.Linear(128, 16, bias=True)
    net.untouched = nn.Linear(16, 16)
    net.forward = lambda x: net.head(net.q_proj(x).float())
    old_q, old_head_weight = net.q_proj, net.head.weight

    cls(net, LoraConfig(r=4, lora_alpha=8, target_modules=["q_proj", "head"], lora_dropout=0.0), "default")
    q = net.q_proj
    assert isinstance(q, models.Linear4bitLt) and q.groupsize == 64 and not q.is_v1_model
    for name in ("qweight", "qzeros", "scales", "g_idx", "bias"):       # aliased, not copied
        assert getattr(q, name).data_ptr() == getattr(old_q, name).data_ptr(), name
    assert q.r["default"] == 4 and q.scaling["default"] == 2.0 and q.active_adapters == ["default"]
    assert q.lora_A["default"].weight.device == q.qweight.device
    assert isinstance(net.head, PeftLinear) and net.head.weight is old_head_weight
    assert isinstance(net.untouched, nn.Linear) and not isinstance(net.untouched, PeftLinear)
    trainable = sorted(n for n, p in net.named_parameters() if p.requires_grad)
    assert trainable == ["head.lora_A.default.weight", "head.lora_B.default.weight",
                         "q_proj.lora_A.default.weight", "q_proj.lora_B.default.weight"]

    # the swapped layer computes base + LoRA
    A, B = synth.make_lora(256, 128, 4, seed=5, dtype=torch.float32)
    q.lora_A["default"].weight.data.copy_(A)
    q.lora_B["default"].weight.data.copy_(B)
    x = synth.make_acts(12, 256, 6)
    w = orc.recons_v2(layer.qweight, layer.scales, layer.qzeros, layer.g_idx).float()
    with fake_backend.installed(), torch.no_grad():
        y = q(x)
    ref = x.float() @ w + orc.lora_forward(x, A, B, 2.0)
    assert torch.allclose(y.float(), ref, atol=3e-2, rtol=1e-2)

    # a target the factory cannot wrap is refused
    net2 = nn.Module()
    net2.conv = nn.Conv1d(4, 4, 1)
    with pytest.raises(ValueError, match="not supported"):
        cls._create_new_module(LoraConfig(), "default", net2.conv, r=2, lora_alpha=2, lora_dropout=0.0, fan_in_fan_out=False)
