"""The slice of ``peft.tuners.lora`` (0.6) that a module factory hook sees."""
import math
from dataclasses import dataclass, field
from typing import List

import torch
import torch.nn as nn


@dataclass
class LoraConfig:
    r: int = 8
    lora_alpha: int = 8
    target_modules: List[str] = field(default_factory=list)
    lora_dropout: float = 0.0
    fan_in_fan_out: bool = False
    init_lora_weights: bool = True
    bias: str = "none"


class LoraLayer:
    def __init__(self, in_features: int, out_features: int, **kwargs):
        self.r = {}
        self.lora_alpha = {}
        self.scaling = {}
        self.lora_dropout = nn.ModuleDict({})
        self.lora_A = nn.ModuleDict({})
        self.lora_B = nn.ModuleDict({})
        self.lora_embedding_A = nn.ParameterDict({})
        self.lora_embedding_B = nn.ParameterDict({})
        self._disable_adapters = False
        self.merged_adapters = []
        self._active_adapter = []
        self.in_features = in_features
        self.out_features = out_features
        self.kwargs = kwargs

    @property
    def disable_adapters(self):
        return self._disable_adapters

    @property
    def active_adapters(self):
        a = self._active_adapter
        return [a] if isinstance(a, str) else list(a)

    def update_layer(self, adapter_name, r, lora_alpha, lora_dropout, init_lora_weights):
        if r <= 0:
            raise ValueError(f"`r` should be a positive integer value but the value passed is {r}")
        self.r[adapter_name] = r
        self.lora_alpha[adapter_name] = lora_alpha
        self.lora_dropout[adapter_name] = nn.Dropout(p=lora_dropout) if lora_dropout > 0.0 else nn.Identity()
        self.lora_A[adapter_name] = nn.Linear(self.in_features, r, bias=False)
        self.lora_B[adapter_name] = nn.Linear(r, self.out_features, bias=False)
        self.scaling[adapter_name] = lora_alpha / r
        if init_lora_weights:
            nn.init.kaiming_uniform_(self.lora_A[adapter_name].weight, a=math.sqrt(5))
            nn.init.zeros_(self.lora_B[adapter_name].weight)

    def set_adapter(self, adapter_names):
        if isinstance(adapter_names, str):
            adapter_names = [adapter_names]
        self._active_adapter = list(adapter_names)


class Linear(nn.Linear, LoraLayer):
    def __init__(self, adapter_name, in_features, out_features, r=0, lora_alpha=1, lora_dropout=0.0, fan_in_fan_out=False,
                 is_target_conv_1d_layer=False, **kwargs):
        init_lora_weights = kwargs.pop("init_lora_weights", True)
        nn.Linear.__init__(self, in_features, out_features, **kwargs)
        LoraLayer.__init__(self, in_features=in_features, out_features=out_features)
        self.weight.requires_grad = False
        self.fan_in_fan_out = fan_in_fan_out
        self.update_layer(adapter_name, r, lora_alpha, lora_dropout, init_lora_weights)
        self.set_adapter(adapter_name)

    def forward(self, x):
        result = nn.functional.linear(x, self.weight, self.bias)
        for name in self.active_adapters:
            result = result + self.lora_B[name](self.lora_A[name](self.lora_dropout[name](x))) * self.scaling[name]
        return result


class LoraModel(nn.Module):
    """Walks the model and swaps every target for what ``_create_new_module`` returns, through
    ``_replace_module`` - the two hooks of PEFT 0.6 that a quant-aware subclass overrides."""

    def __init__(self, model, config, adapter_name):
        super().__init__()
        self.model = model
        self.peft_config = {adapter_name: config}
        for name, target in list(model.named_modules()):
            if not any(name == t or name.endswith("." + t) for t in config.target_modules):
                continue
            kwargs = {"r": config.r, "lora_alpha": config.lora_alpha, "lora_dropout": config.lora_dropout,
                      "fan_in_fan_out": config.fan_in_fan_out, "init_lora_weights": config.init_lora_weights}
            has_bias = getattr(target, "bias", None) is not None
            new_module = self._create_new_module(config, adapter_name, target, bias=has_bias, **kwargs)
            parent_name, _, leaf = name.rpartition(".")
            parent = model.get_submodule(parent_name) if parent_name else model
            self._replace_module(parent, leaf, new_module, target)
        for n, p in model.named_parameters():
            if "lora_" not in n:
                p.requires_grad = False

    @staticmethod
    def _create_new_module(lora_config, adapter_name, target, **kwargs):
        bias = kwargs.pop("bias", False)
        return Linear(adapter_name, target.in_features, target.out_features, bias=bias, **kwargs)

    @staticmethod
    def _replace_module(parent, child_name, new_module, child):
        setattr(parent, child_name, new_module)
        new_module.weight = child.weight
        if getattr(child, "bias", None) is not None:
            new_module.bias = child.bias

    def forward(self, *args, **kwargs):
        return self.model(*args, **kwargs)
