"""Installs the quant-aware LoRA model into PEFT's registry
(monkeypatch/peft_tuners_lora_monkey_patch.py:1-9).  Needs ``peft``; raises ImportError without it."""


def replace_peft_model_with_int4_lora_model():
    import peft.peft_model
    from peft import PeftType
    from peft.tuners.lora import LoraModel

    from ..models import _gptq_lora_model
    cls = _gptq_lora_model()
    peft.peft_model.PEFT_TYPE_TO_MODEL_MAPPING[PeftType.LORA] = cls
    LoraModel._create_new_module = cls._create_new_module
    LoraModel._replace_module = cls._replace_module
    print('Replaced _create_new_module and _replace_module of peft LoraModel')
