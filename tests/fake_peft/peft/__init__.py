"""Test-only stand-in for the parts of PEFT 0.6 that the int4 LoRA hook touches: ``PeftType``, the
``PEFT_TYPE_TO_MODEL_MAPPING`` registry and ``tuners.lora.{LoraLayer, Linear, LoraModel, LoraConfig}`` with the
0.6 call signatures.  It lives outside the import path; ``tests/test_peft_hook_cpu.py`` puts it there for the
duration of one test when the real package is not installed."""
import enum


class PeftType(str, enum.Enum):
    LORA = "LORA"


from . import peft_model, tuners  # noqa: E402,F401
from .tuners.lora import LoraConfig, LoraModel  # noqa: E402,F401
