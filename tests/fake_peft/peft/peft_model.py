from . import PeftType
from .tuners.lora import LoraModel

PEFT_TYPE_TO_MODEL_MAPPING = {PeftType.LORA: LoraModel}
