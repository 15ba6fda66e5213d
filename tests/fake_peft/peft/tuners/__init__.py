from . import lora  # noqa: F401
