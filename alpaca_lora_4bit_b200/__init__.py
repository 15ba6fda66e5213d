"""B200-native int4 (GPTQ) dequant-matmul path behind the alpaca_lora_4bit operator surface.

Submodules mirror the reference package: ``quant_cuda`` (kernel entry points),
``matmul_utils_4bit`` (dispatch), ``autograd_4bit`` (module + autograd function), ``models``
(LoRA-wrapped quant linear) and ``model_attn_mlp_patch`` (fused qkv / gate-up patches).
All of them call hand-written sm_100a kernels in ``libq4b200.so`` through a C ABI; there is
no CPU or library fallback, and a missing library raises at first use.
"""
__version__ = "0.1.0"
