"""rustgrad_b200: B200-native GGUF-quantized Llama inference behind rustgrad's session facade.

The compute path is ``librg_b200.so`` (hand-written sm_100a CUDA behind the C ABI of
``include/rg_b200.h``); anything that computes raises ImportError when that library is missing.
"""
from . import quant, synth, gguf_writer  # noqa: F401  (offline writer tools, no device work)

__all__ = ["quant", "synth", "gguf_writer"]
