"""B200-native GPTQ quantization path behind the Python API of Distributed_GPTQ.

Every computation runs in hand-written sm_100a CUDA kernels reached through the
C ABI declared in ``include/dgq.h``; there is no CPU or eager-PyTorch fallback.
"""
from .gptq import GPTQ, Quantizer, quantize_layer_gptq

__all__ = ["GPTQ", "Quantizer", "quantize_layer_gptq"]
__version__ = "0.1.0"
