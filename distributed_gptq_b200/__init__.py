"""B200-native GPTQ quantization path behind the Python API of Distributed_GPTQ.

Every computation runs in hand-written sm_100a CUDA kernels reached through the
C ABI declared in ``include/dgq.h``; there is no CPU or eager-PyTorch fallback.
Importing the package registers ``torch.ops.gptq.linear``.
"""
from . import ops as _ops
from .communication import CommunicationManager, setup_communication
from .coordinator import (DistributedConfig, DistributedGPTQCoordinator, QuantizationMode,
                          create_distributed_config)
from .dequantizer import GPTQDequantizer, dequantize_model
from .gptq import GPTQ, Quantizer, quantize_layer_gptq
from .kernels import dequantize_tensor, quantize_tensor
from .layers import QuantizedLinear, replace_with_quantized_layers
from .quantizer import (DistributedGPTQuantizer, GPTQQuantizer, QuantizationConfig,
                        quantize_model_simple)
from .streams import ChainPool

_ops.register()

__all__ = [
    "GPTQ", "Quantizer", "quantize_layer_gptq", "QuantizationConfig", "DistributedGPTQuantizer",
    "GPTQQuantizer", "quantize_model_simple", "DistributedConfig", "QuantizationMode",
    "DistributedGPTQCoordinator", "create_distributed_config", "CommunicationManager",
    "setup_communication", "QuantizedLinear", "replace_with_quantized_layers", "GPTQDequantizer",
    "dequantize_model", "quantize_tensor", "dequantize_tensor", "ChainPool",
]
__version__ = "0.1.0"
