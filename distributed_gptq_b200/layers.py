"""Quantized layers: ``QuantizedLinear`` in the reference's storage layout
(``src/distributed_gptq/models/layers.py:15-188``) with packing, dequantization and
the forward pass done by the CUDA library, and ``replace_with_quantized_layers``.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn as nn

from . import _C, ops


class QuantizedLinear(nn.Module):
    """Packed GPTQ linear layer.

    Buffers (reference ``models/layers.py:55-65``): ``qweight`` uint8
    ``(out, ceil(in/2))`` for 4-bit (low nibble = even column) else ``(out, in)``;
    ``scales`` / ``zeros`` fp16 ``(out, ceil(in/group_size))``; ``g_idx`` int32 ``(in)``,
    the group of every input column (the reference initialises it to the column
    index itself; here the default is ``column // group_size``); ``bias``.
    """

    def __init__(self, bits: int, group_size: int, in_features: int, out_features: int,
                 bias: bool = True):
        super().__init__()
        self.bits = bits
        self.group_size = group_size if group_size > 0 else in_features
        self.in_features = in_features
        self.out_features = out_features
        self.num_groups = math.ceil(in_features / self.group_size)
        if bits == 4:
            weight_shape = (out_features, math.ceil(in_features / 2))
        else:
            weight_shape = (out_features, in_features)
        self.register_buffer("qweight", torch.zeros(weight_shape, dtype=torch.uint8))
        self.register_buffer("scales", torch.zeros((out_features, self.num_groups), dtype=torch.float16))
        self.register_buffer("zeros", torch.zeros((out_features, self.num_groups), dtype=torch.float16))
        self.register_buffer("g_idx", (torch.arange(in_features) // self.group_size).to(torch.int32))
        if bias:
            self.register_parameter("bias", nn.Parameter(torch.zeros(out_features)))
        else:
            self.register_parameter("bias", None)

    def pack_weights(self, weight: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor,
                     g_idx: Optional[torch.Tensor] = None) -> None:
        """Stores uint8 codes ``(out, in)`` in the packed layout (reference ``:67-96``)."""
        dev = weight.device if weight.is_cuda else self.qweight.device
        if dev.type != "cuda":
            raise RuntimeError("QuantizedLinear.pack_weights needs a CUDA device")
        codes = weight.to(dev, torch.uint8)
        self.qweight = _C.pack(codes, self.bits, _C.FMT_BYTES_LO_FIRST)
        self.scales = scales.to(dev, torch.float16).reshape(self.out_features, -1).contiguous()
        self.zeros = zeros.to(dev, torch.float16).reshape(self.out_features, -1).contiguous()
        if g_idx is not None:
            self.g_idx = g_idx.to(dev, torch.int32).contiguous()
        else:
            self.g_idx = self.g_idx.to(dev)

    def unpack_weights(self) -> torch.Tensor:
        """fp32 ``(out, in)`` dequantized weights ``(code - zero) * scale`` (reference ``:98-138``)."""
        g_idx = self.g_idx if ops._g_idx_usable(self.g_idx, self.num_groups) else None
        return _C.unpack_dequant(self.qweight, self.scales, self.zeros, g_idx, self.in_features,
                                 self.bits, self.group_size, _C.FMT_BYTES_LO_FIRST, torch.float32)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return torch.ops.gptq.linear(x, self.qweight, self.scales, self.zeros, self.g_idx, self.bias)

    @classmethod
    def from_linear(cls, linear_layer: nn.Linear, bits: int = 4, group_size: int = 128
                    ) -> "QuantizedLinear":
        q = cls(bits=bits, group_size=group_size, in_features=linear_layer.in_features,
                out_features=linear_layer.out_features, bias=linear_layer.bias is not None)
        if linear_layer.bias is not None:
            q.bias.data = linear_layer.bias.data.clone()
        return q.to(linear_layer.weight.device)

    @classmethod
    def from_gptq(cls, gptq) -> "QuantizedLinear":
        """Builds the packed layer from a :class:`~distributed_gptq_b200.gptq.GPTQ` after ``quantize``."""
        lin = gptq.layer
        q = cls.from_linear(lin, gptq.bits, gptq.group_size)
        q.pack_weights(gptq.codes, gptq.scale, gptq.zero, gptq.g_idx)
        return q

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"bits={self.bits}, group_size={self.group_size}")


def replace_with_quantized_layers(model: nn.Module, bits: int = 4, group_size: int = 128,
                                  skip_layers: Optional[list] = None,
                                  quantizers: Optional[Dict[str, object]] = None,
                                  _prefix: str = "") -> nn.Module:
    """Swaps every ``nn.Linear`` for a ``QuantizedLinear`` (reference ``models/layers.py:285-315``).

    With ``quantizers`` (name -> quantized ``GPTQ`` object) the new layers are filled
    with the packed codes; without, they are created empty like the reference's.
    """
    skip = set(skip_layers or [])
    for name, child in list(model.named_children()):
        full = f"{_prefix}.{name}" if _prefix else name
        if isinstance(child, nn.Linear) and name not in skip and full not in skip:
            if quantizers is not None and full in quantizers:
                setattr(model, name, QuantizedLinear.from_gptq(quantizers[full]))
            elif quantizers is None:
                setattr(model, name, QuantizedLinear.from_linear(child, bits, group_size))
        else:
            replace_with_quantized_layers(child, bits, group_size, skip_layers, quantizers, full)
    return model
