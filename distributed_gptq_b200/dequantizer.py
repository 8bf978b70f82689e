"""Dequantization of packed layers and models (reference ``core/dequantizer.py``)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from . import _C


class GPTQDequantizer:
    """``(unpack(qweight) - zeros) * scales`` on the GPU (reference ``core/dequantizer.py:14-143``).

    ``qweight`` is in the ``QuantizedLinear`` layout (4-bit: two codes per byte, low
    nibble first; other widths: one code per byte); ``scales`` / ``zeros`` are
    ``(out, n_groups)`` (or ``(out,)`` / ``(out, 1)`` per channel); ``g_idx`` maps input
    columns to groups.
    """

    def __init__(self, bits: int = 4, group_size: int = 128):
        self.bits = bits
        self.group_size = group_size
        self.max_val = 2 ** bits - 1

    def _unpack_4bit(self, qweight: torch.Tensor) -> torch.Tensor:
        """uint8 nibble pairs -> float codes, low nibble = even column (reference ``:68-89``)."""
        cols = qweight.shape[1] * 2
        return _C.unpack(qweight, cols, 4, _C.FMT_BYTES_LO_FIRST).float()

    def dequantize_weight(self, qweight: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor,
                          g_idx: Optional[torch.Tensor] = None,
                          in_features: Optional[int] = None) -> torch.Tensor:
        out_f = qweight.shape[0]
        cols = in_features or (qweight.shape[1] * 2 if self.bits == 4 else qweight.shape[1])
        scales = scales.reshape(out_f, -1)
        zeros = zeros.reshape(out_f, -1)
        if zeros.dtype != scales.dtype:
            zeros = zeros.to(scales.dtype)
        if scales.dtype not in (torch.float32, torch.float16):
            scales, zeros = scales.float(), zeros.float()
        n_groups = scales.shape[1]
        if g_idx is not None and (g_idx.numel() != cols or int(g_idx.max()) >= n_groups):
            g_idx = None
        return _C.unpack_dequant(qweight, scales, zeros, g_idx, cols, self.bits, self.group_size,
                                 _C.FMT_BYTES_LO_FIRST, torch.float32)

    def dequantize_layer(self, layer: nn.Module) -> nn.Module:
        if not hasattr(layer, "qweight"):
            return layer
        weight = self.dequantize_weight(layer.qweight, layer.scales, layer.zeros,
                                        getattr(layer, "g_idx", None),
                                        getattr(layer, "in_features", None))
        bias = getattr(layer, "bias", None)
        new = nn.Linear(weight.shape[1], weight.shape[0], bias=bias is not None,
                        device=weight.device, dtype=weight.dtype)
        new.weight.data = weight
        if bias is not None:
            new.bias.data = bias.data.to(weight.dtype)
        return new

    def dequantize_model(self, model: nn.Module) -> nn.Module:
        for name, module in list(model.named_children()):
            if hasattr(module, "qweight"):
                setattr(model, name, self.dequantize_layer(module))
            else:
                self.dequantize_model(module)
        return model


def dequantize_model(model: nn.Module, bits: int = 4, group_size: int = 128) -> nn.Module:
    return GPTQDequantizer(bits=bits, group_size=group_size).dequantize_model(model)
