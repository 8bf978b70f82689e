"""Tensor-level helpers with the names of the reference's ``kernels`` package
(``kernels/__init__.py:8-22``, ``kernels/triton_kernels.py:377-481``), backed by the
CUDA library instead of Triton."""
from __future__ import annotations

from typing import Tuple

import torch

from . import _C


def quantize_tensor(tensor: torch.Tensor, bits: int = 4, group_size: int = 128
                    ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Flat round-to-nearest: returns ``(codes uint8 like tensor, scales, zeros)`` with one
    scale/zero per run of ``group_size`` consecutive elements of the flattened tensor."""
    x = tensor.cuda().float().contiguous()
    scales, zeros = _C.rtn_find_params(x, bits, group_size)
    q = _C.rtn_quantize(x, scales, zeros, bits, group_size)
    return q, scales, zeros


def dequantize_tensor(quantized_tensor: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor,
                      group_size: int = 128) -> torch.Tensor:
    q = quantized_tensor.cuda()
    if q.dtype != torch.uint8:
        q = q.to(torch.int16).remainder(256).to(torch.uint8)   # int8 storage wraps codes >= 128
    return _C.rtn_dequantize(q, scales.cuda(), zeros.cuda(), group_size)


def check_triton_availability() -> bool:
    """Kept for callers of the reference API: this package never uses Triton."""
    return False
