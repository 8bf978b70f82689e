"""Registers ``torch.ops.gptq.linear``, the operator the reference's
``QuantizedLinear.forward`` dispatches to (``models/layers.py:150-153``):

    torch.ops.gptq.linear(x, qweight, scales, zeros, g_idx, bias) -> Tensor

The operator receives no bit width or group size, so they are read off the buffer
shapes of the ``QuantizedLinear`` layout: ``in_features = g_idx.numel()``; a
``qweight`` with ``ceil(in_features / 2)`` columns holds 4-bit nibble pairs, any
other holds one code per byte; ``n_groups = scales.shape[1]``.  ``g_idx`` is used
as the group of every input column when its values are valid group numbers; the
reference's constructor default ``range(in_features)`` is not, and then groups are
runs of ``in_features // n_groups`` consecutive columns, which is what the
reference's own dequantize-and-matmul branch computes.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from . import _C

_SCHEMA = "linear(Tensor x, Tensor qweight, Tensor scales, Tensor zeros, Tensor g_idx, Tensor? bias) -> Tensor"
_g_idx_valid: Dict[Tuple[int, int, int], bool] = {}
_lib = None


def _g_idx_usable(g_idx: torch.Tensor, n_groups: int) -> bool:
    key = (g_idx.data_ptr(), g_idx._version, n_groups)
    ok = _g_idx_valid.get(key)
    if ok is None:
        ok = bool(g_idx.numel() > 0 and int(g_idx.max()) < n_groups and int(g_idx.min()) >= 0)
        if len(_g_idx_valid) > 4096:
            _g_idx_valid.clear()
        _g_idx_valid[key] = ok
    return ok


def gptq_linear(x: torch.Tensor, qweight: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor,
                g_idx: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    K = g_idx.numel()
    if x.shape[-1] != K:
        raise RuntimeError(f"gptq::linear: x has {x.shape[-1]} features, g_idx describes {K}")
    four_bit = qweight.shape[1] != K and qweight.shape[1] == (K + 1) // 2
    if not four_bit and qweight.shape[1] != K:
        raise RuntimeError("gptq::linear: qweight is neither nibble-packed nor one byte per code")
    n_groups = scales.shape[1]
    group_size = -(-K // n_groups)
    gi = g_idx if _g_idx_usable(g_idx, n_groups) else None
    return _C.qlinear_forward(x, qweight, scales, zeros, gi, bias, K, 4 if four_bit else 8,
                              group_size)


def register() -> None:
    """Defines ``gptq::linear`` once per process and binds the CUDA implementation."""
    global _lib
    if _lib is not None:
        return
    try:
        lib = torch.library.Library("gptq", "DEF")
        lib.define(_SCHEMA)
    except RuntimeError:
        # the namespace/op already exists (another package defined it): add our kernel to it
        lib = torch.library.Library("gptq", "FRAGMENT")
        try:
            lib.define(_SCHEMA)
        except RuntimeError:
            pass
    lib.impl("linear", gptq_linear, "CUDA")
    _lib = lib
