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
reference's own dequantize-and-matmul branch computes.  A ``g_idx`` that is exactly
that sequential map is not passed on either, so that such layers take the kernel's
tensor-core path.

Act-order checkpoints carry a general map: every group has ``group_size`` columns, scattered
over the row.  For those (4-bit, ``group_size`` a multiple of 128) the columns are brought into
group order once per weight buffer - the reordered packed weights and the column order are
kept on the buffer object, which costs a second copy of the packed weights - and every call
gathers its activations into the same order, after which the layer is a sequential one and
takes the same path.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _C

_SCHEMA = "linear(Tensor x, Tensor qweight, Tensor scales, Tensor zeros, Tensor g_idx, Tensor? bias) -> Tensor"
_INVALID, _SEQUENTIAL, _GENERAL = 0, 1, 2
_lib = None


def _classify_g_idx(g_idx: torch.Tensor, n_groups: int) -> int:
    """Looks at the values once per buffer (one device synchronisation; the answer is kept on
    the tensor object together with its version counter): invalid group numbers, the
    sequential map ``c // group_size`` (which the kernels compute themselves, on their fastest
    path), or a general column-to-group map."""
    tag = getattr(g_idx, "_dgq_g_idx_kind", None)
    if tag is not None and tag[0] == g_idx._version and tag[1] == n_groups:
        return tag[2]
    K = g_idx.numel()
    if K == 0 or int(g_idx.max()) >= n_groups or int(g_idx.min()) < 0:
        kind = _INVALID
    else:
        group_size = -(-K // n_groups)
        seq = torch.arange(K, device=g_idx.device, dtype=g_idx.dtype) // group_size
        kind = _SEQUENTIAL if bool(torch.equal(g_idx.reshape(-1), seq)) else _GENERAL
    try:
        g_idx._dgq_g_idx_kind = (g_idx._version, n_groups, kind)
    except AttributeError:
        pass
    return kind


def _g_idx_usable(g_idx: torch.Tensor, n_groups: int) -> bool:
    return _classify_g_idx(g_idx, n_groups) != _INVALID


def _grouped_layout(qweight: torch.Tensor, g_idx: torch.Tensor, n_groups: int, K: int):
    """For a general ``g_idx`` whose groups all have the same size: ``(qweight with its columns
    in group order, the column order)``, computed once per pair of buffers; ``None`` when the
    groups are uneven."""
    tag = getattr(qweight, "_dgq_grouped", None)
    if tag is not None and tag[0] == (qweight._version, g_idx.data_ptr(), g_idx._version):
        return tag[1]
    group_size = K // n_groups
    out = None
    if n_groups * group_size == K:
        gi = g_idx.reshape(-1).long()
        counts = torch.bincount(gi, minlength=n_groups)
        if bool((counts == group_size).all()):
            order = torch.argsort(gi, stable=True).to(torch.int32)
            codes = _C.unpack(qweight, K, 4, _C.FMT_BYTES_LO_FIRST)
            grouped = _C.pack(_C.permute_cols(codes, order), 4, _C.FMT_BYTES_LO_FIRST)
            out = (grouped, order)
    try:
        qweight._dgq_grouped = ((qweight._version, g_idx.data_ptr(), g_idx._version), out)
    except AttributeError:
        pass
    return out


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
    gi = g_idx if _classify_g_idx(g_idx, n_groups) == _GENERAL else None
    if (gi is not None and four_bit and K % 128 == 0 and group_size % 128 == 0 and
            x.dtype in (torch.float16, torch.bfloat16)):
        layout = _grouped_layout(qweight, g_idx, n_groups, K)
        if layout is not None:
            grouped, order = layout
            x2 = x.reshape(-1, K)
            if x2.stride(-1) != 1:
                x2 = x2.contiguous()
            xg = _C.permute_cols(x2, order)
            y = _C.qlinear_forward(xg, grouped, scales, zeros, None, bias, K, 4, group_size)
            return y.reshape(*x.shape[:-1], y.shape[-1])
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
