"""Packed safetensors output of a quantized model and its loader.

File layout: for every quantized layer ``<name>`` the tensors ``<name>.qweight``,
``<name>.scales`` (fp16, ``(out, n_groups)``), ``<name>.zeros`` (fp16), ``<name>.g_idx``
(int32, ``(in)``) and, if the layer has one, ``<name>.bias`` - the buffers of
``QuantizedLinear`` (reference ``models/layers.py:55-65``); every other entry of the
model's ``state_dict`` is stored unchanged.  ``qweight`` is uint8: nibble pairs, low
nibble = even column, for 4-bit and one code per byte for 8-bit; 2- and 3-bit codes are
stored as int32 words, first code in the low bits (16 resp. 10 codes per word).  A JSON
sidecar ``<path>.json`` carries the reference's keys (``quantization_config``,
``quantized_layers``, ``quantization_errors``; reference ``core/quantizer.py:264-279``)
plus ``layers``: bits, group size, shape and packing of each layer.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict

import torch
import torch.nn as nn

from . import _C
from .layers import QuantizedLinear


def file_format(bits: int) -> int:
    return _C.FMT_BYTES_LO_FIRST if bits in (4, 8) else _C.FMT_INT32_LE


def packed_state(name: str, gptq, fmt: int) -> Dict[str, torch.Tensor]:
    """The tensors written for one quantized layer."""
    out = {
        f"{name}.qweight": _C.pack(gptq.codes, gptq.bits, fmt),
        f"{name}.scales": gptq.scale.to(torch.float16),
        f"{name}.zeros": gptq.zero.to(torch.float16),
        f"{name}.g_idx": gptq.g_idx.to(torch.int32),
    }
    bias = getattr(gptq.layer, "bias", None)
    if bias is not None:
        out[f"{name}.bias"] = bias.data
    return out


def save_packed(path, model: nn.Module, packed: Dict[str, Dict[str, torch.Tensor]],
                meta: dict) -> None:
    """Writes ``path`` (safetensors) and ``path.json``.  ``packed`` maps layer name to the
    tensors of :func:`packed_state`; the layers' float weights are left out of the file."""
    from safetensors.torch import save_file
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    skip = {f"{n}.weight" for n in packed} | {f"{n}.bias" for n in packed}
    tensors = {}
    for k, v in model.state_dict().items():
        if k not in skip:
            tensors[k] = v.detach().cpu().contiguous().clone()   # clone: tied weights share storage
    for entry in packed.values():
        for k, v in entry.items():
            tensors[k] = v.detach().cpu().contiguous()
    save_file(tensors, str(path))
    with open(path.with_suffix(".json"), "w") as f:
        json.dump(meta, f, indent=2)


def load_packed(path, model: nn.Module, device=None) -> dict:
    """Replaces the quantized layers of ``model`` by ``QuantizedLinear`` modules holding the
    stored codes and loads every other tensor.  Returns the sidecar's content."""
    from safetensors.torch import load_file
    path = Path(path)
    meta = json.load(open(path.with_suffix(".json")))
    tensors = load_file(str(path))
    device = torch.device(device) if device is not None else torch.device("cuda")
    for name, info in meta["layers"].items():
        parent_name, _, child = name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        old = getattr(parent, child)
        has_bias = f"{name}.bias" in tensors
        q = QuantizedLinear(bits=info["bits"], group_size=info["group_size"],
                            in_features=info["in_features"], out_features=info["out_features"],
                            bias=has_bias).to(device)
        qw = tensors.pop(f"{name}.qweight").to(device)
        if qw.dtype == torch.int32:   # 2-/3-bit words -> one code per byte, the layer's layout
            qw = _C.unpack(qw, info["in_features"], info["bits"], _C.FMT_INT32_LE)
        q.qweight = qw.contiguous()
        q.scales = tensors.pop(f"{name}.scales").to(device)
        q.zeros = tensors.pop(f"{name}.zeros").to(device)
        q.g_idx = tensors.pop(f"{name}.g_idx").to(device)
        if has_bias:
            q.bias.data = tensors.pop(f"{name}.bias").to(device=device, dtype=q.bias.dtype)
        del old
        setattr(parent, child, q)
    missing = model.load_state_dict(tensors, strict=False)
    unexpected = [k for k in missing.unexpected_keys]
    if unexpected:
        raise RuntimeError(f"unexpected tensors in {path}: {unexpected[:5]}")
    return meta
