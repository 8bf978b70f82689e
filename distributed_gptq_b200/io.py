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


def packed_shapes(name: str, N_out: int, K: int, bits: int, group_size: int, fmt: int):
    """``(key, shape, dtype)`` of the tensors :func:`packed_state` produces for a layer of
    ``N_out x K`` weights, bias aside, in its order: what a rank that did not quantize the
    layer needs to know to receive them."""
    row_bytes = _C.packed_row_bytes(K, bits, fmt)
    per_channel = group_size <= 0 or group_size >= K
    ng = 1 if per_channel else -(-K // group_size)
    qshape, qdtype = ((N_out, row_bytes // 4), torch.int32) if fmt == _C.FMT_INT32_LE \
        else ((N_out, row_bytes), torch.uint8)
    return [(f"{name}.qweight", qshape, qdtype),
            (f"{name}.scales", (N_out, ng), torch.float16),
            (f"{name}.zeros", (N_out, ng), torch.float16),
            (f"{name}.g_idx", (K,), torch.int32)]


# ----------------------------------------------------------------------------- per-block shards
def _settings(cfg) -> dict:
    return {"bits": cfg.bits, "group_size": cfg.group_size, "actorder": cfg.actorder,
            "percdamp": cfg.percdamp, "blocksize": cfg.blocksize,
            "true_sequential": cfg.true_sequential}


def save_block_shard(path, names, layers: Dict[str, nn.Module], results: Dict[str, dict],
                     leader: Dict[str, str], cfg) -> None:
    """Writes what one finished block produced - packed tensors, the dequantized weights the
    model now holds, error sums - so that a repeated run can skip the block.  The file is
    written under a temporary name and renamed, so a shard that exists is complete."""
    from safetensors.torch import save_file
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    tensors, errors = {}, {}
    for n in names:
        for k, v in results[n]["packed"].items():
            if not k.endswith(".bias"):
                tensors[k] = v.detach().cpu().contiguous()
        tensors[f"{n}.weight"] = layers[n].weight.data.detach().cpu().contiguous()
        errors[n] = results[n]["stats"]["total_error"]
    meta = {"settings": json.dumps(_settings(cfg)), "errors": json.dumps(errors),
            "leader": json.dumps({n: leader.get(n, n) for n in names})}
    tmp = path.with_suffix(".tmp")
    save_file(tensors, str(tmp), metadata=meta)
    tmp.replace(path)


def load_block_shard(path, layers: Dict[str, nn.Module], cfg, device) -> dict:
    """Reads a shard of :func:`save_block_shard`; raises if it was written with other
    settings or for other layers.  Returns ``{"results", "weights", "leader"}``."""
    from safetensors import safe_open
    out = {"results": {}, "weights": {}, "leader": {}}
    with safe_open(str(path), framework="pt", device="cpu") as f:
        meta = f.metadata() or {}
        if json.loads(meta.get("settings", "null")) != _settings(cfg):
            raise RuntimeError(f"{path} was written with other quantization settings; "
                               "remove the checkpoint directory or restore the settings")
        errors = json.loads(meta["errors"])
        out["leader"] = json.loads(meta["leader"])
        if set(errors) != set(layers):
            raise RuntimeError(f"{path} holds layers {sorted(errors)[:3]}..., expected "
                               f"{sorted(layers)[:3]}...")
        keys = set(f.keys())
        for n, layer in layers.items():
            packed = {k: f.get_tensor(k).to(device) for k in sorted(keys)
                      if k.rsplit(".", 1)[0] == n and not k.endswith(".weight")}
            bias = getattr(layer, "bias", None)
            if bias is not None:
                packed[f"{n}.bias"] = bias.data
            W = layer.weight.data.flatten(1) if layer.weight.dim() > 2 else layer.weight.data
            K = W.shape[1]
            per_channel = cfg.group_size <= 0 or cfg.group_size >= K
            ng = 1 if per_channel else -(-K // cfg.group_size)
            shape = torch.Size((W.shape[0], ng))
            out["results"][n] = {"packed": packed, "stats": {
                "bits": cfg.bits, "group_size": cfg.group_size, "total_error": errors[n],
                "compression_ratio": 32.0 / cfg.bits, "scale_shape": shape, "zero_shape": shape}}
            out["weights"][n] = f.get_tensor(f"{n}.weight")
    return out


def apply_block_weights(layers: Dict[str, nn.Module], shard: dict) -> None:
    for n, layer in layers.items():
        w = shard["weights"][n]
        layer.weight.data = w.to(device=layer.weight.device, dtype=layer.weight.dtype)


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


def _load_dequantized(name: str, module: nn.Module, info: dict, tensors: dict, device) -> None:
    qw = tensors.pop(f"{name}.qweight").to(device)
    fmt = _C.FMT_INT32_LE if qw.dtype == torch.int32 else _C.FMT_BYTES_LO_FIRST
    scales = tensors.pop(f"{name}.scales").to(device)
    zeros = tensors.pop(f"{name}.zeros").to(device)
    g_idx = tensors.pop(f"{name}.g_idx").to(device)
    w = _C.unpack_dequant(qw, scales, zeros, g_idx, info["in_features"], info["bits"],
                          info["group_size"], fmt, torch.float32)
    shape = info.get("weight_shape") or list(module.weight.shape)
    module.weight.data = w.reshape(shape).to(device=device, dtype=module.weight.dtype)
    if f"{name}.bias" in tensors and getattr(module, "bias", None) is not None:
        module.bias.data = tensors.pop(f"{name}.bias").to(device=device, dtype=module.bias.dtype)
    module.to(device)


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
        if info.get("kind", "linear") != "linear" or not isinstance(old, nn.Linear):
            # QuantizedLinear computes x @ Wq^T: a convolution (or any other module) keeps its
            # own forward and gets the dequantized weights back in its weight's shape
            _load_dequantized(name, old, info, tensors, device)
            continue
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
