"""Model-level driver: ``QuantizationConfig``, ``DistributedGPTQuantizer`` and
``quantize_model_simple`` (reference ``src/distributed_gptq/core/quantizer.py``).

Differences in mechanism, not in interface: Hessians are accumulated inside the forward
hooks (the reference stores every layer's inputs on the host first,
``core/quantizer.py:194-246``); layers that receive the same input tensor share one
Hessian; with several ranks the calibration sequences are split, partial Hessians are
reduced to the rank that owns a layer and layers are quantized in parallel across ranks.
"""
from __future__ import annotations

import json
import logging
import time
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Callable, Dict, Iterable, List, Optional, Union

import torch
import torch.nn as nn

from . import _C, io
from .coordinator import (DistributedConfig, DistributedGPTQCoordinator, assign_owners,
                          create_distributed_config, layer_cost)
from .gptq import GPTQ
from .streams import ChainPool

logger = logging.getLogger(__name__)


@dataclass
class QuantizationConfig:
    """Reference ``core/quantizer.py:24-40``.  ``group_size = -1`` (one scale/zero per output
    channel) is accepted in addition; ``use_triton`` is accepted and ignored."""
    bits: int = 4
    group_size: int = 128
    actorder: bool = False
    percdamp: float = 0.01
    blocksize: int = 128
    calibration_samples: int = 128
    use_triton: bool = False
    save_packed: bool = True

    def validate(self):
        assert self.bits in [2, 3, 4, 8], f"Bits must be 2, 3, 4, or 8, got {self.bits}"
        assert self.group_size > 0 or self.group_size == -1, \
            f"Group size must be positive (or -1 for per-channel), got {self.group_size}"
        assert 0 <= self.percdamp <= 1, f"Percdamp must be between 0 and 1, got {self.percdamp}"
        assert 0 < self.blocksize <= 128, f"Blocksize must be in 1..128, got {self.blocksize}"


# ----------------------------------------------------------------------------- calibration data
def _split_samples(batch) -> List:
    """One calibration batch -> list of single-sequence samples (batch dimension kept, size 1)."""
    if isinstance(batch, dict):
        n = next(iter(batch.values())).shape[0]
        return [{k: (v[i:i + 1] if torch.is_tensor(v) and v.dim() > 0 and v.shape[0] == n else v)
                 for k, v in batch.items()} for i in range(n)]
    if isinstance(batch, (list, tuple)):
        batch = batch[0]
    if batch.dim() == 1:
        batch = batch.unsqueeze(0)
    return [batch[i:i + 1] for i in range(batch.shape[0])]


def calibration_samples(data, limit: int) -> List:
    """Normalises what callers pass as calibration data - a list of batches, one ``[N, ...]``
    tensor, or any iterable of batches such as a ``DataLoader`` - to at most ``limit``
    single-sequence samples.  (The reference wraps a list in ``TensorDataset(*list)``, which
    treats the batches as parallel fields, ``core/quantizer.py:186``; the intent is a list
    of batches.)"""
    out: List = []
    batches: Iterable = [data] if torch.is_tensor(data) else data
    for b in batches:
        out.extend(_split_samples(b))
        if len(out) >= limit:
            break
    return out[:limit]


def _merge(samples: List):
    if isinstance(samples[0], dict):
        return {k: (torch.cat([s[k] for s in samples]) if torch.is_tensor(samples[0][k]) and
                    samples[0][k].dim() > 0 else samples[0][k]) for k in samples[0]}
    return torch.cat(samples)


def _same_shape(a, b) -> bool:
    if isinstance(a, dict):
        return all((not torch.is_tensor(a[k])) or a[k].shape == b[k].shape for k in a)
    return a.shape == b.shape


class DistributedGPTQuantizer:
    """Reference ``core/quantizer.py:43-355``."""

    def __init__(self, quantization_config: Optional[QuantizationConfig] = None,
                 distributed_config: Optional[DistributedConfig] = None,
                 calibration_batch_size: int = 8):
        self.quant_config = quantization_config or QuantizationConfig()
        self.quant_config.validate()
        self.dist_config = distributed_config or create_distributed_config()
        self.coordinator = DistributedGPTQCoordinator(self.dist_config)
        self.calibration_batch_size = calibration_batch_size
        self.quantized_layers: Dict[str, dict] = {}
        self.quantization_errors: Dict[str, float] = {}
        self.packed: Dict[str, Dict[str, torch.Tensor]] = {}
        self.layer_info: Dict[str, dict] = {}
        self.timings: Dict[str, float] = {}
        # diagnostics: when set before quantize_model, the reduced raw Hessian of every layer
        # this rank quantizes is kept (on the host) in `hessians`
        self.keep_hessians = False
        self._pool: Optional[ChainPool] = None
        self.hessians: Dict[str, torch.Tensor] = {}

    # ------------------------------------------------------------------ discovery
    def _find_layers_to_quantize(self, model: nn.Module) -> Dict[str, nn.Module]:
        """Every ``nn.Linear`` / ``nn.Conv2d`` with more than 1000 weights
        (reference ``core/quantizer.py:167-179``)."""
        layers = {}
        for name, module in model.named_modules():
            if isinstance(module, (nn.Linear, nn.Conv2d)) and module.weight.numel() > 1000:
                layers[name] = module
        return layers

    # ------------------------------------------------------------------ calibration
    @torch.no_grad()
    def _accumulate_hessians(self, model: nn.Module, samples: List,
                             layers: Dict[str, nn.Module]) -> Dict[str, GPTQ]:
        cfg = self.quant_config
        dev = self.coordinator.device
        quantizers = {name: GPTQ(layer, bits=cfg.bits, group_size=cfg.group_size,
                                 actorder=cfg.actorder, percdamp=cfg.percdamp,
                                 blocksize=cfg.blocksize, device=dev)
                      for name, layer in layers.items()}
        leader: Dict[str, str] = {}     # layer -> layer whose Hessian it shares
        seen: List = []                 # (input tensor, layer name) of the current forward
        first = {"on": True}

        def make_hook(name):
            def hook(module, args):
                inp = args[0] if isinstance(args, tuple) else args
                if first["on"]:
                    for t, owner in seen:
                        if (t.data_ptr() == inp.data_ptr() and t.shape == inp.shape and
                                t.stride() == inp.stride() and t.dtype == inp.dtype):
                            leader[name] = owner
                            break
                    else:
                        leader[name] = name
                        seen.append((inp, name))   # holding the tensor keeps its address unique
                if leader.get(name, name) == name:
                    quantizers[name].add_batch(inp.detach(), None)
            return hook

        handles = [layer.register_forward_pre_hook(make_hook(n)) for n, layer in layers.items()]
        try:
            i = 0
            while i < len(samples):
                j = i + 1
                while (j < len(samples) and j - i < self.calibration_batch_size and
                       _same_shape(samples[i], samples[j])):
                    j += 1
                batch = _merge(samples[i:j])
                if isinstance(batch, dict):
                    model(**{k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in batch.items()})
                else:
                    model(batch.to(dev))
                seen.clear()
                first["on"] = False
                i = j
        finally:
            for h in handles:
                h.remove()
        self._leader = {n: leader.get(n, n) for n in layers}
        return quantizers

    # ------------------------------------------------------------------ main entry
    def quantize_model(self, model: nn.Module,
                       calibration_data: Union[List[torch.Tensor], torch.Tensor, Iterable],
                       layers_to_quantize: Optional[Union[List[str], Dict[str, nn.Module]]] = None,
                       save_path: Optional[str] = None,
                       progress_callback: Optional[Callable] = None) -> nn.Module:
        """Quantizes ``model`` in place and returns it (reference ``core/quantizer.py:79-165``).

        ``layers_to_quantize``: list of module names, a ``{name: module}`` dict, or ``None`` for
        every linear/conv layer above 1000 weights.  ``progress_callback(done, total, name,
        stats)`` is called on rank 0 after each layer."""
        start = time.time()
        cfg, co = self.quant_config, self.coordinator
        with co.distributed_context():
            _C.device_check()
            model = co.prepare_model(model)
            model.eval()
            if layers_to_quantize is None:
                layers = self._find_layers_to_quantize(model)
            elif isinstance(layers_to_quantize, dict):
                layers = dict(layers_to_quantize)
            else:
                mods = dict(model.named_modules())
                layers = {n: mods[n] for n in layers_to_quantize}
            logger.info("Found %d layers to quantize", len(layers))

            samples = calibration_samples(calibration_data, cfg.calibration_samples)
            if not samples:
                raise ValueError("no calibration data")
            n_global = len(samples)
            samples = co.shard_calibration(samples)

            t0 = time.time()
            quantizers = self._accumulate_hessians(model, samples, layers)
            torch.cuda.synchronize(co.device)
            self.timings["calibration_s"] = time.time() - t0

            # ---- exchange: partial Hessians -> owners
            t0 = time.time()
            names = list(layers)
            groups: Dict[str, List[str]] = {}
            for n in names:
                groups.setdefault(self._leader[n], []).append(n)
            leaders = list(groups)
            costs = [sum(layer_cost(*quantizers[m]._weight_matrix().shape) for m in groups[g])
                     for g in leaders]
            world = self.dist_config.world_size
            owners_list = assign_owners(costs, world) if self.dist_config.hessian_exchange == "owner" \
                else [self.dist_config.rank] * len(leaders)
            owner_of_group = dict(zip(leaders, owners_list))
            if world > 1:
                for g in leaders:   # a rank whose shard was empty still needs a buffer to reduce
                    q = quantizers[g]
                    if q._Hbuf is None:
                        K8 = (q.columns + 7) // 8 * 8
                        q._Hbuf = torch.zeros((K8, K8), dtype=torch.float32, device=co.device)
                co.exchange_hessians({g: quantizers[g]._Hbuf for g in leaders}, owner_of_group)
            for g in leaders:
                quantizers[g].nsamples = n_global
            self.timings["exchange_s"] = time.time() - t0

            # ---- quantize the layers this rank owns
            t0 = time.time()
            all_reduce_mode = self.dist_config.hessian_exchange != "owner" or world == 1
            results: Dict[str, dict] = {}
            # The layers of a stage are independent once their Hessians are complete: their
            # chains (damped inverse, block quantization, packing) are enqueued on side
            # streams, where they run beside each other, and collected afterwards.
            if self._pool is None:      # made once: the caching allocator pools memory per stream
                self._pool = ChainPool(co.device, n_streams=4)
            pool = self._pool
            launched = []
            for g in leaders:
                mine = all_reduce_mode or owner_of_group[g] == self.dist_config.rank
                if mine:
                    for n in groups[g]:
                        q = quantizers[n]
                        if n != g:
                            q._Hbuf, q.nsamples = quantizers[g]._Hbuf, n_global
                        if self.keep_hessians:
                            self.hessians[n] = q.H.detach().cpu().clone()

                        def chain(n=n, q=q):
                            q.quantize_launch()
                            return io.packed_state(n, q, io.file_format(cfg.bits))

                        launched.append((n, g, q, pool.submit(chain)))
            for n, g, q, fut in launched:
                packed = fut.result()
                stats = q.quantize_finish()
                for t in packed.values():
                    t.record_stream(torch.cuda.current_stream(co.device))
                results[n] = {"stats": stats, "packed": packed}
                q.codes = None
                if n != g:
                    q._Hbuf = None
            pool.join()
            for g in leaders:
                quantizers[g].free_hessian()
            torch.cuda.synchronize(co.device)
            self.timings["quantize_s"] = time.time() - t0

            # ---- share results: every rank ends with the same quantized model
            t0 = time.time()
            for idx, n in enumerate(names):
                g = self._leader[n]
                layer = layers[n]
                if not all_reduce_mode:
                    src = owner_of_group[g]
                    entry = results.get(n)
                    shapes = co.comm.broadcast_object(
                        {k: (tuple(v.shape), v.dtype) for k, v in entry["packed"].items()}
                        if entry else None, src=src)
                    stats = co.comm.broadcast_object(entry["stats"] if entry else None, src=src)
                    if entry is None:
                        entry = {"stats": stats, "packed": {
                            k: (layer.bias.data if k.endswith(".bias")      # not quantized: local copy
                                else torch.empty(s, dtype=d, device=co.device))
                            for k, (s, d) in shapes.items()}}
                        results[n] = entry
                    for k in sorted(entry["packed"]):
                        if not k.endswith(".bias"):
                            co.comm.broadcast_tensor(entry["packed"][k], src=src)
                    co.comm.broadcast_tensor(layer.weight.data, src=src)
                entry = results[n]
                self.quantized_layers[n] = entry["stats"]
                self.quantization_errors[n] = entry["stats"].get("total_error", 0)
                self.packed[n] = entry["packed"]
                W = layer.weight.data.flatten(1) if layer.weight.dim() > 2 else layer.weight.data
                self.layer_info[n] = {"bits": cfg.bits, "group_size": cfg.group_size,
                                      "out_features": W.shape[0], "in_features": W.shape[1],
                                      "packing": "int32_le" if io.file_format(cfg.bits) == _C.FMT_INT32_LE
                                      else "bytes_lo_first"}
                if progress_callback and self.dist_config.rank == 0:
                    progress_callback(idx + 1, len(names), n, entry["stats"])
            self.timings["share_s"] = time.time() - t0
            self.timings["total_s"] = time.time() - start
            if self.dist_config.rank == 0:
                self._log_quantization_summary(time.time() - start)
            if save_path:
                self.save_quantized_model(model, save_path)
        return model

    # ------------------------------------------------------------------ save / load
    def _metadata(self) -> dict:
        return {"quantization_config": asdict(self.quant_config),
                "quantized_layers": list(self.quantized_layers.keys()),
                "quantization_errors": self.quantization_errors,
                "layers": self.layer_info}

    def save_quantized_model(self, model: nn.Module, save_path: str,
                             save_format: str = "safetensors") -> None:
        """Rank 0 writes the packed file and its JSON sidecar (reference
        ``core/quantizer.py:248-291``).  With ``save_packed=False`` the float state dict (the
        dequantized weights) is written instead."""
        if self.dist_config.rank != 0:
            return
        path = Path(save_path)
        if save_format == "safetensors" and self.quant_config.save_packed:
            io.save_packed(path, model, self.packed, self._metadata())
        elif save_format == "safetensors":
            from safetensors.torch import save_file
            path.parent.mkdir(parents=True, exist_ok=True)
            save_file({k: v.detach().cpu().contiguous().clone() for k, v in model.state_dict().items()},
                      str(path))
            json.dump(self._metadata(), open(path.with_suffix(".json"), "w"), indent=2)
        else:
            data = self._metadata()
            data["model_state_dict"] = model.state_dict()
            data["packed"] = self.packed
            path.parent.mkdir(parents=True, exist_ok=True)
            torch.save(data, path)
        logger.info("Saved quantized model to %s", path)

    def load_quantized_model(self, model: nn.Module, load_path: str,
                             load_format: str = "safetensors") -> nn.Module:
        """Loads a packed file into ``model``: its quantized layers become ``QuantizedLinear``
        modules (reference ``core/quantizer.py:293-335`` reloads a float state dict)."""
        if load_format != "safetensors":
            ckpt = torch.load(load_path, map_location="cpu")
            model.load_state_dict(ckpt["model_state_dict"])
            meta = ckpt
        else:
            meta = io.load_packed(load_path, model, self.coordinator.device)
        self.quant_config = QuantizationConfig(**meta["quantization_config"])
        self.quantized_layers = {n: {} for n in meta["quantized_layers"]}
        self.quantization_errors = meta["quantization_errors"]
        return model

    def _log_quantization_summary(self, elapsed: float) -> None:
        n = len(self.quantization_errors)
        avg = sum(self.quantization_errors.values()) / n if n else 0.0
        logger.info("Quantized %d layers to %d bits (group %d) in %.2f s; average error %.6f; "
                    "peak GPU memory %.2f GB", n, self.quant_config.bits,
                    self.quant_config.group_size, elapsed, avg,
                    self.coordinator.get_memory_stats()["max_allocated_gb"])


GPTQQuantizer = DistributedGPTQuantizer   # the name the reference imports but never defines


def quantize_model_simple(model: nn.Module, calibration_data, bits: int = 4,
                          save_path: Optional[str] = None) -> nn.Module:
    """Reference ``core/quantizer.py:358-383``."""
    quantizer = DistributedGPTQuantizer(QuantizationConfig(bits=bits))
    return quantizer.quantize_model(model, calibration_data, save_path=save_path)
