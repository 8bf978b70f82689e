"""Distributed coordination of the quantization path (reference
``src/distributed_gptq/distributed/coordinator.py``).

Two things shard.  Calibration is data-parallel: rank r runs the replicated model on
sequences r, r+W, ... (the ``DistributedSampler(shuffle=False)`` split of the reference,
``coordinator.py:164-169``) and accumulates partial Hessians, which are sums and so
reduce with one collective per Hessian.  Quantization is layer-parallel: every linear
layer has one owning rank, chosen by a deterministic cost-balanced placement, and only
the owner needs the reduced Hessian (``reduce`` instead of the reference's
``all_reduce``, ``coordinator.py:224``) and runs the quantizer; results are then
broadcast from the owner (the reference broadcasts rank 0's copy of every parameter,
``coordinator.py:231-233``).
"""
from __future__ import annotations

import contextlib
import datetime
import os
from dataclasses import dataclass
from enum import Enum
from typing import Dict, List, Sequence, Union

import torch
import torch.distributed as dist

from .communication import CommunicationManager, group_options


class QuantizationMode(Enum):
    SINGLE_GPU = "single_gpu"
    DATA_PARALLEL = "data_parallel"
    MODEL_PARALLEL = "model_parallel"
    PIPELINE_PARALLEL = "pipeline_parallel"


@dataclass
class DistributedConfig:
    mode: QuantizationMode = QuantizationMode.SINGLE_GPU
    world_size: int = 1
    rank: int = 0
    local_rank: int = 0
    master_addr: str = "localhost"
    master_port: str = "12355"
    backend: str = "nccl"
    init_timeout: int = 1800
    # extension: "owner" reduces each Hessian to the rank that quantizes the layer and
    # spreads the layers over the ranks; "all_reduce" reproduces the reference's flow
    # (every rank receives every Hessian and quantizes every layer); "peer" is "owner" with
    # the sum over ranks done by the Hessian kernels themselves, which accumulate straight
    # into the owner's buffer over NVLink (block-wise driver; see peer.py).
    hessian_exchange: str = "owner"

    @property
    def is_distributed(self) -> bool:
        return self.world_size > 1

    @property
    def is_main_process(self) -> bool:
        return self.rank == 0


def create_distributed_config(mode: Union[str, QuantizationMode] = "auto") -> DistributedConfig:
    """From the environment torchrun sets (reference ``coordinator.py:264-301``)."""
    world_size = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    master_addr = os.environ.get("MASTER_ADDR", "localhost")
    master_port = os.environ.get("MASTER_PORT", "12355")
    if mode == "auto":
        mode = QuantizationMode.SINGLE_GPU if world_size == 1 else QuantizationMode.DATA_PARALLEL
    elif isinstance(mode, str):
        mode = QuantizationMode(mode)
    return DistributedConfig(mode=mode, world_size=world_size, rank=rank, local_rank=local_rank,
                             master_addr=master_addr, master_port=master_port)


# ----------------------------------------------------------------------------- pure host logic
def shard_indices(n_items: int, rank: int, world_size: int) -> List[int]:
    """Indices of the calibration sequences rank ``rank`` processes: r, r+W, r+2W, ...
    (``DistributedSampler(shuffle=False)`` without its padding: no sequence is counted twice)."""
    return list(range(rank, n_items, world_size))


def layer_cost(out_features: int, in_features: int) -> float:
    """Relative cost of quantizing one layer: the inverse factor (~K^3) plus the column
    loop and its trailing updates (~N_out K^2)."""
    return 0.7 * float(in_features) ** 3 + float(out_features) * float(in_features) ** 2


def assign_owners(costs: Sequence[float], world_size: int) -> List[int]:
    """Deterministic longest-processing-time-first placement: heaviest layer first, each to
    the least loaded rank (ties to the lowest rank).  Unlike the reference's
    ``hash(name) % n_devices`` (``core/gptq.py:323``) it does not depend on the process."""
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    load = [0.0] * world_size
    owner = [0] * len(costs)
    for i in order:
        r = min(range(world_size), key=lambda k: (load[k], k))
        owner[i] = r
        load[r] += costs[i]
    return owner


class DistributedGPTQCoordinator:
    """Process-group set-up, device choice and the collectives of the path
    (reference ``coordinator.py:50-262``)."""

    def __init__(self, config: DistributedConfig):
        self.config = config
        self.device = torch.device("cuda", config.local_rank) if torch.cuda.is_available() \
            else torch.device("cpu")
        self.comm = CommunicationManager(config.rank, config.world_size)
        self._owns_group = False
        self.is_initialized = False

    def initialize(self) -> None:
        """One ``init_process_group`` (the reference calls it twice, ``coordinator.py:75`` and
        ``communication.py:118``); a group created by the launcher is reused."""
        if self.is_initialized:
            return
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        if self.config.is_distributed and not dist.is_initialized():
            addr = "127.0.0.1" if self.config.master_addr == "localhost" else self.config.master_addr
            backend = self.config.backend if self.device.type == "cuda" else "gloo"
            dist.init_process_group(
                backend=backend, init_method=f"tcp://{addr}:{self.config.master_port}",
                rank=self.config.rank, world_size=self.config.world_size,
                timeout=datetime.timedelta(seconds=self.config.init_timeout),
                **group_options(backend))
            self._owns_group = True
        self.is_initialized = True

    def cleanup(self) -> None:
        if self._owns_group and dist.is_initialized():
            dist.destroy_process_group()
            self._owns_group = False
        self.is_initialized = False

    @contextlib.contextmanager
    def distributed_context(self):
        self.initialize()
        try:
            yield self
        finally:
            self.cleanup()

    def prepare_model(self, model: torch.nn.Module) -> torch.nn.Module:
        """Moves the replica to this rank's device.  No DDP wrap: calibration only runs
        forward passes, and wrapping renames the modules the hooks look up
        (reference ``coordinator.py:121-145``)."""
        return model.to(self.device)

    def shard_calibration(self, samples: Sequence) -> List:
        idx = shard_indices(len(samples), self.config.rank, self.config.world_size)
        return [samples[i] for i in idx]

    def distribute_calibration_data(self, dataloader):
        """This rank's share of the calibration data (reference ``coordinator.py:147-181``).
        A ``DataLoader`` comes back as a ``DataLoader`` over the same dataset restricted to
        items r, r+W, ... (the reference's ``DistributedSampler(shuffle=False)`` split, without
        the duplicates it pads with); any other sequence comes back as the list of its items
        r, r+W, ....  A single process gets its argument back."""
        if not self.config.is_distributed:
            return dataloader
        from torch.utils.data import DataLoader, Subset
        if isinstance(dataloader, DataLoader):
            idx = shard_indices(len(dataloader.dataset), self.config.rank, self.config.world_size)
            return DataLoader(Subset(dataloader.dataset, idx), batch_size=dataloader.batch_size,
                              shuffle=False, num_workers=dataloader.num_workers,
                              collate_fn=dataloader.collate_fn, pin_memory=dataloader.pin_memory)
        return self.shard_calibration(list(dataloader))

    def quantize_layer_distributed(self, layer: torch.nn.Module, layer_inputs, quantization_config):
        """One layer, every rank holding part of its inputs (reference
        ``coordinator.py:183-235``): each rank accumulates the Hessian of its ``layer_inputs``,
        the partial Hessians are summed over the ranks (``coordinator.py:224``), every rank
        quantizes with the complete Hessian and ends with the same weights, and the stats are
        returned.  ``quantization_config`` is the reference's dict (``bits``, ``group_size``,
        optional ``actorder`` / ``percdamp`` / ``blocksize``) or a ``QuantizationConfig``.
        Differences: no forward of the layer is run (its output is not used), and the sample
        count is summed too, so shards of unequal size are weighted correctly (the reference
        divides by the world size, which is right for equal shards only); the rank-0 broadcast
        of ``coordinator.py:231-233`` is kept so that ranks cannot drift apart."""
        from .gptq import GPTQ
        cfg = quantization_config if isinstance(quantization_config, dict) else \
            {k: getattr(quantization_config, k) for k in
             ("bits", "group_size", "actorder", "percdamp", "blocksize")}
        self.initialize()
        gptq = GPTQ(layer, bits=cfg["bits"], group_size=cfg["group_size"],
                    actorder=cfg.get("actorder", False), percdamp=cfg.get("percdamp", 0.01),
                    blocksize=cfg.get("blocksize", 128), device=self.device)
        for inp in layer_inputs:
            gptq.add_batch(inp.to(self.device), None)
        if self.comm.active:
            if gptq._Hbuf is None:      # an empty shard still takes part in the sum
                K8 = (gptq.columns + 7) // 8 * 8
                gptq._Hbuf = torch.zeros((K8, K8), dtype=torch.float32, device=self.device)
            self.comm.all_reduce_tensor(gptq._Hbuf)
            n = torch.tensor([float(gptq.nsamples)], device=self.device)
            self.comm.all_reduce_tensor(n)
            gptq.nsamples = int(n.item())
        stats = gptq.quantize()
        self.last_gptq = gptq       # codes / scale / zero / g_idx for pack_weights()
        if self.comm.active:
            for _, param in layer.named_parameters():
                self.comm.broadcast_tensor(param.data, src=0)
        return stats

    # -- the exchange step ------------------------------------------------------------------
    def exchange_hessians(self, hessians: Dict[str, torch.Tensor], owners: Dict[str, int]) -> None:
        """Sums every partial Hessian over the ranks: onto its owner (``hessian_exchange ==
        "owner"``) or onto everybody.  Collectives are issued in the dict's order, which
        must be the same on every rank, asynchronously, and awaited together."""
        if not self.comm.active:
            return
        pending = []
        for name, H in hessians.items():
            if self.config.hessian_exchange == "all_reduce":
                pending.append(self.comm.all_reduce_tensor(H, async_op=True))
            else:
                pending.append(self.comm.reduce_tensor(H, dst=owners[name], async_op=True))
        for w in pending:
            if w is not None:
                w.wait()

    def get_memory_stats(self) -> Dict[str, float]:
        if self.device.type != "cuda":
            return {"allocated_gb": 0.0, "reserved_gb": 0.0, "max_allocated_gb": 0.0}
        return {"allocated_gb": torch.cuda.memory_allocated(self.device) / 1e9,
                "reserved_gb": torch.cuda.memory_reserved(self.device) / 1e9,
                "max_allocated_gb": torch.cuda.max_memory_allocated(self.device) / 1e9}
