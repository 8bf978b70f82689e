"""Collectives used by the quantization path (reference
``src/distributed_gptq/distributed/communication.py:87-279``): thin wrappers over
``torch.distributed`` that are no-ops in a single process."""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


class CommunicationManager:
    """``all_reduce_tensor`` / ``broadcast_tensor`` / ``reduce_tensor`` / ``barrier`` on the
    default process group (NCCL over NVLink for CUDA tensors, gloo for CPU tensors)."""

    def __init__(self, rank: int = 0, world_size: int = 1):
        self.rank = rank
        self.world_size = world_size

    @property
    def active(self) -> bool:
        return self.world_size > 1 and dist.is_available() and dist.is_initialized()

    def all_reduce_tensor(self, tensor: torch.Tensor, op=dist.ReduceOp.SUM, async_op: bool = False):
        """In-place sum over ranks (reference ``communication.py:182-197``)."""
        if not self.active:
            return None if async_op else tensor
        work = dist.all_reduce(tensor, op=op, async_op=async_op)
        return work if async_op else tensor

    def reduce_tensor(self, tensor: torch.Tensor, dst: int, async_op: bool = False):
        """In-place sum onto rank ``dst`` only (the other ranks' buffers are left undefined)."""
        if not self.active:
            return None if async_op else tensor
        work = dist.reduce(tensor, dst=dst, op=dist.ReduceOp.SUM, async_op=async_op)
        return work if async_op else tensor

    def broadcast_tensor(self, tensor: torch.Tensor, src: int = 0, async_op: bool = False):
        """Reference ``communication.py:130-145``."""
        if not self.active:
            return None if async_op else tensor
        work = dist.broadcast(tensor, src=src, async_op=async_op)
        return work if async_op else tensor

    def broadcast_object(self, obj, src: int = 0):
        if not self.active:
            return obj
        box = [obj if self.rank == src else None]
        dist.broadcast_object_list(box, src=src)
        return box[0]

    def barrier(self) -> None:
        if self.active:
            dist.barrier()


def group_options(backend: str) -> dict:
    """Keyword arguments for ``init_process_group``: NCCL's own stream gets high priority, so
    that the blocks of a reduction or broadcast are scheduled as soon as thread blocks of the
    calibration pass retire instead of behind everything already resident."""
    if backend != "nccl" or not hasattr(dist, "ProcessGroupNCCL"):
        return {}
    return {"pg_options": dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)}


def setup_communication(rank: int, world_size: int, master_addr: str = "127.0.0.1",
                        master_port: str = "12355", backend: str = "nccl",
                        timeout_s: Optional[int] = None) -> CommunicationManager:
    """Initialises the default process group once (reference ``communication.py:358-380``)."""
    if world_size > 1 and not dist.is_initialized():
        import datetime
        kwargs = group_options(backend)
        if timeout_s:
            kwargs["timeout"] = datetime.timedelta(seconds=timeout_s)
        dist.init_process_group(backend=backend, init_method=f"tcp://{master_addr}:{master_port}",
                                rank=rank, world_size=world_size, **kwargs)
    return CommunicationManager(rank, world_size)
