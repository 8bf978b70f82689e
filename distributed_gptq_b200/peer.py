"""Hessian accumulation across ranks by the kernel itself (``hessian_exchange = "peer"``).

The Hessian kernel adds its tiles with ``red.global.add`` and does not care whose memory the
target is: when every rank's ``add_batch`` is handed the *owner's* buffer (mapped into its own
address space over NVLink), ``H = Σ_r X_rᵀX_r`` is complete on the owner when the ranks' passes
are, the reduction rides inside the kernels' epilogues tile by tile, and the collective that
remains is a barrier (the reference all-reduces every Hessian after calibration,
``distributed/coordinator.py:218-225``).

The buffers come from one arena of symmetric memory (``torch.distributed._symmetric_memory``:
the same allocation on every rank, each mapped into every peer): one rendezvous per run
instead of one per Hessian.  An arena holds ``generations`` copies of a block's Hessians; the
driver hands generation ``b mod generations`` to block ``b`` and guarantees that the block
that used it before has been collected (its owner zeroes a Hessian as soon as the chain has
read it).  Only plain peer stores and reductions are used: no multicast object is bound
(``TORCH_SYMM_MEM_DISABLE_MULTICAST``), no load crosses the link.
"""
from __future__ import annotations

import logging
import os
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

logger = logging.getLogger(__name__)

# no multicast object is bound to the arena: nothing here uses multimem, and a rank that dies
# with memory bound to one takes its peers' links down with it.  Set before torch's symmetric
# memory allocator is first used.
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")

ALIGN = 256


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def slot_bytes(K8: int) -> int:
    return _round_up(K8 * K8 * 4, ALIGN)


def generation_layout(widths: List[int]) -> Tuple[List[int], int]:
    """Byte offsets of one block's Hessians (padded widths ``K8``) inside a generation, and
    the generation's size."""
    offsets, off = [], 0
    for K8 in widths:
        offsets.append(off)
        off += slot_bytes(K8)
    return offsets, off


class PeerArena:
    """One symmetric allocation of ``generations * generation_bytes`` bytes, zero-filled."""

    def __init__(self, device: torch.device, generation_bytes: int, generations: int):
        import torch.distributed._symmetric_memory as symm
        self.device = device
        self.generation_bytes = generation_bytes
        self.generations = generations
        self.rank = dist.get_rank()
        self.world = dist.get_world_size()
        total = generation_bytes * generations
        self.buf = symm.empty((total,), dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.group = dist.group.WORLD
        self.handle = symm.rendezvous(self.buf, self.group)
        self.dirty = False

    def view(self, rank: int, generation: int, offset: int, K8: int) -> torch.Tensor:
        """The ``K8 x K8`` fp32 Hessian at ``offset`` of ``generation`` in rank ``rank``'s
        arena, addressable from this rank's kernels."""
        byte0 = generation * self.generation_bytes + offset
        assert byte0 % 4 == 0 and offset + K8 * K8 * 4 <= self.generation_bytes
        if rank == self.rank:
            return self.buf[byte0:byte0 + K8 * K8 * 4].view(torch.float32).view(K8, K8)
        return self.handle.get_buffer(rank, (K8, K8), torch.float32, byte0 // 4)

    def fits(self, generation_bytes: int, generations: int) -> bool:
        return generation_bytes <= self.generation_bytes and generations <= self.generations

    def clear(self) -> None:
        self.buf.zero_()


def make_arena(device: torch.device, generation_bytes: int, generations: int,
               barrier) -> Optional[PeerArena]:
    """Collective: every rank calls it with the same sizes.  Returns ``None`` on every rank if
    the allocation or the rendezvous failed on any of them (``barrier``: the communication
    manager's host barrier, called once the arena is zeroed everywhere)."""
    arena, ok = None, 1
    try:
        arena = PeerArena(device, generation_bytes, generations)
        torch.cuda.synchronize(device)
    except Exception as exc:        # noqa: BLE001 - any failure means "not available here"
        logger.warning("symmetric memory is not available (%s); Hessians are reduced with NCCL",
                       str(exc).splitlines()[0] if str(exc) else type(exc).__name__)
        ok = 0
    flag = torch.tensor([ok], dtype=torch.int32, device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if int(flag.item()) == 0:
        return None
    barrier()
    return arena
