"""Model-level driver: ``QuantizationConfig``, ``DistributedGPTQuantizer`` and
``quantize_model_simple`` (reference ``src/distributed_gptq/core/quantizer.py``).

Differences in mechanism, not in interface:

* Hessians are accumulated inside forward hooks (the reference stores every layer's inputs
  on the host first, ``core/quantizer.py:194-246``); layers that receive the same input
  tensor share one Hessian and are quantized as one stacked matrix.
* A model whose quantized layers sit in a ``ModuleList`` of blocks applied one after the
  other (every decoder-only transformer) is calibrated block by block: the inputs of the
  first block are captured once, then every block is run over all calibration batches and
  its outputs are kept as the next block's inputs.  A block's Hessians are therefore
  complete when its pass ends, and their exchange between ranks, the damped inverse and the
  block quantization of that block run on side streams while the next block's pass keeps
  the tensor cores busy; only one or two blocks' Hessians are alive at a time.  Other models
  take one whole-model pass per batch and quantize afterwards.
* With several ranks the calibration sequences are split, partial Hessians are reduced to
  the rank that owns a layer group, owners quantize in parallel and every block's results
  travel in one flat buffer per owner.
* ``true_sequential=True`` re-runs every block with its quantized weights before the next
  block is calibrated (what the reference's CLI flag ``--true-sequential`` promises,
  ``cli.py:207-211``); ``checkpoint_dir`` writes one shard per finished block and skips the
  blocks already present when the run is repeated (``README.md:18``).
"""
from __future__ import annotations

import inspect
import json
import logging
import time
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Callable, Dict, Iterable, List, Optional, Tuple, Union

import torch
import torch.nn as nn

from . import _C, io, peer
from .coordinator import (DistributedConfig, DistributedGPTQCoordinator,
                          create_distributed_config, layer_cost)
from .gptq import GPTQ, quantize_group_launch
from .streams import ChainPool

logger = logging.getLogger(__name__)


@dataclass
class QuantizationConfig:
    """Reference ``core/quantizer.py:24-40``.  ``group_size = -1`` (one scale/zero per output
    channel) is accepted in addition; ``use_triton`` is accepted and ignored.
    ``true_sequential`` and ``checkpoint_dir`` are the two modes described in the module
    docstring."""
    bits: int = 4
    group_size: int = 128
    actorder: bool = False
    percdamp: float = 0.01
    blocksize: int = 128
    calibration_samples: int = 128
    use_triton: bool = False
    save_packed: bool = True
    true_sequential: bool = False
    checkpoint_dir: Optional[str] = None

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


def make_batches(samples: List, batch_size: int) -> List:
    """Consecutive samples of equal shape are merged, up to ``batch_size`` per batch."""
    out, i = [], 0
    while i < len(samples):
        j = i + 1
        while j < len(samples) and j - i < batch_size and _same_shape(samples[i], samples[j]):
            j += 1
        out.append(_merge(samples[i:j]))
        i = j
    return out


class _StopForward(Exception):
    """Raised by a hook to leave a forward pass that has delivered what was wanted."""


def find_blocks(model: nn.Module, layers: Dict[str, nn.Module]) -> Optional[Tuple[str, nn.ModuleList]]:
    """The ``ModuleList`` (two entries or more) that contains the most of ``layers``, with its
    name; ``None`` if no list contains any."""
    best, best_count = None, 0
    for name, mod in model.named_modules():
        if isinstance(mod, nn.ModuleList) and len(mod) >= 2:
            prefix = name + "." if name else ""
            count = sum(1 for n in layers
                        if n.startswith(prefix) and n[len(prefix):].split(".", 1)[0].isdigit())
            if count > best_count:
                best, best_count = (name, mod), count
    return best


def _align(n: int, a: int = 16) -> int:
    return (n + a - 1) // a * a


class _Group:
    """The layers of one block that share one Hessian, and what became of them."""

    def __init__(self, leader: str, members: List[str], quantizers: Dict[str, GPTQ]):
        self.leader = leader
        self.members = members
        self.q = [quantizers[m] for m in members]
        self.owner = 0
        self.mine = True
        self.future = None          # chain enqueued -> (device status tensors, packed dicts)
        self.reduce_work = None
        self.peer = False           # Hessian accumulated in the owner's buffer by every rank


class DistributedGPTQuantizer:
    """Reference ``core/quantizer.py:43-355``."""

    def __init__(self, quantization_config: Optional[QuantizationConfig] = None,
                 distributed_config: Optional[DistributedConfig] = None,
                 calibration_batch_size: int = 8, blockwise: Union[str, bool] = "auto",
                 share_weights: bool = True, blocks_in_flight: Optional[int] = None):
        self.quant_config = quantization_config or QuantizationConfig()
        self.quant_config.validate()
        self.dist_config = distributed_config or create_distributed_config()
        self.coordinator = DistributedGPTQCoordinator(self.dist_config)
        self.calibration_batch_size = calibration_batch_size
        # "auto": block by block when the model has a list of blocks (see find_blocks) and the
        # replay of its first block reproduces the second block's input; False: always one
        # whole-model pass per batch
        self.blockwise = blockwise
        # several ranks: ship the dequantized weights with the packed results, so that every
        # rank ends with the same model (the reference's behaviour, coordinator.py:231-233);
        # False leaves the weights of layers another rank quantized untouched on this rank
        self.share_weights = share_weights
        # block-wise, one-shot: how many blocks may have their chains enqueued but their results
        # not collected.  The host stands still in a collect, and the main stream runs dry if
        # that lasts longer than the passes queued ahead; with many ranks a block's pass is
        # short against its exchange + chain + broadcast, so more blocks are kept in flight
        # (each holds its Hessians on their owners: 0.7 GB for a Llama-7B block).
        if blocks_in_flight is None:
            blocks_in_flight = 2 if self.dist_config.world_size <= 2 else 4
        self.blocks_in_flight = max(1, int(blocks_in_flight))
        self.quantized_layers: Dict[str, dict] = {}
        self.quantization_errors: Dict[str, float] = {}
        self.packed: Dict[str, Dict[str, torch.Tensor]] = {}
        self.layer_info: Dict[str, dict] = {}
        self.timings: Dict[str, float] = {}
        # diagnostics: when set before quantize_model, the reduced raw Hessian of every layer
        # this rank quantizes is kept (on the host) in `hessians`
        self.keep_hessians = False
        # when set, CUDA events are recorded around the phases and summed into `timings`
        self.profile = False
        self._pool: Optional[ChainPool] = None
        self._share_stream: Optional[torch.cuda.Stream] = None
        self._xchg_stream: Optional[torch.cuda.Stream] = None
        self.hessians: Dict[str, torch.Tensor] = {}
        self._leader: Dict[str, str] = {}
        self.mode_used: Optional[str] = None
        # hessian_exchange == "peer": symmetric buffers, the grouping of a block learned from
        # the first one, and how many blocks have been given a generation of buffers
        self._arena: Optional[peer.PeerArena] = None
        self._arena_failed = False
        self._group_pattern: Optional[Dict[str, str]] = None
        self._peer_counter = 0
        self.peer_groups = 0        # groups of the last run whose Hessians were summed by the kernels

    # ------------------------------------------------------------------ discovery
    def _find_layers_to_quantize(self, model: nn.Module) -> Dict[str, nn.Module]:
        """Every ``nn.Linear`` / ``nn.Conv2d`` with more than 1000 weights
        (reference ``core/quantizer.py:167-179``)."""
        layers = {}
        for name, module in model.named_modules():
            if isinstance(module, (nn.Linear, nn.Conv2d)) and module.weight.numel() > 1000:
                layers[name] = module
        return layers

    # ------------------------------------------------------------------ hooks
    def _new_quantizers(self, layers: Dict[str, nn.Module]) -> Dict[str, GPTQ]:
        cfg, dev = self.quant_config, self.coordinator.device
        return {name: GPTQ(layer, bits=cfg.bits, group_size=cfg.group_size, actorder=cfg.actorder,
                           percdamp=cfg.percdamp, blocksize=cfg.blocksize, device=dev)
                for name, layer in layers.items()}

    def _hook_layers(self, layers: Dict[str, nn.Module], quantizers: Dict[str, GPTQ],
                     state: dict):
        """Forward pre-hooks that feed ``add_batch``.  During the first pass (``state["first"]``)
        layers that receive the very same tensor are grouped under the first of them (its
        ``leader``); only leaders accumulate.  ``state["accumulate"] = False`` makes a pass that
        only discovers the grouping."""
        leader: Dict[str, str] = state.setdefault("leader", {})
        seen: List = state.setdefault("seen", [])

        def make_hook(name):
            def hook(module, args):
                inp = args[0] if isinstance(args, tuple) else args
                if state["first"]:
                    for t, owner in seen:
                        if (t.data_ptr() == inp.data_ptr() and t.shape == inp.shape and
                                t.stride() == inp.stride() and t.dtype == inp.dtype):
                            leader[name] = owner
                            break
                    else:
                        leader[name] = name
                        seen.append((inp, name))   # holding the tensor keeps its address unique
                if leader.get(name, name) == name and state.get("accumulate", True):
                    quantizers[name].add_batch(inp.detach(), None)
            return hook

        return [layer.register_forward_pre_hook(make_hook(n)) for n, layer in layers.items()]

    def _to_device(self, batch):
        dev = self.coordinator.device
        if isinstance(batch, dict):
            return {k: (v.to(dev, non_blocking=True) if torch.is_tensor(v) else v)
                    for k, v in batch.items()}
        return batch.to(dev, non_blocking=True)

    def _run_model(self, model: nn.Module, batch, extra: dict):
        batch = self._to_device(batch)
        if isinstance(batch, dict):
            return model(**{**extra, **batch})
        return model(batch, **extra)

    @staticmethod
    def _forward_extras(model: nn.Module) -> dict:
        """Keyword arguments added to every calibration forward: a model that can build a
        key/value cache is told not to (it would hold every batch's keys and values)."""
        try:
            params = inspect.signature(model.forward).parameters
        except (TypeError, ValueError):
            return {}
        return {"use_cache": False} if "use_cache" in params else {}

    # ------------------------------------------------------------------ whole-model calibration
    @torch.no_grad()
    def _accumulate_hessians(self, model: nn.Module, batches: List,
                             layers: Dict[str, nn.Module], discovery_batch=None) -> Dict[str, GPTQ]:
        quantizers = self._new_quantizers(layers)
        state = {"first": True}
        extra = self._forward_extras(model)
        handles = self._hook_layers(layers, quantizers, state)
        try:
            if not batches and discovery_batch is not None:
                # this rank's shard is empty: one pass over a sample every rank has, so that the
                # grouping (hence the order and size of the collectives) is the same everywhere
                state["accumulate"] = False
                self._run_model(model, discovery_batch, extra)
                state["seen"].clear()
                state["first"] = False
            for batch in batches:
                self._run_model(model, batch, extra)
                state["seen"].clear()
                state["first"] = False
        finally:
            for h in handles:
                h.remove()
        self._leader.update({n: state["leader"].get(n, n) for n in layers})
        return quantizers

    # ------------------------------------------------------------------ block-wise calibration
    @torch.no_grad()
    def _capture_block_inputs(self, model: nn.Module, blocks: nn.ModuleList, batches: List,
                              outside: Dict[str, nn.Module], outside_q: Dict[str, GPTQ],
                              state: dict, stop_early: bool, probe: bool = False):
        """Runs the model on every batch up to its first block and records what the block is
        called with.  With ``probe`` the pass goes on to the second block, whose input is
        returned too (to check the replay of the first block), and stops there.  Layers outside
        the blocks are calibrated here when the pass may not stop early."""
        captured: List[Tuple[tuple, dict]] = []
        seen_h1: Dict[str, torch.Tensor] = {}

        def first_hook(module, args, kwargs):
            captured.append((tuple(a.detach() if torch.is_tensor(a) else a for a in args),
                             dict(kwargs)))
            if stop_early and not probe:
                raise _StopForward()

        def second_hook(module, args, kwargs):
            h = args[0] if args else kwargs.get("hidden_states")
            seen_h1["h1"] = h.detach()
            raise _StopForward()

        handles = [blocks[0].register_forward_pre_hook(first_hook, with_kwargs=True)]
        if probe:
            handles.append(blocks[1].register_forward_pre_hook(second_hook, with_kwargs=True))
        elif not stop_early:
            handles += self._hook_layers(outside, outside_q, state)
        extra = self._forward_extras(model)
        try:
            for batch in batches:
                try:
                    self._run_model(model, batch, extra)
                except _StopForward:
                    pass
                if not probe:
                    state.setdefault("seen", []).clear()
                    state["first"] = False
        finally:
            for h in handles:
                h.remove()
        return captured, seen_h1.get("h1")

    @staticmethod
    def _block_call(block: nn.Module, h: torch.Tensor, args: tuple, kwargs: dict) -> torch.Tensor:
        kw = dict(kwargs)
        if "past_key_values" in kw:
            kw["past_key_values"] = None
        if "use_cache" in kw:
            kw["use_cache"] = False
        if args:
            out = block(h, *args[1:], **kw)
        else:
            kw["hidden_states"] = h
            out = block(**kw)
        return out[0] if isinstance(out, (tuple, list)) else out

    # ------------------------------------------------------------------ exchange, chains, sharing
    def _dispatch(self, groups: List[_Group], load: List[float],
                  after: Optional[torch.cuda.Event] = None) -> None:
        """Places the groups on ranks (greedy on the cumulative load, heaviest first), starts
        the reduction of their Hessians and enqueues the owners' chains on the side streams.
        ``after``: the event that marks the Hessians complete on the main stream; without it
        everything queued on the main stream so far is waited for."""
        cfg, co, dc = self.quant_config, self.coordinator, self.dist_config
        world, rank = dc.world_size, dc.rank
        owner_mode = dc.hessian_exchange in ("owner", "peer") and world > 1
        costs = [sum(layer_cost(*q._weight_matrix().shape) for q in g.q) for g in groups]
        order = sorted(range(len(groups)), key=lambda i: (-costs[i], i))
        for i in order:
            g = groups[i]
            if g.peer:              # owner chosen before the pass (_peer_prepare)
                continue
            if owner_mode:
                g.owner = min(range(world), key=lambda k: (load[k], k))
                load[g.owner] += costs[i]
                g.mine = g.owner == rank
            else:
                # the reference's flow (coordinator.py:224-233): every rank receives the whole
                # Hessian and quantizes, then rank 0's result is what all ranks keep
                g.owner = 0
                g.mine = True
        n_global = self._n_global
        if world > 1:
            # The collectives are issued from a stream of their own that waits for `after` only:
            # issued from the main stream they would also wait for whatever has been queued
            # there since (the next block's pass).
            main = torch.cuda.current_stream(co.device)
            if self._xchg_stream is None:
                self._xchg_stream = torch.cuda.Stream(device=co.device, priority=-1)
            xs = self._xchg_stream
            if after is not None:
                xs.wait_event(after)
            else:
                xs.wait_stream(main)
            summed = [g for g in groups if g.peer]
            if summed:
                # Their Hessians are complete on the owners once every rank's pass is: what is
                # left of the exchange is a barrier.  It carries the status words of the ranks'
                # Hessian kernels (maximum over ranks), which the owner reports with its own.
                with torch.cuda.stream(xs):
                    for g in summed:
                        g.q[0]._info.record_stream(xs)
                    words = torch.stack([g.q[0]._info for g in summed])
                    t0 = self._mark()
                    work = co.comm.all_reduce_tensor(words, op=torch.distributed.ReduceOp.MAX,
                                                     async_op=True)
                    self._span("exchange_s", t0, work)
                for i, g in enumerate(summed):
                    g.reduce_work = work
                    if g.mine:
                        g.q[0]._info = words[i]
                self.peer_groups += len(summed)
            for g in groups:    # same order on every rank
                if g.peer:
                    continue
                lead = g.q[0]
                if lead._Hbuf is None:   # this rank saw no sample: it still takes part
                    K8 = (lead.columns + 7) // 8 * 8
                    with torch.cuda.stream(xs):
                        lead._Hbuf = torch.zeros((K8, K8), dtype=torch.float32, device=co.device)
                lead._Hbuf.record_stream(xs)
                with torch.cuda.stream(xs):
                    t0 = self._mark()
                    if owner_mode:
                        g.reduce_work = co.comm.reduce_tensor(lead._Hbuf, dst=g.owner, async_op=True)
                    else:
                        g.reduce_work = co.comm.all_reduce_tensor(lead._Hbuf, async_op=True)
                    self._span("exchange_s", t0, g.reduce_work)
                lead._lower_stale = True    # the partial sums only carry the upper triangle
        if self._pool is None:      # made once: the caching allocator pools memory per stream
            self._pool = ChainPool(co.device, n_streams=4)
        fmt = io.file_format(cfg.bits)
        for i in order:             # heaviest chain first
            g = groups[i]
            lead = g.q[0]
            if not g.mine:
                lead.free_hessian()
                continue
            lead.nsamples = n_global
            for q in g.q[1:]:
                q._Hbuf, q.nsamples = lead._Hbuf, n_global
            if self.keep_hessians:
                if g.reduce_work is not None:
                    g.reduce_work.wait()
                for m in g.members:
                    self.hessians[m] = lead.H.detach().cpu().clone()

            def chain(g=g):
                if g.reduce_work is not None:
                    g.reduce_work.wait()        # this side stream waits, the host does not
                status = quantize_group_launch(g.q)
                packed = [io.packed_state(m, q, fmt) for m, q in zip(g.members, g.q)]
                return status, packed

            g.future = self._pool.submit(chain, after=after)

    # ------------------------------------------------------------------ Hessians summed by the kernels
    def _peer_begin(self) -> bool:
        """Start of a block-wise run with ``hessian_exchange == "peer"``: an arena a failed run
        left half-used is cleared on every rank."""
        co, dc = self.coordinator, self.dist_config
        self._group_pattern, self._peer_counter, self.peer_groups = None, 0, 0
        if dc.hessian_exchange != "peer" or dc.world_size <= 1 or co.device.type != "cuda":
            return False
        if self._arena is not None and self._arena.group is not torch.distributed.group.WORLD:
            self._arena = None              # its process group is gone
        if self._arena is not None:
            flag = torch.tensor([int(self._arena.dirty)], dtype=torch.int32, device=co.device)
            co.comm.all_reduce_tensor(flag, op=torch.distributed.ReduceOp.MAX)
            if int(flag.item()):
                self._arena.clear()
                torch.cuda.synchronize(co.device)
                co.comm.barrier()
                self._arena.dirty = False
        return True

    def _peer_prepare(self, head: str, names_b: List[str], quantizers: Dict[str, GPTQ],
                      load: List[float]) -> Optional[Dict[str, int]]:
        """Before a block's pass: predicts the block's groups from the first block's, chooses
        their owners and points every predicted leader's Hessian at its owner's buffer, so that
        ``add_batch`` on every rank accumulates there.  Returns ``{leader: owner}`` or ``None``
        (no prediction, or no symmetric memory: the block takes the NCCL reduction).  Every
        rank computes the same plan from the same names, shapes and loads."""
        co, dc = self.coordinator, self.dist_config
        pat = self._group_pattern
        if pat is None or self._arena_failed:
            return None
        rel = {n: n[len(head):] for n in names_b}
        if any(not n.startswith(head) or rel[n] not in pat for n in names_b):
            return None
        leaders = [n for n in names_b if pat[rel[n]] == rel[n]]
        members = {l: [n for n in names_b if head + pat[rel[n]] == l] for l in leaders}
        widths = [(quantizers[l].columns + 7) // 8 * 8 for l in leaders]
        offsets, gen_bytes = peer.generation_layout(widths)
        generations = self.blocks_in_flight + 2     # see the collect rule in _quantize_blockwise
        if self._arena is not None and not self._arena.fits(gen_bytes, generations):
            self._arena = None
        if self._arena is None:
            self._arena = peer.make_arena(co.device, gen_bytes, generations, co.comm.barrier)
            if self._arena is None:
                self._arena_failed = True
                return None
        arena = self._arena
        gen = self._peer_counter % arena.generations
        self._peer_counter += 1
        costs = [sum(layer_cost(*quantizers[m]._weight_matrix().shape) for m in members[l])
                 for l in leaders]
        plan: Dict[str, int] = {}
        for i in sorted(range(len(leaders)), key=lambda i: (-costs[i], i)):
            owner = min(range(dc.world_size), key=lambda k: (load[k], k))
            load[owner] += costs[i]
            q = quantizers[leaders[i]]
            q._Hbuf = arena.view(owner, gen, offsets[i], widths[i])
            q._info = _C.new_info(co.device)
            q._lower_stale = True
            q._recycle = owner == dc.rank       # the owner zeroes it once its chain has read it
            plan[leaders[i]] = owner
        arena.dirty = True
        return plan

    def _mark_peer(self, groups: List[_Group], plan: Optional[Dict[str, int]]) -> None:
        """After the pass: a group whose leader was given an owner's buffer is complete there,
        whatever its members turned out to be; a leader the prediction missed has accumulated
        into a buffer of its own and takes the NCCL reduction."""
        if not plan:
            return
        for g in groups:
            if g.leader in plan:
                g.peer = True
                g.owner = plan[g.leader]
                g.mine = g.owner == self.dist_config.rank

    def _share_layout(self, groups: List[_Group], owner: int):
        """Pieces of the flat buffer rank ``owner`` sends for one block: for every layer it
        quantized the packed tensors, optionally the dequantized weight, then the status words
        and error sums of its groups.  Sizes follow from shapes and settings alone, so every
        rank lays the buffer out identically.  Returns ``(pieces, total_bytes)`` with pieces
        ``(kind, group, member_index, key, shape, dtype, offset)``."""
        cfg = self.quant_config
        fmt = io.file_format(cfg.bits)
        pieces, off = [], 0

        def add(kind, g, mi, key, shape, dtype):
            nonlocal off
            n = 1
            for s in shape:
                n *= s
            pieces.append((kind, g, mi, key, tuple(shape), dtype, off))
            off = _align(off + n * torch.empty((), dtype=dtype).element_size())

        for g in groups:
            if g.owner != owner:
                continue
            for mi, (m, q) in enumerate(zip(g.members, g.q)):
                N_out, K = q._weight_matrix().shape
                for key, shape, dtype in io.packed_shapes(m, N_out, K, cfg.bits, cfg.group_size, fmt):
                    add("packed", g, mi, key, shape, dtype)
                if self.share_weights:
                    add("weight", g, mi, "weight", tuple(q.layer.weight.shape), q.layer.weight.dtype)
            add("info", g, -1, "info", (2,), torch.int32)
            add("hinfo", g, -1, "hessian_info", (2,), torch.int32)
            add("terr", g, -1, "terr", (len(g.members),), torch.float64)
        return pieces, off

    @staticmethod
    def _piece(flat: torch.Tensor, shape, dtype, off: int) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return flat[off:off + nbytes].view(dtype).view(shape)

    def _share_block(self, groups: List[_Group]) -> list:
        """One broadcast per owning rank of everything it produced for this block.  Enqueued on
        a stream of its own, which waits for the owner's chains; returns what `_finalize`
        needs."""
        co, dc = self.coordinator, self.dist_config
        dev = co.device
        if self._share_stream is None:
            self._share_stream = torch.cuda.Stream(device=dev, priority=-1)
        shared = []
        main = torch.cuda.current_stream(dev)
        for owner in sorted({g.owner for g in groups}):
            pieces, total = self._share_layout(groups, owner)
            mine = owner == dc.rank
            results = {}
            if mine:
                for g in groups:
                    if g.owner == owner:
                        results[id(g)] = g.future.result()      # enqueued (not necessarily run)
                self._pool.stream_wait(self._share_stream,
                                       [g.future for g in groups if g.owner == owner])
            with torch.cuda.stream(self._share_stream):
                flat = torch.empty(max(total, 16), dtype=torch.uint8, device=dev)
                if mine:
                    for kind, g, mi, key, shape, dtype, off in pieces:
                        dst = self._piece(flat, shape, dtype, off)
                        status, packed = results[id(g)]
                        if kind == "packed":
                            dst.copy_(packed[mi][key].reshape(shape))
                        elif kind == "weight":
                            dst.copy_(g.q[mi].layer.weight.data)
                        else:
                            dst.copy_(status[key].reshape(shape))
                t0 = self._mark()
                work = co.comm.broadcast_tensor(flat, src=owner, async_op=True)
                self._span("share_s", t0, work)
                work.wait()
                tail = [p for p in pieces if p[0] in ("info", "hinfo", "terr")]
                host = {}
                for kind, g, mi, key, shape, dtype, off in tail:
                    h = torch.empty(shape, dtype=dtype, pin_memory=True)
                    h.copy_(self._piece(flat, shape, dtype, off), non_blocking=True)
                    host[(id(g), key)] = h
                done = torch.cuda.Event()
                done.record(self._share_stream)
            flat.record_stream(main)
            shared.append({"owner": owner, "flat": flat, "pieces": pieces, "host": host,
                           "done": done})
        return shared

    # ------------------------------------------------------------------ profiling helpers
    def _mark(self):
        if not self.profile:
            return None
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    def _host(self, key: str, t0: float) -> None:
        """Adds the host time since t0 (perf_counter) to timings[key]."""
        self.timings[key] = self.timings.get(key, 0.0) + time.perf_counter() - t0

    def _span(self, key: str, start, work=None) -> None:
        """Adds (now - start) on the current stream to timings[key]; with `work`, the span is
        measured on a stream of its own that waits for the collective."""
        if start is None:
            return
        if work is not None:
            dev = self.coordinator.device
            s = self._probe_streams[self._probe_next % len(self._probe_streams)]
            self._probe_next += 1
            s.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(s):
                a = torch.cuda.Event(enable_timing=True)
                a.record()
                work.wait()
                b = torch.cuda.Event(enable_timing=True)
                b.record()
            self._spans.append((key, a, b))
            return
        b = torch.cuda.Event(enable_timing=True)
        b.record()
        self._spans.append((key, start, b))

    # ------------------------------------------------------------------ finishing a block
    def _finalize(self, names: List[str], layers: Dict[str, nn.Module], groups: List[_Group],
                  shared: Optional[list]) -> Dict[str, dict]:
        """Waits for a block's chains (and broadcasts), raises on a device-side failure - the
        same one on every rank - and returns ``{layer: {"stats", "packed"}}``."""
        cfg, co, dc = self.quant_config, self.coordinator, self.dist_config
        results: Dict[str, dict] = {}
        cur = torch.cuda.current_stream(co.device)
        if shared is not None:
            for sh in shared:
                sh["done"].synchronize()
                cur.wait_event(sh["done"])
            for sh in shared:       # every rank sees the same status words
                for kind, g, mi, key, shape, dtype, off in sh["pieces"]:
                    if kind == "hinfo":
                        _C.raise_on_info(sh["host"][(id(g), key)], f"hessian accumulation ({g.leader})")
                    elif kind == "info":
                        _C.raise_on_info(sh["host"][(id(g), key)], f"damped inverse ({g.leader})")
        for g in groups:
            if g.mine:
                status, packed = g.future.result()
                for mi, (m, q) in enumerate(zip(g.members, g.q)):
                    stats = q.quantize_finish()
                    for t in packed[mi].values():
                        t.record_stream(cur)
                    results[m] = {"stats": stats, "packed": packed[mi]}
                    q.codes = None
                    if mi > 0:
                        q._Hbuf = None
                g.q[0].free_hessian()
        if shared is not None:
            for sh in shared:
                if sh["owner"] == dc.rank:
                    continue
                per_layer: Dict[Tuple[int, int], dict] = {}
                for kind, g, mi, key, shape, dtype, off in sh["pieces"]:
                    if kind == "packed":
                        per_layer.setdefault((id(g), mi), {})[key] = self._piece(sh["flat"], shape, dtype, off)
                    elif kind == "weight":
                        g.q[mi].layer.weight.data = self._piece(sh["flat"], shape, dtype, off)
                for g in groups:
                    if g.owner != sh["owner"]:
                        continue
                    terr = sh["host"][(id(g), "terr")]
                    for mi, (m, q) in enumerate(zip(g.members, g.q)):
                        packed = per_layer[(id(g), mi)]
                        bias = getattr(q.layer, "bias", None)
                        if bias is not None:     # not quantized: the local copy
                            packed[f"{m}.bias"] = bias.data
                        per_channel = cfg.group_size <= 0 or cfg.group_size >= q.columns
                        ng = 1 if per_channel else -(-q.columns // cfg.group_size)
                        N_out = q._weight_matrix().shape[0]
                        results[m] = {"packed": packed, "stats": {
                            "bits": cfg.bits, "group_size": cfg.group_size,
                            "total_error": float(terr[mi].item()),
                            "compression_ratio": 32.0 / cfg.bits,
                            "scale_shape": torch.Size((N_out, ng)),
                            "zero_shape": torch.Size((N_out, ng))}}
        return results

    def _record(self, name: str, layer: nn.Module, entry: dict) -> None:
        cfg = self.quant_config
        self.quantized_layers[name] = entry["stats"]
        self.quantization_errors[name] = entry["stats"].get("total_error", 0)
        self.packed[name] = entry["packed"]
        W = layer.weight.data.flatten(1) if layer.weight.dim() > 2 else layer.weight.data
        self.layer_info[name] = {
            "bits": cfg.bits, "group_size": cfg.group_size,
            "out_features": W.shape[0], "in_features": W.shape[1],
            "kind": "conv2d" if isinstance(layer, nn.Conv2d) else "linear",
            "weight_shape": list(layer.weight.shape),
            "packing": "int32_le" if io.file_format(cfg.bits) == _C.FMT_INT32_LE else "bytes_lo_first"}

    def _groups_of(self, names: List[str], quantizers: Dict[str, GPTQ]) -> List[_Group]:
        by_leader: Dict[str, List[str]] = {}
        for n in names:
            by_leader.setdefault(self._leader[n], []).append(n)
        groups = []
        for lead, members in by_leader.items():
            members = [lead] + [m for m in members if m != lead]
            # layers of one group are stacked into one matrix: same width required
            K = quantizers[lead].columns
            same = [m for m in members if quantizers[m].columns == K]
            groups.append(_Group(lead, same, quantizers))
            for m in members:
                if m not in same:       # cannot happen for layers fed the same tensor
                    raise RuntimeError(f"{m} shares an input with {lead} but not its width")
        return groups

    def _check_grouping(self, names: List[str]) -> None:
        """All ranks must have found the same grouping: it decides order and size of every
        collective that follows."""
        co = self.coordinator
        if not co.comm.active:
            return
        mine = [(n, self._leader[n]) for n in names]
        ref = co.comm.broadcast_object(mine, src=0)
        if ref != mine:
            raise RuntimeError("ranks disagree on which layers share an input; "
                               "the calibration passes took different paths through the model")

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

            h_setup = time.perf_counter()
            samples = calibration_samples(calibration_data, cfg.calibration_samples)
            if not samples:
                raise ValueError("no calibration data")
            self._n_global = len(samples)
            self._leader = {}
            first_sample = samples[0]
            samples = co.shard_calibration(samples)
            batches = make_batches(samples, self.calibration_batch_size)
            self.timings = {}
            self.peer_groups = 0
            self._spans = []
            self._probe_next = 0
            self._probe_streams = ([torch.cuda.Stream(device=co.device) for _ in range(8)]
                                   if self.profile else [])
            self._progress = {"done": 0, "total": len(layers), "cb": progress_callback}
            self._results: Dict[str, dict] = {}

            plan = find_blocks(model, layers) if self.blockwise else None
            self._host("host_setup_s", h_setup)
            done = False
            if plan is not None:
                done = self._quantize_blockwise(model, plan, layers, batches, first_sample)
            if not done:
                self._quantize_whole(model, layers, batches, first_sample)
            h0 = time.perf_counter()
            torch.cuda.synchronize(co.device)
            self._host("host_final_sync_s", h0)

            for n in layers:        # model order
                self._record(n, layers[n], self._results[n])
            self._results = {}
            if self.profile:
                for key, a, b in self._spans:
                    self.timings[key] = self.timings.get(key, 0.0) + a.elapsed_time(b) * 1e-3
            self._spans = []
            self.timings["total_s"] = time.time() - start
            if self.dist_config.rank == 0:
                self._log_quantization_summary(time.time() - start)
            if save_path:
                self.save_quantized_model(model, save_path)
        return model

    def _report(self, names: List[str], results: Dict[str, dict]) -> None:
        self._results.update(results)
        p = self._progress
        for n in names:
            p["done"] += 1
            if p["cb"] and self.dist_config.rank == 0:
                p["cb"](p["done"], p["total"], n, results[n]["stats"])

    # ---- one pass over the whole model per batch, then all layers
    def _quantize_whole(self, model, layers, batches, first_sample) -> None:
        co, dc = self.coordinator, self.dist_config
        self.mode_used = "whole-model"
        t0 = time.time()
        quantizers = self._accumulate_hessians(model, batches, layers, discovery_batch=first_sample)
        names = list(layers)
        self._check_grouping(names)
        self.timings["calibration_s"] = time.time() - t0
        groups = self._groups_of(names, quantizers)
        load = [0.0] * dc.world_size
        self._dispatch(groups, load)
        shared = self._share_block(groups) if dc.world_size > 1 else None
        self._report(names, self._finalize(names, layers, groups, shared))
        self._pool.join()

    # ---- block by block
    @torch.no_grad()
    def _quantize_blockwise(self, model, plan, layers, batches, first_sample) -> bool:
        cfg, co, dc = self.quant_config, self.coordinator, self.dist_config
        list_name, blocks = plan
        prefix = list_name + "." if list_name else ""
        per_block: List[Dict[str, nn.Module]] = [dict() for _ in blocks]
        outside: Dict[str, nn.Module] = {}
        for n, layer in layers.items():
            head = n[len(prefix):].split(".", 1)[0] if n.startswith(prefix) else ""
            if head.isdigit() and int(head) < len(blocks):
                per_block[int(head)][n] = layer
            else:
                outside[n] = layer
        share = dc.world_size > 1           # results travel between ranks in both exchange modes
        load = [0.0] * dc.world_size
        sequential = cfg.true_sequential
        ckpt = Path(cfg.checkpoint_dir) if cfg.checkpoint_dir else None

        # ---- inputs of the first block (and, in one-shot mode, the layers outside the blocks:
        # they see the activations of the unquantized model, so their pass comes first)
        state = {"first": True}
        outside_q = self._new_quantizers(outside)
        run_batches = batches if batches else make_batches([first_sample], 1)
        discovery_only = not batches
        state["accumulate"] = not discovery_only
        outside_now = bool(outside) and not sequential
        t_cal = self._mark()
        h0 = time.perf_counter()
        # Replay check on one sequence: the model is run up to its second block, and the first
        # block, called the way the model called it, must reproduce the second block's input.
        probe_sample = _split_samples(run_batches[0])[0]
        pc, h1 = self._capture_block_inputs(model, blocks, [probe_sample], {}, {}, {"first": True},
                                            stop_early=True, probe=True)
        ok = len(pc) == 1 and h1 is not None
        if ok:
            ph = pc[0][0][0] if pc[0][0] else pc[0][1].get("hidden_states")
            out = self._block_call(blocks[0], ph, pc[0][0], pc[0][1]) if torch.is_tensor(ph) else None
            ok = (out is not None and out.shape == h1.shape and
                  bool(torch.allclose(out.float(), h1.float(), rtol=1e-3, atol=1e-5)))
            del out
        if not ok:
            logger.warning("block-wise calibration: replaying %s[0] does not reproduce the input "
                           "of %s[1]; using whole-model passes", list_name, list_name)
            return False
        self._host("host_replay_check_s", h0)
        captured, _ = self._capture_block_inputs(model, blocks, run_batches, outside, outside_q,
                                                 state, stop_early=not outside_now)
        self._host("host_capture_s", h0)
        if not captured or len(captured) != len(run_batches):
            logger.warning("block-wise calibration: %s[0] was not reached once per batch; "
                           "using whole-model passes", list_name)
            return False
        hidden = [(c[0][0] if c[0] else c[1]["hidden_states"]) for c in captured]
        self.mode_used = "block-wise" + (" true-sequential" if sequential else "")
        self._span("forward_s", t_cal)
        if outside_now:
            self._leader.update({n: state["leader"].get(n, n) for n in outside})
            self._check_grouping(list(outside))
            og = self._groups_of(list(outside), outside_q)
            self._dispatch(og, load)
            pending_outside = (list(outside), og, self._share_block(og) if share else None)
        else:
            pending_outside = None

        # Hessians summed by the kernels themselves: block b accumulates in generation
        # b mod (blocks_in_flight + 2) of the owners' buffers.  The passes of block b are
        # enqueued after the collects of iteration b - 1, which leave at most blocks_in_flight
        # blocks (the youngest being b - 2) uncollected: the block that used the generation
        # before, b - blocks_in_flight - 2, has been collected by every rank, so its owners'
        # chains have read and zeroed the buffers.
        peer_mode = self._peer_begin()
        lag: List[tuple] = []       # blocks whose chains are enqueued but not collected yet
        # One-shot mode: the chains of block b are enqueued only after the pass of block b+1.
        # A chain is a thousand and more launches on a stream that cannot start before its
        # block's pass has run on the device, and the launch queue of a stream is finite: the
        # host blocks in the middle of enqueueing the chain until the device gets there.  With
        # the next pass already queued, the main stream has work for that time.
        deferred: Optional[tuple] = None

        unshared: List[list] = []   # dispatched, results not yet on their way to the other ranks

        def share_pending():
            while unshared:
                it = unshared.pop(0)
                it[4] = self._share_block(it[3])

        def dispatch_deferred():
            nonlocal deferred
            if deferred is None:
                return
            b_, names_, targets_, quantizers_, shard_, ev_, plan_ = deferred
            deferred = None
            h0_ = time.perf_counter()
            groups_ = self._groups_of(names_, quantizers_)
            self._mark_peer(groups_, plan_)
            self._dispatch(groups_, load, after=ev_)
            # The broadcasts of a block are issued after the exchange of the next one: the
            # collectives of a process group run in the order of issue, and a broadcast waits
            # for its owner's chain; issued at once it would hold back the next block's
            # Hessian exchange - and with it that block's chains - until this block's chains
            # are done, one block after the other.
            share_pending()
            item = [b_, names_, targets_, groups_, None, shard_]
            if share:
                unshared.append(item)
                if sequential:
                    share_pending()
            self._host("host_enqueue_chains_s", h0_)
            lag.append(item)

        for b, block in enumerate(blocks):
            targets = per_block[b]
            names_b = list(targets)
            shard = ckpt / f"block_{b:05d}.safetensors" if ckpt is not None else None
            resumed = None
            if shard is not None and targets and shard.is_file():
                resumed = io.load_block_shard(shard, targets, cfg, co.device)
                if sequential:      # later blocks are calibrated on the quantized model
                    io.apply_block_weights(targets, resumed)
            quantizers = self._new_quantizers(targets) if resumed is None else {}
            head = f"{prefix}{b}."
            plan_b = (self._peer_prepare(head, names_b, quantizers, load)
                      if peer_mode and resumed is None and targets else None)
            bstate = {"first": True, "accumulate": not discovery_only}
            handles = self._hook_layers(targets, quantizers, bstate) if resumed is None else []
            nxt = []
            t0 = self._mark()
            h0 = time.perf_counter()
            try:
                for i, h in enumerate(hidden):
                    out = self._block_call(block, h, captured[i][0], captured[i][1])
                    bstate.setdefault("seen", []).clear()
                    bstate["first"] = False
                    if not sequential or resumed is not None or not targets:
                        nxt.append(out)
            finally:
                for hd in handles:
                    hd.remove()
            self._span("forward_s", t0)
            self._host("host_enqueue_forward_s", h0)
            done_b = torch.cuda.Event()
            done_b.record(torch.cuda.current_stream(co.device))     # this block's Hessians are complete
            dispatch_deferred()                                     # the previous block's chains
            if resumed is not None:
                if not sequential:  # one-shot: every block sees the unquantized model's activations
                    io.apply_block_weights(targets, resumed)
                for n in names_b:
                    self._leader[n] = resumed["leader"].get(n, n)
                self._report(names_b, resumed["results"])
                hidden = nxt
                continue
            if targets:
                self._leader.update({n: bstate["leader"].get(n, n) for n in names_b})
                if b == 0:
                    self._check_grouping(names_b)
                if peer_mode and self._group_pattern is None:
                    # what the later blocks' groups are predicted from
                    self._group_pattern = {n[len(head):]: self._leader[n][len(head):]
                                           for n in names_b if n.startswith(head)}
                deferred = (b, names_b, targets, quantizers, shard, done_b, plan_b)
                if sequential:
                    dispatch_deferred()
            if sequential and targets:
                # the next block must see this block's quantized weights: collect now, re-run
                self._collect(lag.pop())
                t0 = self._mark()
                nxt = [self._block_call(block, h, captured[i][0], captured[i][1])
                       for i, h in enumerate(hidden)]
                self._span("forward_s", t0)
            elif len(lag) > self.blocks_in_flight:
                if lag[0][4] is None:       # cannot be collected before its results travel
                    share_pending()
                self._collect(lag.pop(0))    # bounds how far the host runs ahead of the device
            hidden = nxt
        dispatch_deferred()
        share_pending()
        h0 = time.perf_counter()
        while lag:
            self._collect(lag.pop(0))
        self._host("host_tail_collect_s", h0)
        if pending_outside is not None:
            names_o, og, sh = pending_outside
            self._report(names_o, self._finalize(names_o, outside, og, sh))
        elif outside:
            # true-sequential: the layers after the blocks see the quantized model
            oq = self._accumulate_hessians(model, batches, outside, discovery_batch=first_sample)
            names_o = list(outside)
            self._check_grouping(names_o)
            og = self._groups_of(names_o, oq)
            self._dispatch(og, load)
            sh = self._share_block(og) if share else None
            self._report(names_o, self._finalize(names_o, outside, og, sh))
        if self._pool is not None:
            self._pool.join()
        if self._arena is not None:
            self._arena.dirty = False       # every buffer has been read and zeroed again
        return True

    def _collect(self, item) -> None:
        b, names_b, targets, groups, shared, shard = item
        t0 = time.perf_counter()
        results = self._finalize(names_b, targets, groups, shared)
        # how long the host stood still for this block's chains (it runs ahead otherwise)
        self.timings["host_wait_s"] = self.timings.get("host_wait_s", 0.0) + time.perf_counter() - t0
        if shard is not None and self.dist_config.rank == 0:
            io.save_block_shard(shard, names_b, targets, results,
                                {n: self._leader[n] for n in names_b}, self.quant_config)
        self._report(names_b, results)

    # ------------------------------------------------------------------ save / load
    def _metadata(self) -> dict:
        config = asdict(self.quant_config)
        config.pop("checkpoint_dir", None)     # where shards were kept is not a property of the result
        return {"quantization_config": config,
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
        logger.info("Quantized %d layers to %d bits (group %d) in %.2f s (%s); average error %.6f; "
                    "peak GPU memory %.2f GB", n, self.quant_config.bits,
                    self.quant_config.group_size, elapsed, self.mode_used, avg,
                    self.coordinator.get_memory_stats()["max_allocated_gb"])


GPTQQuantizer = DistributedGPTQuantizer   # the name the reference imports but never defines


def quantize_model_simple(model: nn.Module, calibration_data, bits: int = 4,
                          save_path: Optional[str] = None) -> nn.Module:
    """Reference ``core/quantizer.py:358-383``."""
    quantizer = DistributedGPTQuantizer(QuantizationConfig(bits=bits))
    return quantizer.quantize_model(model, calibration_data, save_path=save_path)
