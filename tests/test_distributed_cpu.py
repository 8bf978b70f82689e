"""Host-side logic of the multi-GPU path on CPU: sharding, owner placement and the Hessian
exchange over a world_size-2 gloo group."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from distributed_gptq_b200.coordinator import (DistributedConfig, DistributedGPTQCoordinator,
                                               QuantizationMode, assign_owners,
                                               create_distributed_config, layer_cost, shard_indices)
from distributed_gptq_b200.quantizer import QuantizationConfig, calibration_samples


def test_shard_indices_partition():
    for n in (0, 1, 7, 128, 129):
        for w in (1, 2, 3, 8):
            parts = [shard_indices(n, r, w) for r in range(w)]
            flat = sorted(i for p in parts for i in p)
            assert flat == list(range(n))                       # every sequence exactly once
            assert max(len(p) for p in parts) - min(len(p) for p in parts) <= 1
            assert parts[0][:3] == list(range(0, n, w))[:3]     # rank r takes r, r+W, ...


def test_assign_owners_is_deterministic_and_balanced():
    # one Llama-7B decoder block: q,k,v,o (4096x4096), gate/up (11008x4096), down (4096x11008)
    shapes = [(4096, 4096)] * 4 + [(11008, 4096)] * 2 + [(4096, 11008)]
    costs = [layer_cost(o, i) for o, i in shapes] * 32
    for w in (1, 2, 4, 8):
        own = assign_owners(costs, w)
        assert own == assign_owners(list(costs), w)
        assert set(own) <= set(range(w))
        load = [sum(c for c, o in zip(costs, own) if o == r) for r in range(w)]
        assert max(load) <= 1.05 * (sum(costs) / w)
    assert assign_owners([5.0, 1.0, 1.0], 2) == [0, 1, 1]


def test_config_surface(monkeypatch):
    c = QuantizationConfig()
    assert (c.bits, c.group_size, c.actorder, c.percdamp, c.blocksize, c.calibration_samples,
            c.use_triton, c.save_packed) == (4, 128, False, 0.01, 128, 128, False, True)
    c.validate()
    QuantizationConfig(bits=8, group_size=-1).validate()
    for bad in (dict(bits=5), dict(group_size=0), dict(percdamp=1.5)):
        with pytest.raises(AssertionError):
            QuantizationConfig(**bad).validate()
    for k in ("WORLD_SIZE", "RANK", "LOCAL_RANK"):
        monkeypatch.delenv(k, raising=False)
    d = create_distributed_config()
    assert d.mode == QuantizationMode.SINGLE_GPU and d.world_size == 1 and d.is_main_process
    assert d.master_port == "12355" and d.backend == "nccl" and d.init_timeout == 1800
    monkeypatch.setenv("WORLD_SIZE", "4")
    monkeypatch.setenv("RANK", "2")
    d = create_distributed_config()
    assert d.mode == QuantizationMode.DATA_PARALLEL and d.is_distributed and not d.is_main_process
    assert create_distributed_config("model_parallel").mode == QuantizationMode.MODEL_PARALLEL


def test_calibration_sample_normalisation():
    assert len(calibration_samples([torch.zeros(2, 5), torch.zeros(3, 5)], 128)) == 5
    assert len(calibration_samples(torch.zeros(7, 5), 4)) == 4
    s = calibration_samples([{"input_ids": torch.zeros(2, 5, dtype=torch.long), "use_cache": False}], 9)
    assert len(s) == 2 and s[0]["input_ids"].shape == (1, 5) and s[0]["use_cache"] is False
    loader = torch.utils.data.DataLoader(torch.utils.data.TensorDataset(torch.zeros(6, 3)), batch_size=4)
    assert len(calibration_samples(loader, 128)) == 6


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        cfg = DistributedConfig(mode=QuantizationMode.DATA_PARALLEL, world_size=world, rank=rank,
                                local_rank=0, master_addr="127.0.0.1", master_port=str(port),
                                backend="gloo", init_timeout=60, hessian_exchange=mode)
        co = DistributedGPTQCoordinator(cfg)
        co.device = torch.device("cpu")
        with co.distributed_context():
            assert dist.get_world_size() == world
            hs = {"a": torch.full((4, 4), float(rank + 1)), "b": torch.full((2, 2), 10.0 * (rank + 1))}
            owners = {"a": 0, "b": 1}
            co.exchange_hessians(hs, owners)
            total_a, total_b = float(sum(range(1, world + 1))), 10.0 * sum(range(1, world + 1))
            if mode == "all_reduce" or rank == 0:
                assert torch.all(hs["a"] == total_a)
            if mode == "all_reduce" or rank == 1:
                assert torch.all(hs["b"] == total_b)
            t = torch.tensor([float(rank)])
            co.comm.broadcast_tensor(t, src=1)
            assert float(t) == 1.0
            t = torch.tensor([1.0])
            co.comm.all_reduce_tensor(t)
            assert float(t) == world
            assert co.comm.broadcast_object({"x": rank}, src=0) == {"x": 0}
            shard = co.shard_calibration(list(range(7)))
            assert shard == list(range(rank, 7, world))
            # the reference's name for the split (coordinator.py:147-181): lists and DataLoaders
            assert co.distribute_calibration_data(list(range(7))) == shard
            from torch.utils.data import DataLoader, TensorDataset
            dl = DataLoader(TensorDataset(torch.arange(10).float()), batch_size=2)
            mine = torch.cat([b[0] for b in co.distribute_calibration_data(dl)])
            assert mine.tolist() == [float(i) for i in range(rank, 10, world)]
            # every rank must have found the same grouping of layers; one that did not is told
            from distributed_gptq_b200 import DistributedGPTQuantizer
            qz = DistributedGPTQuantizer.__new__(DistributedGPTQuantizer)
            qz.coordinator = co
            qz._leader = {"a": "a", "b": "a"}
            qz._check_grouping(["a", "b"])
            qz._leader = {"a": "a", "b": "a" if rank == 0 else "b"}
            try:
                qz._check_grouping(["a", "b"])
                disagreed = False
            except RuntimeError as e:
                disagreed = "disagree" in str(e)
            assert disagreed == (rank == 1)
            co.comm.barrier()
        assert not dist.is_initialized()
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, f"{type(e).__name__}: {e}"))


@pytest.mark.parametrize("mode", ["owner", "all_reduce"])
def test_exchange_over_gloo(mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, mode, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results


def test_reference_method_names_exist():
    """Callers written against the reference's coordinator find its methods
    (reference coordinator.py:147-235)."""
    from distributed_gptq_b200.coordinator import DistributedConfig, DistributedGPTQCoordinator
    co = DistributedGPTQCoordinator(DistributedConfig())
    assert callable(co.quantize_layer_distributed) and callable(co.distribute_calibration_data)
    data = [1, 2, 3]
    assert co.distribute_calibration_data(data) is data     # single process: unchanged


def test_device_status_words_raise():
    """The host half of the device status path: the two words a kernel leaves behind become
    Python errors that name the condition."""
    import pytest
    from distributed_gptq_b200 import _C
    _C.raise_on_info(torch.tensor([_C.INFO_OK, 0], dtype=torch.int32), "x")
    with pytest.raises(RuntimeError, match=r"inverse.*not positive definite \(pivot 17\)"):
        _C.raise_on_info(torch.tensor([_C.INFO_NOT_POSDEF, 17], dtype=torch.int32), "damped inverse")
    with pytest.raises(RuntimeError, match=r"bounded wait.*ran out \(wait 3\)"):
        _C.raise_on_info(torch.tensor([_C.INFO_WAIT_TIMEOUT, 3], dtype=torch.int32), "hessian")
    with pytest.raises(RuntimeError, match="unknown device status 9"):
        _C.raise_on_info(torch.tensor([9, 0], dtype=torch.int32), "x")


def test_block_discovery_and_batching():
    import torch.nn as nn
    from distributed_gptq_b200.quantizer import calibration_samples, find_blocks, make_batches

    class M(nn.Module):
        def __init__(self):
            super().__init__()
            self.pre = nn.Linear(8, 8)
            self.short = nn.ModuleList([nn.Linear(8, 8)])
            self.layers = nn.ModuleList(nn.Sequential(nn.Linear(8, 8), nn.Linear(8, 8)) for _ in range(3))
            self.head = nn.Linear(8, 8)
    m = M()
    layers = {n: mod for n, mod in m.named_modules() if isinstance(mod, nn.Linear)}
    name, blocks = find_blocks(m, layers)
    assert name == "layers" and len(blocks) == 3
    assert find_blocks(nn.Sequential(nn.Linear(4, 4), nn.Linear(4, 4)),
                       {"0": None, "1": None}) is None
    samples = calibration_samples([torch.zeros(3, 5), torch.zeros(2, 7), torch.zeros(4, 5)], 8)
    assert len(samples) == 8
    batches = make_batches(samples, 2)
    assert [tuple(b.shape) for b in batches] == [(2, 5), (1, 5), (2, 7), (2, 5), (1, 5)]


def test_share_layout_is_aligned_and_deterministic():
    """Every rank lays the per-block result buffer out from shapes and settings alone."""
    import torch.nn as nn
    from distributed_gptq_b200 import DistributedGPTQuantizer, QuantizationConfig
    from distributed_gptq_b200.coordinator import DistributedConfig
    from distributed_gptq_b200.quantizer import _Group

    class FakeQ:
        def __init__(self, layer):
            self.layer = layer
            self.columns = layer.weight.shape[1]

        def _weight_matrix(self):
            return self.layer.weight.data
    for bits, group in ((4, 128), (3, 128), (8, -1), (2, 64)):
        qz = DistributedGPTQuantizer(QuantizationConfig(bits=bits, group_size=group), DistributedConfig())
        lins = {"a": nn.Linear(384, 100, bias=False), "b": nn.Linear(384, 36), "c": nn.Linear(256, 50)}
        qs = {n: FakeQ(l) for n, l in lins.items()}
        g1, g2 = _Group("a", ["a", "b"], qs), _Group("c", ["c"], qs)
        g1.owner, g2.owner = 1, 0
        pieces, total = qz._share_layout([g1, g2], 1)
        assert [p[3] for p in pieces if p[0] == "packed"][:4] == ["a.qweight", "a.scales", "a.zeros", "a.g_idx"]
        assert all(p[6] % 16 == 0 for p in pieces) and total % 16 == 0
        assert {p[1] for p in pieces} == {g1}
        assert [p[0] for p in pieces][-3:] == ["info", "hinfo", "terr"] and pieces[-1][4] == (2,)
        flat = torch.zeros(total, dtype=torch.uint8)
        for kind, g, mi, key, shape, dtype, off in pieces:
            view = qz._piece(flat, shape, dtype, off)
            assert tuple(view.shape) == tuple(shape) and view.dtype == dtype
        # non-overlapping
        spans = sorted((p[6], p[6] + qz._piece(flat, p[4], p[5], p[6]).numel() *
                        qz._piece(flat, p[4], p[5], p[6]).element_size()) for p in pieces)
        assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:]))
        assert qz._share_layout([g1, g2], 1) == (pieces, total)


def test_peer_plan_is_the_same_on_every_rank(monkeypatch):
    """``hessian_exchange == "peer"``: before a block's pass every rank predicts the block's
    groups from the first block's, chooses the same owners and takes the same slot of the
    same generation of the arena; only the owner hands the buffer back zeroed."""
    import torch.nn as nn
    from distributed_gptq_b200 import DistributedGPTQuantizer, QuantizationConfig, _C, peer
    from distributed_gptq_b200.coordinator import DistributedConfig
    from distributed_gptq_b200.quantizer import _Group

    offsets, size = peer.generation_layout([4096, 4096, 11008])
    assert offsets == [0, 4096 * 4096 * 4, 2 * 4096 * 4096 * 4] and size % peer.ALIGN == 0
    assert peer.generation_layout([100])[1] == 40192                 # 40000 padded to 256 bytes

    class FakeQ:
        def __init__(self, layer):
            self.layer, self.columns = layer, layer.weight.shape[1]
            self._Hbuf = self._info = None
            self._recycle = False

        def _weight_matrix(self):
            return self.layer.weight.data

    class FakeArena:
        generations, dirty = 4, False

        def fits(self, b, g):
            return True

        def view(self, rank, gen, off, K8):
            return ("slot", rank, gen, off, K8)

    monkeypatch.setattr(_C, "new_info", lambda dev: torch.zeros(2, dtype=torch.int32))
    pattern = {"q": "q", "k": "q", "v": "q", "up": "up", "down": "down"}
    shapes = {"q": (64, 64), "k": (64, 64), "v": (64, 64), "up": (160, 64), "down": (64, 160)}
    plans = []
    for rank in range(2):
        qz = DistributedGPTQuantizer(QuantizationConfig(),
                                     DistributedConfig(world_size=2, rank=rank, hessian_exchange="peer"))
        assert qz.blocks_in_flight == 2
        qz._arena, qz._group_pattern = FakeArena(), dict(pattern)
        load, seen = [0.0, 0.0], []
        for b in (1, 2, 3, 4, 5):
            head = f"layers.{b}."
            qs = {head + n: FakeQ(nn.Linear(i, o, bias=False)) for n, (o, i) in shapes.items()}
            plan = qz._peer_prepare(head, list(qs), qs, load)
            assert set(plan) == {head + "q", head + "up", head + "down"}
            for lead, owner in plan.items():
                slot = qs[lead]._Hbuf
                assert slot[1] == owner and slot[2] == (b - 1) % 4 and qs[lead]._recycle == (owner == rank)
                assert qs[lead]._info is not None
            assert qs[head + "k"]._Hbuf is None
            groups = [_Group(head + "q", [head + "q", head + "k", head + "v"], qs),
                      _Group(head + "up", [head + "up"], qs), _Group(head + "down", [head + "down"], qs),
                      _Group(head + "k", [head + "k"], qs)]      # a leader the prediction missed
            qz._mark_peer(groups, plan)
            assert [g.peer for g in groups] == [True, True, True, False]
            assert all(g.mine == (g.owner == rank) for g in groups[:3])
            seen.append({k: (v, qs[k]._Hbuf) for k, v in plan.items()})
        assert abs(load[0] - load[1]) <= max(load) * 0.5
        plans.append((seen, load))
        # a block whose names the pattern does not know takes the NCCL reduction
        odd = {"layers.9.other": FakeQ(nn.Linear(8, 8))}
        assert qz._peer_prepare("layers.9.", list(odd), odd, load) is None
    assert plans[0] == plans[1]


def test_command_line_surface():
    """Option names, defaults and choices of the reference's `quantize` command (cli.py:130-300)."""
    from distributed_gptq_b200 import cli
    a = cli.create_parser().parse_args(["quantize", "--model", "m"])
    assert (a.bits, a.group_size, a.damp, a.num_samples, a.seq_len, a.batch_size, a.dataset,
            a.torch_dtype, a.output_dir, a.act_order, a.true_sequential) == \
        (4, 128, 0.01, 128, 2048, 1, "wikitext", "float16", "./quantized_models", False, False)
    assert a.hessian_exchange == "owner"        # not in the reference: how partial Hessians are summed
    import pytest
    with pytest.raises(SystemExit):
        cli.create_parser().parse_args(["quantize", "--model", "m", "--bits", "5"])
    b = cli.create_parser().parse_args(["benchmark", "--model", "m", "--quantized-model", "q"])
    assert b.device == "cuda" and b.func is cli.benchmark_command
