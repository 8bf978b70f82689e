"""Block-by-block driver: same results as whole-model passes, stacked quantization of layers
that share an input, the true-sequential mode and the per-block checkpoint / resume."""
import os

import pytest
import torch
import torch.nn as nn

pytestmark = pytest.mark.gpu


class Block(nn.Module):
    """q/k/v read one tensor (one Hessian, quantized as one stacked matrix), then an MLP."""

    def __init__(self, d=256, ff=512):
        super().__init__()
        self.norm = nn.LayerNorm(d)
        self.q = nn.Linear(d, d, bias=False)
        self.k = nn.Linear(d, d, bias=False)
        self.v = nn.Linear(d, d, bias=True)
        self.up = nn.Linear(d, ff, bias=False)
        self.down = nn.Linear(ff, d, bias=False)

    def forward(self, x, scale=1.0):
        h = self.norm(x)
        h = x + scale * (self.q(h) + self.k(h) + self.v(h))
        return (h + self.down(torch.relu(self.up(h))),)     # tuple, like some decoder layers


class Decoder(nn.Module):
    def __init__(self, n_blocks=3, d=256, vocab=1000):
        super().__init__()
        self.embed = nn.Embedding(vocab, d)
        self.layers = nn.ModuleList(Block(d) for _ in range(n_blocks))
        self.head = nn.Linear(d, vocab, bias=False)

    def forward(self, ids):
        h = self.embed(ids)
        for blk in self.layers:
            h = blk(h, scale=0.5)[0]
        return self.head(h)


def _model(seed=0):
    torch.manual_seed(seed)
    return Decoder()


def _ids(n=24, seq=48, seed=1):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 1000, (n, seq), generator=g)


def _run(cfg_kwargs=None, model=None, callback=None, **qz_kwargs):
    from distributed_gptq_b200 import DistributedGPTQuantizer, QuantizationConfig
    cfg = QuantizationConfig(bits=4, group_size=128, actorder=True, calibration_samples=24,
                             **(cfg_kwargs or {}))
    qz = DistributedGPTQuantizer(cfg, calibration_batch_size=8, **qz_kwargs)
    model = model if model is not None else _model()
    qz.quantize_model(model, _ids(), progress_callback=callback)
    return qz, model


def test_blockwise_equals_whole_model(dgq):
    qa, ma = _run(blockwise=False)
    qb, mb = _run()
    assert qa.mode_used == "whole-model" and qb.mode_used == "block-wise"
    assert list(qa.quantized_layers) == list(qb.quantized_layers)
    assert "head" in qb.quantized_layers and len(qb.quantized_layers) == 16
    assert qb._leader["layers.1.k"] == "layers.1.q" and qb._leader["layers.1.v"] == "layers.1.q"
    for n in qa.packed:
        for k in qa.packed[n]:
            assert torch.equal(qa.packed[n][k], qb.packed[n][k]), k
        assert qa.quantization_errors[n] == qb.quantization_errors[n]
    for (na, pa), (nb, pb) in zip(ma.state_dict().items(), mb.state_dict().items()):
        assert torch.equal(pa, pb), na


@pytest.mark.parametrize("depth", [1, 4])
def test_blocks_in_flight_do_not_change_results(dgq, depth):
    """How many blocks have chains enqueued but not collected is scheduling only."""
    qa, ma = _run()
    qb, mb = _run(blocks_in_flight=depth)
    assert qa.blocks_in_flight == 2 and qb.blocks_in_flight == depth
    for n in qa.packed:
        for k in qa.packed[n]:
            assert torch.equal(qa.packed[n][k], qb.packed[n][k]), (n, k)
        assert qa.quantization_errors[n] == qb.quantization_errors[n]
    for (na, pa), (nb, pb) in zip(ma.state_dict().items(), mb.state_dict().items()):
        assert torch.equal(pa, pb), na


def test_stacked_group_equals_single_layers(dgq):
    """q/k/v quantized as one stacked matrix == each quantized by itself with the same Hessian."""
    from distributed_gptq_b200 import GPTQ
    from distributed_gptq_b200.gptq import quantize_group_launch
    torch.manual_seed(3)
    X = torch.randn(4, 200, 384, device="cuda")
    for actorder in (False, True):
        layers = [nn.Linear(384, n, bias=False).cuda() for n in (256, 128, 640)]
        twins = [nn.Linear(384, n, bias=False).cuda() for n in (256, 128, 640)]
        for a, b in zip(layers, twins):
            b.weight.data.copy_(a.weight.data)
        group = [GPTQ(l, bits=3, group_size=128, actorder=actorder) for l in layers]
        group[0].add_batch(X)
        for g in group[1:]:
            g._Hbuf, g.nsamples = group[0]._Hbuf, group[0].nsamples
        quantize_group_launch(group)
        stats = [g.quantize_finish() for g in group]
        for g, t, st in zip(group, twins, stats):
            s = GPTQ(t, bits=3, group_size=128, actorder=actorder)
            s.add_batch(X)
            ref = s.quantize()
            assert torch.equal(g.codes, s.codes) and torch.equal(g.scale, s.scale)
            assert torch.equal(g.zero, s.zero) and torch.equal(g.g_idx, s.g_idx)
            assert torch.equal(g.layer.weight.data, t.weight.data)
            assert abs(st["total_error"] - ref["total_error"]) <= 1e-9 * ref["total_error"]


def test_true_sequential_differs_and_resumes(dgq, tmp_path):
    from safetensors.torch import load_file
    q1, m1 = _run()
    qs, ms = _run({"true_sequential": True})
    assert qs.mode_used == "block-wise true-sequential"
    # the first block sees the same inputs in both modes, later blocks do not
    assert torch.equal(m1.layers[0].q.weight.data, ms.layers[0].q.weight.data)
    assert torch.equal(q1.packed["layers.0.down"]["layers.0.down.qweight"],
                       qs.packed["layers.0.down"]["layers.0.down.qweight"])
    assert not torch.equal(q1.packed["layers.2.up"]["layers.2.up.qweight"],
                           qs.packed["layers.2.up"]["layers.2.up.qweight"])
    assert not torch.equal(q1.packed["head"]["head.qweight"], qs.packed["head"]["head.qweight"])

    # uninterrupted run with checkpoints == run without; then an interrupted run, resumed
    ck_a, ck_b = str(tmp_path / "a"), str(tmp_path / "b")
    qa, ma = _run({"true_sequential": True, "checkpoint_dir": ck_a})
    assert sorted(os.listdir(ck_a)) == [f"block_{i:05d}.safetensors" for i in range(3)]
    for n in qs.packed:
        for k in qs.packed[n]:
            assert torch.equal(qs.packed[n][k], qa.packed[n][k])

    class Interrupt(Exception):
        pass

    def stop_after_first_block(done, total, name, stats):
        if name.startswith("layers.1."):
            raise Interrupt()

    with pytest.raises(Interrupt):
        _run({"true_sequential": True, "checkpoint_dir": ck_b}, callback=stop_after_first_block)
    torch.cuda.synchronize()
    assert "block_00000.safetensors" in os.listdir(ck_b)
    seen = []
    qb, mb = _run({"true_sequential": True, "checkpoint_dir": ck_b},
                  callback=lambda d, t, n, s: seen.append(n))
    assert len(seen) == 16
    pa, pb = str(tmp_path / "a.safetensors"), str(tmp_path / "b.safetensors")
    qa.save_quantized_model(ma, pa)
    qb.save_quantized_model(mb, pb)
    assert open(pa, "rb").read() == open(pb, "rb").read()
    assert open(pa[:-12] + ".json").read() == open(pb[:-12] + ".json").read()
    ta = load_file(pa)
    assert "layers.0.q.qweight" in ta and "layers.0.q.weight" not in ta

    # a shard written with other settings is refused, not silently reused
    from distributed_gptq_b200 import DistributedGPTQuantizer, QuantizationConfig
    bad = DistributedGPTQuantizer(QuantizationConfig(bits=3, calibration_samples=24,
                                                     true_sequential=True, checkpoint_dir=ck_b))
    with pytest.raises(RuntimeError, match="other quantization settings"):
        bad.quantize_model(_model(), _ids())


def test_replay_mismatch_falls_back(dgq):
    """A model whose block list is not a plain chain (here: applied in reverse) cannot be
    replayed block by block; the driver notices and takes whole-model passes."""
    class Odd(Decoder):
        def forward(self, ids):
            h = self.embed(ids)
            for blk in reversed(self.layers):
                h = blk(h, scale=0.5)[0]
            return self.head(h)

    torch.manual_seed(0)
    qz, _ = _run(model=Odd())
    assert qz.mode_used == "whole-model" and len(qz.quantized_layers) == 16
