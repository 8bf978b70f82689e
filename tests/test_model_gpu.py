"""Model-level driver: quantize_model / quantize_model_simple, shared-input Hessians, packed
safetensors round trip, QuantizedLinear / dequantizer / torch.ops.gptq.linear."""
import json
import os

import pytest
import torch
import torch.nn as nn

from oracle import oracle_gptq as O

pytestmark = pytest.mark.gpu


class Block(nn.Module):
    """A toy decoder block: q/k/v read the same tensor (one shared Hessian), then an MLP."""

    def __init__(self, d=256, ff=512):
        super().__init__()
        self.q = nn.Linear(d, d, bias=False)
        self.k = nn.Linear(d, d, bias=False)
        self.v = nn.Linear(d, d, bias=True)
        self.up = nn.Linear(d, ff, bias=False)
        self.down = nn.Linear(ff, d, bias=False)
        self.tiny = nn.Linear(d, 2, bias=False)      # 512 weights: below the 1000-weight threshold

    def forward(self, x):
        h = self.q(x) + self.k(x) + self.v(x)
        y = self.down(torch.relu(self.up(h)))
        return y + self.tiny(x).sum(-1, keepdim=True)


def _model(seed=0):
    torch.manual_seed(seed)
    m = nn.Sequential()
    m.add_module("b0", Block())
    m.add_module("b1", Block())
    return m


def _calib(n=16, seq=64, d=256, seed=1):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(2, seq, d, generator=g) for _ in range(n // 2)]


def test_quantize_model_matches_layerwise_oracle(dgq, tmp_path):
    from distributed_gptq_b200 import (DistributedGPTQuantizer, QuantizationConfig, QuantizedLinear)
    model = _model()
    ref_model = _model()
    calib = _calib()
    seen = []
    cfg = QuantizationConfig(bits=4, group_size=128, actorder=True, calibration_samples=16)
    qz = DistributedGPTQuantizer(cfg)
    path = tmp_path / "q.safetensors"
    out = qz.quantize_model(model, calib, save_path=str(path),
                            progress_callback=lambda i, n, name, st: seen.append((i, n, name)))
    assert out is model
    names = [n for n, m in ref_model.named_modules() if isinstance(m, nn.Linear) and m.weight.numel() > 1000]
    assert [s[2] for s in seen] == names and seen[-1][0] == seen[-1][1] == len(names) == 10
    assert set(qz.quantized_layers) == set(names) and "b0.tiny" not in qz.quantized_layers
    assert qz._leader["b0.k"] == "b0.q" and qz._leader["b0.v"] == "b0.q" and qz._leader["b0.up"] == "b0.up"

    # layer-by-layer oracle on activations captured from the unquantized reference model
    acts = {}
    hooks = [m.register_forward_pre_hook(lambda mod, a, n=n: acts.setdefault(n, []).append(a[0].detach()))
             for n, m in ref_model.named_modules() if n in names]
    with torch.no_grad():
        for b in calib:
            ref_model(b)
    for h in hooks:
        h.remove()
    mods = dict(model.named_modules())
    refmods = dict(ref_model.named_modules())
    for n in names:
        X = torch.cat([a.reshape(-1, a.shape[-1]) for a in acts[n]]).bfloat16().float()
        H = X.t() @ X
        W = refmods[n].weight.data
        ref = O.gptq_quantize(W, H, 16, 4, 128, 128, 0.01, True)
        Q = mods[n].weight.data.float().cpu()
        r_gpu, r_ref = O.recon_error(W, Q, H), O.recon_error(W, ref["Q"], H)
        assert abs(r_gpu - r_ref) <= 0.05 * r_ref, (n, r_gpu, r_ref)   # act-order ties may reorder columns
        assert qz.quantization_errors[n] > 0
        assert qz.quantized_layers[n]["bits"] == 4

    # packed file + sidecar
    meta = json.load(open(path.with_suffix(".json")))
    assert meta["quantization_config"]["bits"] == 4 and meta["quantized_layers"] == names
    assert set(meta["quantization_errors"]) == set(names)
    from safetensors.torch import load_file
    tensors = load_file(str(path))
    assert tensors["b0.q.qweight"].dtype == torch.uint8 and tensors["b0.q.qweight"].shape == (256, 128)
    assert tensors["b0.q.scales"].dtype == torch.float16 and tensors["b0.q.g_idx"].dtype == torch.int32
    assert "b0.q.weight" not in tensors and "b0.tiny.weight" in tensors and "b0.v.bias" in tensors

    # load into a fresh model: quantized layers become QuantizedLinear and compute the same function
    fresh = _model(seed=5).cuda()
    qz2 = DistributedGPTQuantizer(QuantizationConfig())
    qz2.load_quantized_model(fresh, str(path))
    assert isinstance(fresh.b0.q, QuantizedLinear) and isinstance(fresh.b0.tiny, nn.Linear)
    assert qz2.quant_config.actorder is True
    x = calib[0][:1].cuda()
    with torch.no_grad():
        y_q = fresh(x)
        y_d = model(x)
    assert float((y_q - y_d).abs().max()) <= 2e-3 * float(y_d.abs().max())   # fp16 scales in the file
    w = fresh.b0.q.unpack_weights()
    assert float((w - model.b0.q.weight.data.float()).abs().max()) <= 1e-3 * float(w.abs().max())


def test_quantize_model_simple_and_dequantize(dgq):
    from distributed_gptq_b200 import (GPTQDequantizer, QuantizedLinear, quantize_model_simple,
                                       replace_with_quantized_layers)
    torch.manual_seed(3)
    model = nn.Sequential(nn.Linear(512, 1024), nn.ReLU(), nn.Linear(1024, 512), nn.ReLU(),
                          nn.Linear(512, 256))
    W0 = [m.weight.data.clone() for m in model if isinstance(m, nn.Linear)]
    calib = [torch.randn(1, 512) for _ in range(50)]       # the reference quickstart's shape
    out = quantize_model_simple(model, calib, bits=4)
    assert out is model and next(model.parameters()).is_cuda
    for m, w0 in zip([m for m in model if isinstance(m, nn.Linear)], W0):
        w = m.weight.data.cpu()
        assert not torch.equal(w, w0)
        assert float((w - w0).abs().max()) <= 1.5 * float(w0.abs().max())   # 50 samples: H is rank deficient
        # 4-bit, group 128: at most 16 distinct values per (row, group)
        assert all(len(torch.unique(w[0, g * 128:(g + 1) * 128])) <= 16 for g in range(w.shape[1] // 128))

    # QuantizedLinear from a GPTQ object + the op hook + the dequantizer
    from distributed_gptq_b200 import GPTQ
    lin = nn.Linear(256, 64, bias=True).cuda()
    q = GPTQ(lin, bits=4, group_size=64, actorder=True)
    q.add_batch(torch.randn(4, 128, 256, device="cuda"), None)
    q.quantize()
    ql = QuantizedLinear.from_gptq(q)
    x = torch.randn(3, 256, device="cuda")
    want = torch.nn.functional.linear(x, lin.weight.data, lin.bias.data)
    got = ql(x)
    assert got.shape == (3, 64)
    assert float((got - want).abs().max()) <= 2e-3 * float(want.abs().max())
    got_op = torch.ops.gptq.linear(x, ql.qweight, ql.scales, ql.zeros, ql.g_idx, ql.bias)
    assert torch.equal(got_op, got)
    deq = GPTQDequantizer(4, 64).dequantize_layer(ql)
    assert isinstance(deq, nn.Linear)
    assert float((deq.weight.data - lin.weight.data).abs().max()) <= 1e-3 * float(lin.weight.abs().max())
    assert torch.equal(GPTQDequantizer(4, 64)._unpack_4bit(ql.qweight), q.codes.float())
    # the reference's constructor default g_idx (the column index itself) falls back to c // group
    ql2 = QuantizedLinear(4, 64, 256, 64, bias=False).cuda()
    ql2.pack_weights(q.codes, q.scale, q.zero)
    ql2.g_idx = torch.arange(256, dtype=torch.int32, device="cuda")
    y = ql2(x)
    w_plain = O.dequant(q.codes.cpu(), q.scale.half().cpu(), q.zero.half().cpu(), None, 64)
    assert float((y.cpu() - x.cpu() @ w_plain.t()).abs().max()) <= 1e-3 * float(y.abs().max()) + 1e-4
    emp = replace_with_quantized_layers(nn.Sequential(nn.Linear(128, 128), nn.ReLU()), bits=4)
    assert isinstance(emp[0], QuantizedLinear)


def test_kernels_module(dgq):
    from distributed_gptq_b200 import dequantize_tensor, quantize_tensor
    x = torch.randn(64, 300)
    q, s, z = quantize_tensor(x, bits=4, group_size=128)
    qo, so, zo = O.rtn_quantize(x, 4, 128)
    assert torch.equal(q.cpu(), qo) and torch.equal(s.cpu(), so)
    d = dequantize_tensor(q, s, z, 128)
    assert torch.equal(d.cpu(), O.rtn_dequantize(qo, so, zo, 128))


def test_command_line_quantize_and_benchmark(dgq, tmp_path, capsys):
    """`quantize` then `benchmark` of the command line (reference cli.py:36-95) on a small
    Llama-architecture model given by its config alone."""
    transformers = pytest.importorskip("transformers")
    from distributed_gptq_b200 import cli
    mdir, out = tmp_path / "model", tmp_path / "out"
    transformers.LlamaConfig(vocab_size=512, hidden_size=256, intermediate_size=512,
                             num_hidden_layers=2, num_attention_heads=4,
                             max_position_embeddings=256).save_pretrained(str(mdir))
    torch.manual_seed(0)
    cli.main(["quantize", "--model", str(mdir), "--torch-dtype", "bfloat16", "--bits", "4",
              "--group-size", "128", "--act-order", "--dataset", "random", "--num-samples", "8",
              "--seq-len", "96", "--batch-size", "4", "--output-dir", str(out)])
    metrics = json.load(open(out / "quantization_metrics.json"))
    assert metrics["layers"] == 14 and metrics["mode"] == "block-wise" and metrics["bits"] == 4
    meta = json.load(open(out / "model.json"))
    assert len(meta["quantized_layers"]) == 14 and "lm_head" not in meta["quantized_layers"]
    torch.manual_seed(0)        # the same random weights for the float side of the comparison
    cli.main(["benchmark", "--model", str(mdir), "--quantized-model", str(out / "model.safetensors"),
              "--torch-dtype", "bfloat16", "--test-samples", "4", "--seq-len", "64",
              "--save-results", str(out / "bench.json")])
    res = json.load(open(out / "bench.json"))
    assert res["compression_ratio"] > 1.5 and res["quantized"]["perplexity"] > 0
    assert "Compression Ratio" in capsys.readouterr().out
