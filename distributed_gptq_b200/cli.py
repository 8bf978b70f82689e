"""Command line of the quantization path: ``quantize`` and ``benchmark`` (reference
``src/distributed_gptq/cli.py:36-95,453-565``, whose commands cannot run: the module imports
names that do not exist).

    python -m distributed_gptq_b200.cli quantize --model /path/to/hf_model --bits 4 \\
        --group-size 128 --act-order --dataset custom --dataset-path ids.pt --output-dir out
    python -m torch.distributed.run --nproc-per-node 8 -m distributed_gptq_b200.cli quantize ...
    python -m distributed_gptq_b200.cli benchmark --model /path/to/hf_model \\
        --quantized-model out/model.safetensors

Option names, defaults and choices are the reference's.  What differs: several GPUs are used
by launching one process per GPU with ``torch.distributed.run`` (the reference spawned them
itself, ``cli.py:38-44``); ``--dataset custom --dataset-path`` takes a ``.pt`` file holding an
integer tensor ``(n, seq_len)`` of token ids or a text file that the model's tokenizer splits;
the named datasets need a network and are only reached through the ``datasets`` package when
it is installed; ``--dataset random`` draws uniform-random token ids (what the benchmark of
this repository uses).
"""
from __future__ import annotations

import argparse
import json
import logging
import os
import sys
import time
from pathlib import Path

# The driver keeps many streams busy; with CUDA's default of 8 hardware queues per device the
# chains' short kernels would queue behind whole forward passes.  Read when CUDA starts.
os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")

import torch  # noqa: E402

logger = logging.getLogger("distributed_gptq_b200.cli")


def create_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(description="Distributed GPTQ Quantization Tool")
    sub = parser.add_subparsers(dest="command")

    q = sub.add_parser("quantize", help="Quantize a model")
    q.add_argument("--model", "-m", required=True, help="Model name or path (HuggingFace layout)")
    q.add_argument("--model-type", choices=["transformers", "custom"], default="transformers")
    q.add_argument("--torch-dtype", choices=["float16", "bfloat16", "float32"], default="float16")
    q.add_argument("--bits", type=int, default=4, choices=[2, 3, 4, 8])
    q.add_argument("--group-size", type=int, default=128)
    q.add_argument("--act-order", action="store_true")
    q.add_argument("--true-sequential", action="store_true")
    q.add_argument("--damp", type=float, default=0.01)
    q.add_argument("--dataset", default="wikitext", choices=["wikitext", "c4", "ptb", "custom", "random"])
    q.add_argument("--dataset-path")
    q.add_argument("--num-samples", type=int, default=128)
    q.add_argument("--seq-len", type=int, default=2048)
    q.add_argument("--batch-size", type=int, default=1, help="sequences per calibration forward")
    q.add_argument("--output-dir", default="./quantized_models")
    q.add_argument("--save-format", default="safetensors", choices=["safetensors", "pytorch"])
    q.add_argument("--checkpoint-dir", help="keep one shard per finished block here and resume from it")
    q.add_argument("--hessian-exchange", default="owner", choices=["owner", "all_reduce", "peer"],
                   help="several ranks: reduce each Hessian to the rank that quantizes the layer "
                        "(default), all_reduce it like the reference, or let every rank's Hessian "
                        "kernel accumulate into the owner's buffer over NVLink")
    q.add_argument("--include-lm-head", action="store_true",
                   help="also quantize linear layers outside the decoder blocks")
    q.add_argument("--seed", type=int, default=0)
    q.add_argument("--log-level", default="INFO")
    q.set_defaults(func=quantize_command)

    b = sub.add_parser("benchmark", help="Benchmark a quantized model")
    b.add_argument("--model", "-m", required=True)
    b.add_argument("--quantized-model", required=True, help="packed .safetensors written by `quantize`")
    b.add_argument("--torch-dtype", choices=["float16", "bfloat16", "float32"], default="float16")
    b.add_argument("--test-samples", type=int, default=16)
    b.add_argument("--seq-len", type=int, default=512)
    b.add_argument("--batch-size", type=int, default=1)
    b.add_argument("--device", default="cuda")
    b.add_argument("--save-results")
    b.add_argument("--seed", type=int, default=0)
    b.add_argument("--log-level", default="INFO")
    b.set_defaults(func=benchmark_command)
    return parser


def _dtype(name: str) -> torch.dtype:
    return {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}[name]


def load_model(path: str, dtype: torch.dtype):
    """A causal language model in HuggingFace layout: a directory with weights, or one with only
    ``config.json`` (random initialisation, for dry runs without a checkpoint)."""
    import transformers
    p = Path(path)
    has_weights = (not p.is_dir()) or any(p.glob("*.safetensors")) or any(p.glob("*.bin"))
    if not has_weights:
        cfg = transformers.AutoConfig.from_pretrained(str(p))
        old = torch.get_default_dtype()
        torch.set_default_dtype(dtype)
        try:
            model = transformers.AutoModelForCausalLM.from_config(cfg)
        finally:
            torch.set_default_dtype(old)
        return model.eval(), None
    model = transformers.AutoModelForCausalLM.from_pretrained(path, dtype=dtype)
    try:
        tok = transformers.AutoTokenizer.from_pretrained(path)
    except Exception:  # noqa: BLE001  (a model directory without tokenizer files)
        tok = None
    return model.eval(), tok


def calibration_ids(args, vocab_size: int, tokenizer) -> torch.Tensor:
    """``(num_samples, seq_len)`` int64 token ids."""
    g = torch.Generator().manual_seed(args.seed)
    n, L = args.num_samples, args.seq_len
    if args.dataset == "random":
        return torch.randint(0, vocab_size, (n, L), generator=g)
    if args.dataset == "custom":
        if not args.dataset_path:
            raise SystemExit("--dataset custom needs --dataset-path")
        if args.dataset_path.endswith(".pt"):
            ids = torch.load(args.dataset_path)
            if ids.dim() != 2:
                raise SystemExit("the .pt calibration file must hold a (samples, seq_len) tensor of token ids")
            return ids[:n, :L].long()
        if tokenizer is None:
            raise SystemExit("a text calibration file needs the model's tokenizer")
        text = Path(args.dataset_path).read_text()
        stream = tokenizer(text, return_tensors="pt").input_ids[0]
    else:
        try:
            import datasets
        except ImportError:
            raise SystemExit(f"--dataset {args.dataset} needs the `datasets` package and a network; "
                             "use --dataset custom or --dataset random")
        name = {"wikitext": ("wikitext", "wikitext-2-raw-v1", "train", "text"),
                "c4": ("allenai/c4", "en", "train", "text"),
                "ptb": ("ptb_text_only", "penn_treebank", "train", "sentence")}[args.dataset]
        data = datasets.load_dataset(name[0], name[1], split=name[2])
        stream = tokenizer("\n\n".join(data[name[3]][:20000]), return_tensors="pt").input_ids[0]
    if stream.numel() < L + 1:
        raise SystemExit("calibration text is shorter than one sequence")
    starts = torch.randint(0, stream.numel() - L, (n,), generator=g)
    return torch.stack([stream[s:s + L] for s in starts.tolist()])


def decoder_linears(model) -> list:
    """Names of the linear layers inside the model's list of blocks (the head and anything
    else outside it stays in floating point, as GPTQ tools leave it)."""
    import torch.nn as nn
    from .quantizer import find_blocks
    linears = {n: m for n, m in model.named_modules() if isinstance(m, nn.Linear)}
    plan = find_blocks(model, linears)
    if plan is None:
        return list(linears)
    prefix = plan[0] + "."
    return [n for n in linears if n.startswith(prefix)]


def quantize_command(args) -> None:
    from . import DistributedGPTQuantizer, QuantizationConfig
    from .coordinator import create_distributed_config
    dcfg = create_distributed_config()
    dcfg.hessian_exchange = args.hessian_exchange
    model, tok = load_model(args.model, _dtype(args.torch_dtype))
    vocab = getattr(model.config, "vocab_size", 32000)
    ids = calibration_ids(args, vocab, tok)
    qcfg = QuantizationConfig(bits=args.bits, group_size=args.group_size, actorder=args.act_order,
                              percdamp=args.damp, calibration_samples=args.num_samples,
                              true_sequential=args.true_sequential, checkpoint_dir=args.checkpoint_dir)
    qz = DistributedGPTQuantizer(qcfg, dcfg, calibration_batch_size=max(1, args.batch_size))
    layers = None if args.include_lm_head else decoder_linears(model)
    out_dir = Path(args.output_dir)
    suffix = ".safetensors" if args.save_format == "safetensors" else ".pt"
    t0 = time.time()

    def progress(done, total, name, stats):
        logger.info("[%d/%d] %s  error %.4e", done, total, name, stats.get("total_error", 0.0))

    qz.quantize_model(model, ids, layers_to_quantize=layers, progress_callback=progress)
    elapsed = time.time() - t0
    if dcfg.rank == 0:
        path = out_dir / ("model" + suffix)
        qz.save_quantized_model(model, str(path), save_format=args.save_format)
        metrics = {"model": args.model, "bits": args.bits, "group_size": args.group_size,
                   "act_order": args.act_order, "true_sequential": args.true_sequential,
                   "world_size": dcfg.world_size, "seconds": elapsed, "mode": qz.mode_used,
                   "layers": len(qz.quantized_layers),
                   "mean_total_error": sum(qz.quantization_errors.values()) / max(1, len(qz.quantization_errors)),
                   "peak_gpu_memory_gb": qz.coordinator.get_memory_stats()["max_allocated_gb"]}
        with open(out_dir / "quantization_metrics.json", "w") as f:     # reference utils/metrics.py:83-86
            json.dump(metrics, f, indent=2)
        logger.info("quantized %d layers in %.1f s -> %s", metrics["layers"], elapsed, path)


def benchmark_command(args) -> None:
    """Float model against its packed quantized form: size, latency per forward, perplexity on
    uniform-random token ids (a stand-in that needs no dataset; reference ``cli.py:49-81``)."""
    from . import DistributedGPTQuantizer
    dev = torch.device(args.device)
    dtype = _dtype(args.torch_dtype)
    g = torch.Generator().manual_seed(args.seed)

    def measure(model):
        model = model.to(dev).eval()
        vocab = getattr(model.config, "vocab_size", 32000)
        ids = torch.randint(0, vocab, (args.test_samples, args.seq_len), generator=g).to(dev)
        nll, tokens = 0.0, 0
        torch.cuda.synchronize(dev)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.no_grad():
            model(ids[:args.batch_size], use_cache=False)       # warm-up
            a.record()
            for i in range(0, args.test_samples, args.batch_size):
                x = ids[i:i + args.batch_size]
                logits = model(x, use_cache=False).logits.float()
                nll += float(torch.nn.functional.cross_entropy(
                    logits[:, :-1].reshape(-1, logits.shape[-1]), x[:, 1:].reshape(-1), reduction="sum"))
                tokens += x[:, 1:].numel()
            b.record()
        torch.cuda.synchronize(dev)
        nbytes = sum(t.numel() * t.element_size() for t in model.state_dict().values())
        return {"ms_per_forward": a.elapsed_time(b) / max(1, -(-args.test_samples // args.batch_size)),
                "perplexity": float(torch.exp(torch.tensor(nll / tokens))), "bytes": nbytes}

    model, _ = load_model(args.model, dtype)
    g.manual_seed(args.seed)
    base = measure(model)
    qz = DistributedGPTQuantizer()
    qmodel, _ = load_model(args.model, dtype)
    qz.load_quantized_model(qmodel, args.quantized_model)
    g.manual_seed(args.seed)
    quant = measure(qmodel)
    results = {"compression_ratio": base["bytes"] / quant["bytes"],
               "speedup": base["ms_per_forward"] / quant["ms_per_forward"],
               "memory_reduction": base["bytes"] / quant["bytes"],
               "perplexity_change": quant["perplexity"] - base["perplexity"],
               "float": base, "quantized": quant}
    print("\nBenchmark Results:")
    print("-" * 50)
    print(f"Model: {args.model}")
    print(f"Quantized Model: {args.quantized_model}")
    print(f"Compression Ratio: {results['compression_ratio']:.2f}x")
    print(f"Speed Up: {results['speedup']:.2f}x")
    print(f"Memory Reduction: {results['memory_reduction']:.2f}x")
    print(f"Perplexity Change: {results['perplexity_change']:.4f}")
    print("-" * 50)
    if args.save_results:
        with open(args.save_results, "w") as f:
            json.dump(results, f, indent=2)


def main(argv=None) -> None:
    parser = create_parser()
    args = parser.parse_args(argv)
    if not hasattr(args, "func"):
        parser.print_help()
        sys.exit(1)
    logging.basicConfig(level=getattr(logging, args.log_level.upper(), logging.INFO),
                        format="%(asctime)s - %(name)s - %(levelname)s - %(message)s")
    args.func(args)


if __name__ == "__main__":
    main()
