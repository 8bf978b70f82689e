#!/usr/bin/env python
"""Benchmark of the GPTQ quantization path on B200.

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the CPU restatement of the reference, timed
    python bench.py --workload sweep|opt1.3b|llama13b|opt125m ...

Default workload ("llama7b"): a Llama-2-7B-architecture model (32 decoder blocks, d_model 4096,
32 heads, SwiGLU FFN 11008, RMSNorm, RoPE, vocabulary 32000) with random bf16 weights
~N(0, 0.02), calibrated on 256 sequences x 2048 uniform-random token ids and quantized to
4 bits, group 128, act-order, blocksize 128, percdamp 0.01, through the package's public
entry point ``DistributedGPTQuantizer.quantize_model``.  One step = one whole model: the
calibration forward passes, the Hessians of all 224 decoder linears (q/k/v and gate/up share
one each), the damped inverse factors, the blockwise quantization and the packing.  The
`lm_head` is left out (it is tied to no decoder block and GPTQ tools leave it in float).  All
inputs are synthetic and seeded.  Between steps the layers get their original weights back
(a pointer assignment: the driver never writes into a weight tensor, it replaces it).
The calibration activations of one block (4.3 GB per pass at one GPU) exceed the L2 cache, so
no flush is needed between steps.

`value` is seconds per model with the token ids already on the device; `e2e` is the same
from token ids in pinned host memory to the packed tensors (codes, scales, zeros, g_idx of every
layer) in pinned host memory on rank 0.  At N > 1 the sequences are split over the ranks
(data-parallel calibration), every block's partial Hessians are reduced to the rank that owns
the layer group, owners quantize in parallel (layer-parallel) and results are broadcast:
total work is fixed, i.e. strong scaling.

Other workloads: "sweep" - the standalone layer sweep (three layers x {4,3}-bit x act-order
off/on); "opt1.3b" - OPT-1.3B architecture, 3-bit g128 (`--exchange all_reduce` reproduces the
reference's flow in which every rank receives every Hessian); "llama13b" - Llama-2-13B
architecture, `--variant 2bit-g64` or `8bit-perchannel`; "opt125m" - the reference's CPU-sized
case (fp32, 128 x 512).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

# The model driver keeps a dozen and more streams busy (the main stream, four chain streams,
# the inverse factor's side streams, the exchange streams).  With CUDA's default of 8 hardware
# queues per device several of them share a queue, and a chain's short kernels then wait behind
# a whole forward pass queued earlier on the main stream.  Must be set before CUDA starts.
os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")

import torch  # noqa: E402

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BLOCK, PERCDAMP = 128, 0.01
HESS_TILE = 256

MODELS = {
    "llama7b": dict(kind="llama", name="Llama-2-7B architecture", layers=32, d=4096, heads=32,
                    ffn=11008, vocab=32000, nseq=256, seq=2048, dtype="bf16", batch=32,
                    variants={"4bit-g128-actorder": dict(bits=4, group=128, actorder=True)}),
    "llama13b": dict(kind="llama", name="Llama-2-13B architecture", layers=40, d=5120, heads=40,
                     ffn=13824, vocab=32000, nseq=128, seq=2048, dtype="bf16", batch=32,
                     variants={"2bit-g64": dict(bits=2, group=64, actorder=False),
                               "8bit-perchannel": dict(bits=8, group=-1, actorder=False)}),
    "opt1.3b": dict(kind="opt", name="OPT-1.3B architecture", layers=24, d=2048, heads=32,
                    ffn=8192, vocab=50272, nseq=128, seq=2048, dtype="bf16", batch=32,
                    variants={"3bit-g128": dict(bits=3, group=128, actorder=False)}),
    "opt125m": dict(kind="opt", name="OPT-125m architecture", layers=12, d=768, heads=12,
                    ffn=3072, vocab=50272, nseq=128, seq=512, dtype="f32", batch=32,
                    variants={"4bit-g128": dict(bits=4, group=128, actorder=False)}),
}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.thread = [], None, None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-i", str(self.gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0])); mx.append(float(r[1])); power.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        # "under load": samples drawing clearly more than idle power
        busy = [s for s, p in zip(sm, power) if p > 250.0] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None,
                "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# dram__bytes_read.sum + dram__bytes_write.sum of one hessian_syrk_kernel launch from ncu
# captures on small cases (profiles/hessian_syrk_kernel.md): (K, T) -> bytes
HESS_TRAFFIC_CAPTURES = {4096: (65536, 575.5e6), 11008: (32768, 4.148e9)}


def hessian_traffic(K: int, T: int) -> float:
    """DRAM bytes of one launch.  Where a capture of this K exists it is scaled by the tokens
    of the launch (X dominates and is streamed once per wave of concurrently running tiles,
    so the traffic grows in proportion to T); other K use that model directly:
    2*T*K bytes of X per wave of 148 tiles + 8*K^2 bytes of H read-modify-write."""
    if K in HESS_TRAFFIC_CAPTURES:
        t0, b0 = HESS_TRAFFIC_CAPTURES[K]
        return b0 * T / t0
    P = -(-K // HESS_TILE)
    waves = max(1.0, (P * (P + 1) // 2) / 148.0)
    return 2.0 * T * K * waves + 8.0 * K * K


def hessian_flops(K: int, T: int):
    P = -(-K // HESS_TILE)
    executed = (P * (P + 1) // 2) * 2.0 * HESS_TILE * HESS_TILE * T
    return executed, 2.0 * T * K * K


# ============================================================================= model workloads
def model_linears(spec):
    """(name suffix, N_out, K, shares the input of) for the linears of one decoder block."""
    d, f = spec["d"], spec["ffn"]
    if spec["kind"] == "llama":
        return [("q_proj", d, d, None), ("k_proj", d, d, "q_proj"), ("v_proj", d, d, "q_proj"),
                ("o_proj", d, d, None), ("gate_proj", f, d, None), ("up_proj", f, d, "gate_proj"),
                ("down_proj", d, f, None)]
    return [("q_proj", d, d, None), ("k_proj", d, d, "q_proj"), ("v_proj", d, d, "q_proj"),
            ("out_proj", d, d, None), ("fc1", f, d, None), ("fc2", d, f, None)]


def build_model(spec, n_layers: int, device, seed: int = 0):
    """Random-init model of the named architecture, built on the device."""
    import transformers
    dtype = torch.bfloat16 if spec["dtype"] == "bf16" else torch.float32
    if spec["kind"] == "llama":
        cfg = transformers.LlamaConfig(
            vocab_size=spec["vocab"], hidden_size=spec["d"], intermediate_size=spec["ffn"],
            num_hidden_layers=n_layers, num_attention_heads=spec["heads"],
            num_key_value_heads=spec["heads"], max_position_embeddings=4096, rms_norm_eps=1e-5,
            initializer_range=0.02, tie_word_embeddings=False, attn_implementation="sdpa")
        cls = transformers.LlamaForCausalLM
    else:
        cfg = transformers.OPTConfig(
            vocab_size=spec["vocab"], hidden_size=spec["d"], num_hidden_layers=n_layers,
            ffn_dim=spec["ffn"], num_attention_heads=spec["heads"], max_position_embeddings=2048,
            word_embed_proj_dim=spec["d"], activation_function="relu", init_std=0.02,
            attn_implementation="sdpa")
        cls = transformers.OPTForCausalLM
    torch.manual_seed(seed)
    old = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        with torch.device(device):
            model = cls(cfg)
    finally:
        torch.set_default_dtype(old)
    return model.eval()


class ModelWorkload:
    def __init__(self, spec, variant, n_layers, rank, world, device, exchange, seed=0,
                 true_sequential=False, blocks_in_flight=None):
        import torch.nn as nn
        from distributed_gptq_b200 import DistributedGPTQuantizer, QuantizationConfig
        from distributed_gptq_b200.coordinator import create_distributed_config
        self.spec, self.variant, self.rank, self.world, self.device = spec, variant, rank, world, device
        self.n_layers = n_layers
        self.model = build_model(spec, n_layers, device, seed)
        block_list = "model.layers." if spec["kind"] == "llama" else "model.decoder.layers."
        self.names = [n for n, m in self.model.named_modules()
                      if isinstance(m, nn.Linear) and n.startswith(block_list)]
        mods = dict(self.model.named_modules())
        self.layers = {n: mods[n] for n in self.names}
        self.pristine = {n: m.weight.data for n, m in self.layers.items()}
        g = torch.Generator().manual_seed(seed + 1)
        ids = torch.randint(0, spec["vocab"], (spec["nseq"], spec["seq"]), generator=g)
        self.ids_host = ids.pin_memory()
        self.ids_dev = ids.to(device)
        v = spec["variants"][variant]
        qcfg = QuantizationConfig(bits=v["bits"], group_size=v["group"], actorder=v["actorder"],
                                  percdamp=PERCDAMP, blocksize=BLOCK,
                                  calibration_samples=spec["nseq"], true_sequential=true_sequential)
        dcfg = create_distributed_config()
        dcfg.hessian_exchange = exchange
        self.qz = DistributedGPTQuantizer(qcfg, dcfg, calibration_batch_size=spec["batch"],
                                          blocks_in_flight=blocks_in_flight)
        self.qz.profile = True
        self.host_out = None
        self.h2d_bytes = self.d2h_bytes = 0
        self.my_seqs = len(range(rank, spec["nseq"], world))

    def restore(self):
        for n, m in self.layers.items():
            m.weight.data = self.pristine[n]

    def step(self, from_host: bool):
        self.restore()
        ids = self.ids_host if from_host else self.ids_dev
        self.qz.quantize_model(self.model, ids, layers_to_quantize=self.names)
        self.h2d_bytes = self.d2h_bytes = 0
        if from_host:
            self.h2d_bytes = self.my_seqs * self.spec["seq"] * 8
            if self.rank == 0:
                # the step's result leaves the device: every packed tensor of the model
                flat = [t for n in self.names for k, t in sorted(self.qz.packed[n].items())
                        if not k.endswith(".bias")]
                if self.host_out is None:
                    self.host_out = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in flat]
                for h, t in zip(self.host_out, flat):
                    h.copy_(t, non_blocking=True)
                    self.d2h_bytes += h.numel() * h.element_size()
                torch.cuda.current_stream().synchronize()
        return self.qz

    def hessian_flops_per_step(self):
        """Executed and algorithmic FLOP of this rank's Hessian kernels in one step."""
        T = self.my_seqs * self.spec["seq"]
        ex = al = 0.0
        for _, _, K, shared in model_linears(self.spec):
            if shared is None:
                e, a = hessian_flops(K, T)
                ex += e
                al += a
        return ex * self.n_layers, al * self.n_layers, T

    def describe(self):
        s, v = self.spec, self.spec["variants"][self.variant]
        layers = f"{self.n_layers} decoder blocks" + (
            "" if self.n_layers == s["layers"] else f" (REDUCED from {s['layers']}: not the named model)")
        return (f"{s['name']} ({layers}, d_model {s['d']}, {s['heads']} heads, FFN {s['ffn']}, "
                f"vocab {s['vocab']}), random-init {s['dtype']} weights ~N(0,0.02); calibration "
                f"{s['nseq']} x {s['seq']} uniform-random token ids; GPTQ {v['bits']}-bit, group "
                f"{v['group']}, act-order {'on' if v['actorder'] else 'off'}, blocksize {BLOCK}, "
                f"percdamp {PERCDAMP}; {len(self.names)} decoder linears quantized through "
                f"DistributedGPTQuantizer.quantize_model ({self.qz.mode_used or 'block-wise'}), "
                f"lm_head left in float")


def linear_check(spec, device, actorder: bool):
    """The packed 4-bit quantized linear (``torch.ops.gptq.linear``, the operator the reference's
    ``QuantizedLinear.forward`` calls) at batch 1, 4 and 16 on the three layer shapes of the
    model, checked against dequantize + matmul (the reference's own fallback branch,
    models/layers.py:155-157) and timed with CUDA events over back-to-back calls."""
    import distributed_gptq_b200  # noqa: F401
    from distributed_gptq_b200 import _C
    d, f, g = spec["d"], spec["ffn"], 128
    out = []
    gen = torch.Generator(device=device).manual_seed(7)
    for N_out, K in ((d, d), (f, d), (d, f)):
        codes = torch.randint(0, 16, (N_out, K), generator=gen, device=device, dtype=torch.uint8)
        qw = _C.pack(codes, 4, _C.FMT_BYTES_LO_FIRST)
        scales = (torch.rand(N_out, K // g, generator=gen, device=device) * 0.02 + 0.001).half()
        zeros = torch.randint(0, 16, (N_out, K // g), generator=gen, device=device).half()
        g_idx = (torch.arange(K, device=device) // g).to(torch.int32)
        if actorder:
            g_idx = g_idx[torch.randperm(K, generator=gen, device=device)]
        W = _C.unpack_dequant(qw, scales, zeros, g_idx, K, 4, g, _C.FMT_BYTES_LO_FIRST, torch.float32)
        for M in (1, 4, 16):
            x = torch.randn(M, K, generator=gen, device=device).to(torch.bfloat16)
            y = torch.ops.gptq.linear(x, qw, scales, zeros, g_idx, None)
            want = x.double() @ W.double().t()
            err = float((y.double() - want).abs().max() / want.abs().max())
            reps = 200
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(reps):
                torch.ops.gptq.linear(x, qw, scales, zeros, g_idx, None)
            b.record()
            torch.cuda.synchronize()
            us = a.elapsed_time(b) * 1e3 / reps
            nbytes = N_out * K / 2 + 4 * N_out * (K // g) + 2 * M * (K + N_out)
            out.append({"N_out": N_out, "K": K, "M": M, "act_order": actorder, "us_per_call": round(us, 2),
                        "algorithmic_GBs": round(nbytes / us / 1e3, 1),
                        "max_err_vs_dequant_matmul": err, "ok": err <= 4.5e-3})
    return out


# ============================================================================= layer sweep
LAYERS = [("4096x4096", 4096, 4096), ("11008x4096", 11008, 4096), ("4096x11008", 4096, 11008)]
SETTINGS = [(4, False), (4, True), (3, False), (3, True)]   # (bits, act-order)
NSEQ, SEQ = 128, 2048
GROUP = 128
CHUNK_SEQS = 32          # sequences per add_batch call


def outlier_channels(K: int, layer_idx: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(9000 + layer_idx)
    return torch.randperm(K, generator=g)[: -(-K // 100)]


def make_weights(layer_idx: int, N_out: int, K: int, device) -> torch.Tensor:
    g = torch.Generator(device=device).manual_seed(1000 + layer_idx)
    return (torch.randn(N_out, K, generator=g, device=device) * 0.02).to(torch.bfloat16)


def make_activations(layer_idx: int, K: int, seq_ids, device) -> torch.Tensor:
    """(len(seq_ids), SEQ, K) bf16; every sequence has its own seed, so any split of the
    sequences over ranks sees the same global data."""
    out = torch.empty((len(seq_ids), SEQ, K), dtype=torch.bfloat16, device=device)
    idx = outlier_channels(K, layer_idx).to(device)
    g = torch.Generator(device=device)
    for i, s in enumerate(seq_ids):
        g.manual_seed(100000 * (layer_idx + 1) + s)
        x = torch.randn(SEQ, K, generator=g, device=device)
        x[:, idx] *= 20.0
        out[i] = x.to(torch.bfloat16)
    return out


def run_cost(N_out: int, K: int) -> float:
    return 0.7 * K ** 3 + float(N_out) * K * K


def assign_owners(world: int):
    """Longest-processing-time-first placement of the 12 runs on the ranks."""
    runs = [(li, bits, act) for li in range(len(LAYERS)) for bits, act in SETTINGS]
    order = sorted(range(len(runs)), key=lambda i: -run_cost(LAYERS[runs[i][0]][1], LAYERS[runs[i][0]][2]))
    load = [0.0] * world
    owner = [0] * len(runs)
    for i in order:
        r = min(range(world), key=lambda k: load[k])
        owner[i] = r
        load[r] += run_cost(LAYERS[runs[i][0]][1], LAYERS[runs[i][0]][2])
    return runs, owner


class Sweep:
    """The standalone layer sweep: 12 independent GPTQ runs per step, each with its own
    Hessian accumulation.  At N > 1 all Hessians are accumulated and reduced first and the
    owners' chains follow (`chains="after"`); starting a run's chain right after its reduce
    (`"during"`) was measured slower at every N (8 GPUs: 76 ms against 41 ms per sweep): the
    chains of the widest layers are the critical path, and their hundreds of short dependent
    kernels each wait for a free SM while Hessian kernels fill the GPU."""

    def __init__(self, rank: int, world: int, device, chains: str = "after"):
        from distributed_gptq_b200 import _C  # noqa: F401  (fails loudly without the library)
        self.rank, self.world, self.device = rank, world, device
        self.chains = chains     # several GPUs: chains "during" the Hessian phase or "after" it
        self.runs, self.owner = assign_owners(world)
        self.my_seqs = list(range(rank, NSEQ, world))
        self.W = [make_weights(i, n, k, device) for i, (_, n, k) in enumerate(LAYERS)]
        self.X_dev = None
        self.X_host = None
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        # Streams are made once: torch's caching allocator keeps a pool of freed blocks per
        # stream, so fresh streams every step would find their pools empty and call cudaMalloc.
        from distributed_gptq_b200.streams import ChainPool
        self.pool = ChainPool(device, n_streams=6)
        self.copy_stream = torch.cuda.Stream(device=device)

    def load_device_inputs(self):
        self.X_dev = [make_activations(i, k, self.my_seqs, self.device)
                      for i, (_, _, k) in enumerate(LAYERS)]

    def load_host_inputs(self):
        self.X_host = []
        for i, (_, _, k) in enumerate(LAYERS):
            src = self.X_dev[i] if self.X_dev is not None else make_activations(
                i, k, self.my_seqs, self.device)
            h = torch.empty(src.shape, dtype=src.dtype, pin_memory=True)
            h.copy_(src)
            self.X_host.append(h)

    def _chunks(self, x):
        for s in range(0, x.shape[0], CHUNK_SEQS):
            yield x[s:s + CHUNK_SEQS]

    def _launch(self, item, from_host: bool, pool):
        """Layer-parallel quantization: the owner of a run quantizes and packs it.  The chain is
        only enqueued here, on one of the pool's side streams (which waits for the reduction
        of the run's Hessian); `_collect` waits for it."""
        from distributed_gptq_b200 import _C
        ri, q, work = item
        if self.owner[ri] != self.rank:
            q.free_hessian()
            return None
        bits = self.runs[ri][1]
        fmt = _C.FMT_BYTES_LO_FIRST if bits == 4 else _C.FMT_INT32_LE

        def chain():
            if work is not None:
                work.wait()         # the side stream waits for the reduce, the host does not
            q.quantize_launch()
            packed = q.pack_weights(format=fmt)
            out = {"run": ri, "qweight": packed["packed_weights"],
                   "scales": q.scale.to(torch.float16), "zeros": q.zero.to(torch.float16),
                   "g_idx": q.g_idx}
            out["d2h_bytes"] = 0
            if from_host:
                for k in ("qweight", "scales", "zeros", "g_idx"):
                    host = torch.empty(out[k].shape, dtype=out[k].dtype, pin_memory=True)
                    host.copy_(out[k], non_blocking=True)
                    out["d2h_bytes"] += host.numel() * host.element_size()
                    out[k] = host
            return out

        return (q, pool.submit(chain))

    def _collect(self, job, results: list):
        if job is None:
            return
        q, fut = job
        out = fut.result()            # the chain is enqueued (not necessarily run)
        out["stats"] = q.quantize_finish()
        self.d2h_bytes += out.pop("d2h_bytes")
        results.append(out)
        q.free_hessian()

    def step(self, from_host: bool):
        """One sweep.  Returns the packed results of the runs this rank owns."""
        import torch.distributed as dist
        import torch.nn as nn
        from distributed_gptq_b200 import GPTQ
        dev = self.device
        self.h2d_bytes = self.d2h_bytes = 0
        staged = None
        if from_host:
            # Every layer's activations cross PCIe once per step: all host->device copies are
            # queued on a side stream up front (inside the timed region) and each add_batch
            # waits only for the chunk it consumes, so copies overlap the kernels.  The four
            # runs of a layer read the same device copy.
            copy_stream = self.copy_stream
            staged = []
            with torch.cuda.stream(copy_stream):
                for li in range(len(LAYERS)):
                    chunks = []
                    for c in self._chunks(self.X_host[li]):
                        buf = c.to(dev, non_blocking=True)
                        ev = torch.cuda.Event()
                        ev.record(copy_stream)
                        chunks.append((buf, ev))
                        self.h2d_bytes += c.numel() * c.element_size()
                    staged.append(chunks)
        pending, jobs, results = [], [], []
        pool = self.pool
        # `chains="during"`: the runs with the widest input (the longest chains, K = 11008) go
        # first and every run's chain is enqueued right after its reduce.
        order = list(range(len(self.runs)))
        overlap = self.world > 1 and self.chains == "during"
        if overlap:
            order.sort(key=lambda ri: -run_cost(LAYERS[self.runs[ri][0]][1], LAYERS[self.runs[ri][0]][2]))
        for ri in order:
            li, bits, act = self.runs[ri]
            _, N_out, K = LAYERS[li]
            lin = nn.Linear(K, N_out, bias=False, device=dev, dtype=torch.bfloat16)
            lin.weight.data.copy_(self.W[li])
            q = GPTQ(lin, bits=bits, group_size=GROUP, actorder=act, percdamp=PERCDAMP,
                     blocksize=BLOCK, device=dev)
            if from_host:
                for buf, ev in staged[li]:
                    torch.cuda.current_stream().wait_event(ev)
                    q.add_batch(buf, None)
                    buf.record_stream(torch.cuda.current_stream())
            else:
                for c in self._chunks(self.X_dev[li]):
                    q.add_batch(c, None)
            work = None
            if self.world > 1:
                q.nsamples = NSEQ
                work = dist.reduce(q._Hbuf, dst=self.owner[ri], async_op=True)
            pending.append((ri, q, work))
            # One GPU, device-resident inputs: the Hessian kernels saturate the GPU (tensor pipe
            # and power cap); chains enqueued beside them only slowed both down, so they follow
            # in phase B.  Host inputs (the accumulation waits for PCIe) or several GPUs (most
            # ranks do not own the run): the chain is enqueued at once.
            if overlap or (self.world == 1 and from_host):
                jobs.append(self._launch(pending.pop(0), from_host, pool))
        pending.sort(key=lambda it: -run_cost(LAYERS[self.runs[it[0]][0]][1],
                                              LAYERS[self.runs[it[0]][0]][2]))
        while pending:
            jobs.append(self._launch(pending.pop(0), from_host, pool))
        while jobs:
            self._collect(jobs.pop(0), results)
        pool.join()
        if from_host:
            torch.cuda.current_stream().synchronize()   # the asynchronous result copies
        return results

    def hessian_flops_per_step(self):
        ex = al = 0.0
        T = len(self.my_seqs) * SEQ
        for (li, _, _) in self.runs:
            e, a = hessian_flops(LAYERS[li][2], T)
            ex += e
            al += a
        return ex, al, min(CHUNK_SEQS, len(self.my_seqs)) * SEQ


# ============================================================================= CPU baseline
def cpu_reference_sample(workload: str, variant: str, scale: float = 1.0):
    """Times the CPU restatement of the reference (oracle/) on a bounded sample of the workload
    with all host threads and extrapolates to seconds per model.

    Sample (drawn before the clocks start): the Hessian product X^T X in fp32 at the two input
    widths of the workload on a subset of the tokens; the Cholesky -> inverse -> Cholesky chain
    at both widths in full; the block / column loop at the narrow width on a subset of rows
    (rows are independent: scaled by N_out / rows and by (K / K_narrow)^2 for the wide layers).
    The reference accumulates one Hessian and one inverse per linear layer (no sharing between
    q/k/v), which is what is extrapolated.  For model workloads the calibration forward passes
    are added as FLOP / the GEMM rate measured on the Hessian product.
    """
    from oracle import oracle_gptq as O
    torch.set_num_threads(os.cpu_count() or 1)
    cores = torch.get_num_threads()
    if workload == "sweep":
        Kn, Kw, bits, group, act = 4096, 11008, 4, GROUP, True
        linears = [(n, k) for _, n, k in LAYERS for _ in SETTINGS]
        T = NSEQ * SEQ
        fwd_flop = 0.0
    else:
        spec = MODELS[workload]
        v = spec["variants"][variant]
        Kn, Kw, bits, group, act = spec["d"], spec["ffn"], v["bits"], v["group"], v["actorder"]
        linears = [(n, k) for _, n, k, _ in model_linears(spec)] * spec["layers"]
        T = spec["nseq"] * spec["seq"]
        fwd_flop = 2.0 * T * sum(n * k for n, k in linears)
    g = torch.Generator().manual_seed(0)
    tok = {Kn: max(2048, int(49152 * scale * (4096 / Kn) ** 2) // 2048 * 2048),
           Kw: max(2048, int(6144 * scale * (11008 / Kw) ** 2) // 2048 * 2048)}
    tok = {K: min(n, max(2048, T // 2048 * 2048)) for K, n in tok.items()}    # never more than the workload has
    X = {K: torch.randn(tok[K], K, generator=g) for K in (Kn, Kw)}
    rows = max(16, int(512 * scale))
    Wrows = torch.randn(rows, Kn, generator=g) * 0.02
    t_all0 = time.perf_counter()
    per_token, H_of, gemm_rate = {}, {}, 0.0
    for K in (Kn, Kw):
        H = None
        t0 = time.perf_counter()
        for s0 in range(0, tok[K], 2048):
            H, _ = O.hessian_add_batch(H, 0, X[K][s0:s0 + 2048])
        dt = time.perf_counter() - t0
        per_token[K] = dt / tok[K]
        gemm_rate = max(gemm_rate, 2.0 * tok[K] * K * K / dt)
        H_of[K] = H + torch.eye(K) * float(H.diagonal().mean())
    del X
    inv = {}
    for K in (Kn, Kw):
        t0 = time.perf_counter()
        O.damped_inv_chol(H_of[K], PERCDAMP)
        inv[K] = time.perf_counter() - t0
    t0 = time.perf_counter()
    O.gptq_quantize(Wrows, H_of[Kn], 4, bits, group, BLOCK, PERCDAMP, act)
    loop_n = max(time.perf_counter() - t0 - inv[Kn], 1e-3)
    spent = time.perf_counter() - t_all0
    parts = {"hessian": 0.0, "inverse": 0.0, "loop": 0.0, "forward": fwd_flop / gemm_rate}
    for N_out, K in linears:
        parts["hessian"] += per_token[K] * T
        parts["inverse"] += inv[K]
        parts["loop"] += loop_n * (N_out / rows) * (K / Kn) ** 2
    total = sum(parts.values())
    sample = (f"oracle port, torch fp32 CPU, {cores} threads: X^T X on {tok[Kn]} tokens (K={Kn}, "
              f"x{T / tok[Kn]:.0f} to the full token count) and {tok[Kw]} tokens (K={Kw}, "
              f"x{T / tok[Kw]:.0f}), Cholesky->inverse->Cholesky at both K in full, column loop on "
              f"{rows} rows at K={Kn} (x N_out/{rows}, x(K/{Kn})^2); {len(linears)} linears, one "
              f"Hessian and inverse each; extrapolated parts [s]: "
              + ", ".join(f"{k} {v:.0f}" for k, v in parts.items())
              + (f" (forward = {fwd_flop:.2e} FLOP at the measured {gemm_rate / 1e9:.0f} GFLOP/s)"
                 if fwd_flop else "")
              + f"; {spent:.1f} s of CPU work timed")
    return total, cores, sample


def cpu_reference_outright(workload: str, variant: str):
    """The oracle on the whole workload, nothing extrapolated (small models only): forward
    passes of the unquantized model with fp32 Hessian hooks, then every layer quantized."""
    import torch.nn as nn
    from oracle import oracle_gptq as O
    spec = MODELS[workload]
    v = spec["variants"][variant]
    torch.set_num_threads(os.cpu_count() or 1)
    model = build_model(spec, spec["layers"], "cpu")
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, spec["vocab"], (spec["nseq"], spec["seq"]), generator=g)
    block_list = "model.layers." if spec["kind"] == "llama" else "model.decoder.layers."
    layers = {n: m for n, m in model.named_modules()
              if isinstance(m, nn.Linear) and n.startswith(block_list)}
    t0 = time.perf_counter()
    H = {}

    def hook(name):
        def f(mod, args):
            H[name] = O.hessian_add_batch(H.get(name, (None, 0))[0], 0, args[0].detach())
        return f
    handles = [m.register_forward_pre_hook(hook(n)) for n, m in layers.items()]
    with torch.no_grad():
        for i in range(0, spec["nseq"], 8):
            model(input_ids=ids[i:i + 8], use_cache=False)
    for h in handles:
        h.remove()
    t_cal = time.perf_counter() - t0
    for n, m in layers.items():
        O.gptq_quantize(m.weight.data.float(), H[n][0], spec["nseq"], v["bits"], v["group"], BLOCK,
                        PERCDAMP, v["actorder"])
    total = time.perf_counter() - t0
    cores = torch.get_num_threads()
    return total, cores, (f"oracle port, torch fp32 CPU, {cores} threads, the whole workload measured "
                          f"outright: calibration forward + Hessians {t_cal:.0f} s, "
                          f"{len(layers)} layers quantized {total - t_cal:.0f} s")


# ============================================================================= main
EXCHANGE_NAMES = {"owner": "reduce to owner", "all_reduce": "all_reduce",
                  "peer": "summed by the Hessian kernels in the owner's buffer (peer reductions)"}
# Size of the CPU sample (1.0 = 3-4 s of timed work on 16 cores): the one-off cpu_baseline of
# the default run times 10-20 s; every step of the reference arm half of that, so that its
# warm-up + steps stay within a few minutes.
CPU_BASELINE_SCALE = 4.0
REF_ARM_SCALE = 2.0
E2E_BUDGET_S = 150.0      # time the host-input pass may take (see main)


def main():
    # Libraries (NCCL's version banner, for one) may write to stdout; the JSON line must be
    # the only thing there, so everything else is sent to stderr.
    real_stdout = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    sys.stdout = sys.stderr

    def emit(obj):
        real_stdout.write(json.dumps(obj) + "\n")
        real_stdout.flush()

    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama7b", choices=["llama7b", "sweep", "opt1.3b",
                                                              "llama13b", "opt125m"])
    ap.add_argument("--variant", default=None, help="quantization setting of a model workload")
    ap.add_argument("--exchange", default="owner", choices=["owner", "all_reduce", "peer"],
                    help="how partial Hessians are summed: NCCL reduce to the owner, NCCL "
                         "all_reduce (the reference's flow), or by the Hessian kernels "
                         "themselves into the owner's buffer over NVLink")
    ap.add_argument("--layers", type=int, default=0,
                    help="debugging: fewer decoder blocks than the named model (flagged in config)")
    ap.add_argument("--true-sequential", action="store_true")
    ap.add_argument("--blocks-in-flight", type=int, default=None,
                    help="blocks whose chains are enqueued but not collected (default: the "
                         "library's choice, 2 up to two ranks, 4 above)")
    ap.add_argument("--sweep-chains", default="after", choices=["during", "after"],
                    help="sweep on several GPUs: enqueue a run's chain after all Hessians (default) or "
                         "right after its reduce, beside the remaining Hessian kernels (measured slower: "
                         "the chains are on the critical path and run 3x slower on a busy GPU)")
    ap.add_argument("--cpu-outright", action="store_true",
                    help="reference arm: time the whole workload on the CPU (small models only)")
    ap.add_argument("--linear-check", action="store_true",
                    help="model workloads: also run the packed 4-bit linear at batch 1/4/16 on the "
                         "model's layer shapes against dequantize + matmul")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-input pass")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    metric, unit = "gptq_wall_clock_s_per_model", "s/model"
    is_model = args.workload != "sweep"
    variant = args.variant
    if is_model:
        spec = MODELS[args.workload]
        variant = variant or next(iter(spec["variants"]))
        if variant not in spec["variants"]:
            raise SystemExit(f"--variant must be one of {list(spec['variants'])}")
    par = (f"dp{world} calibration + layer-parallel quantization, Hessian exchange: "
           f"{EXCHANGE_NAMES[args.exchange]}") if world > 1 \
        else "single GPU"

    if args.impl == "reference":
        if rank != 0:
            return
        times = []
        for i in range(args.warmup + args.steps):
            if args.cpu_outright and is_model:
                t, cores, sample = cpu_reference_outright(args.workload, variant)
            else:
                t, cores, sample = cpu_reference_sample(args.workload, variant, REF_ARM_SCALE)
            if i >= args.warmup:
                times.append(t)
        v = sum(times) / len(times)
        if is_model:
            s, q = MODELS[args.workload], MODELS[args.workload]["variants"][variant]
            wl = (f"{s['name']}, calibration {s['nseq']} x {s['seq']}, GPTQ {q['bits']}-bit group "
                  f"{q['group']} act-order {'on' if q['actorder'] else 'off'}: the reference's "
                  f"algorithm (CPU restatement) on this workload")
        else:
            wl = "layer sweep (3 linear layers x {4,3}-bit x act-order {off,on}), CPU restatement"
        emit(({
            "impl": "reference", "metric": metric, "value": v, "unit": unit, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": v * 1e3,
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": {"workload": wl, "parallelism": f"{cores} host threads"},
            "cpu_baseline": {"value": v, "unit": unit, "cores": cores, "kind": "port",
                             "sample": sample},
            "e2e": {"value": v, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}))
        return

    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (this package has no CPU path)")
    if args.gpus != world:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        from distributed_gptq_b200.communication import group_options
        dist.init_process_group("nccl", device_id=device, **group_options("nccl"))
    from distributed_gptq_b200 import _C
    _C.device_check()

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps, label):
        sync_all()
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        marks[0].record()
        mallocs = []
        for i in range(steps):
            m0 = torch.cuda.memory_stats(device).get("num_device_alloc", 0)
            fn()
            marks[i + 1].record()
            mallocs.append(torch.cuda.memory_stats(device).get("num_device_alloc", 0) - m0)
        sync_all()
        per_step = [marks[i].elapsed_time(marks[i + 1]) for i in range(steps)]
        print(f"[bench] rank {rank} {label}: ms per step {[round(t, 1) for t in per_step]}, "
              f"cudaMalloc calls per step {mallocs}", file=sys.stderr, flush=True)
        ms = torch.tensor([marks[0].elapsed_time(marks[steps])], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms) / steps

    t_build = time.time()
    if is_model:
        n_layers = args.layers or spec["layers"]
        wl = ModelWorkload(spec, variant, n_layers, rank, world, device, args.exchange,
                           true_sequential=args.true_sequential,
                           blocks_in_flight=args.blocks_in_flight)
        step_dev, step_host = (lambda: wl.step(False)), (lambda: wl.step(True))
    else:
        wl = Sweep(rank, world, device, args.sweep_chains)
        wl.load_device_inputs()
        step_dev, step_host = (lambda: wl.step(False)), (lambda: wl.step(True))
    print(f"[bench] rank {rank}: workload built in {time.time() - t_build:.1f} s", file=sys.stderr,
          flush=True)
    for _ in range(args.warmup):
        step_dev()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    timers = _C.KernelTimers()
    _C.set_timers(timers)
    launches0 = _C.launch_count()
    phase_acc = {}
    if is_model:
        def step_dev_acc():
            qz = wl.step(False)
            for k, v in qz.timings.items():
                phase_acc[k] = phase_acc.get(k, 0.0) + v
        ms_step = timed(step_dev_acc, args.steps, "device-resident")
    else:
        ms_step = timed(step_dev, args.steps, "device-resident")
    launches = _C.launch_count() - launches0
    _C.set_timers(None)
    clocks = sampler.stop() if rank == 0 else None
    ksum = timers.summary()
    lt = torch.tensor([float(launches)], device=device)
    if world > 1:
        dist.all_reduce(lt)

    e2e = None
    if not args.no_e2e:
        if not is_model:
            wl.load_host_inputs()
            wl.X_dev = None
            torch.cuda.empty_cache()
        # The host-input pass repeats the same job: it takes as many steps as fit in about
        # E2E_BUDGET_S (at least 3, at most --steps), so that a long --steps does not double
        # the run; every rank derives the same count from the reduced step time.
        e2e_steps = max(1, min(args.steps, max(3, int(E2E_BUDGET_S / max(ms_step / 1e3, 1e-3)))))
        for _ in range(1 if ms_step > 2000 else min(2, max(1, args.warmup))):   # allocator / pinned buffers
            step_host()
        ms_e2e = timed(step_host, e2e_steps, "host inputs")
        bt = torch.tensor([float(wl.h2d_bytes), float(wl.d2h_bytes)], device=device)
        if world > 1:
            dist.all_reduce(bt)
        e2e = {"value": ms_e2e / 1e3, "unit": unit, "h2d_bytes_per_step": int(bt[0]),
               "d2h_bytes_per_step": int(bt[1]), "steps": e2e_steps}

    if rank == 0:
        pk = peaks()
        # roofline of the flop-dominant kernel of the library (Hessian), from the events
        # recorded live around every dgq_hessian_accum call of the timed region on this rank
        n_calls, hess_ms = ksum.get("hessian_accum", (0, 0.0))
        ex, al, tokens_per_call = wl.hessian_flops_per_step()
        if is_model:
            tokens_per_call = min(spec["batch"], wl.my_seqs) * spec["seq"]
        ex *= args.steps
        al *= args.steps
        achieved = ex / (hess_ms * 1e-3) / 1e12 if hess_ms > 0 else None
        total_ms = sum(v[1] for v in ksum.values()) or 1.0
        kernels = {k: {"calls": v[0], "ms": round(v[1], 3), "share": round(v[1] / total_ms, 4)}
                   for k, v in sorted(ksum.items(), key=lambda kv: -kv[1][1])}
        # DRAM traffic per launch, averaged over the launch shapes of a step
        if is_model:
            Ks = [K for _, _, K, sh in model_linears(spec) if sh is None]
        else:
            Ks = [LAYERS[li][2] for li, _, _ in wl.runs]
        traffic = sum(hessian_traffic(K, tokens_per_call) for K in Ks) / len(Ks) if n_calls else None
        roofline = {
            "kernel": "hessian_syrk_kernel (dgq_hessian_accum)", "bound": "tensor",
            "achieved": achieved, "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
            "frac": achieved / pk["bf16_tflops_sustained"] if achieved else None,
            "peak_source": f"{pk['source']} sustained cuBLAS bf16 (burst {pk['bf16_tflops']})",
            "flops_counted": "executed (upper-triangle 256x256 tiles); the algorithmic 2*T*K^2 rate is "
                             f"{al / (hess_ms * 1e-3) / 1e12:.1f} TFLOP/s" if hess_ms > 0 else "",
            "launches": n_calls, "avg_launch_ms": hess_ms / n_calls if n_calls else None,
            "tokens_per_launch": tokens_per_call,
            "traffic": traffic,
            "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of single-launch captures "
                              "(K=4096/T=65536: 575.5 MB, K=11008/T=32768: 4.148 GB), scaled by the "
                              "tokens per launch and averaged over the launch shapes of a step"
            if traffic else None,
            "kernels_by_time": kernels,
            "kernels_by_time_note": "per-call CUDA-event sums on the call's own stream; chains of "
                                    "different layers overlap, so these do not add up to the step",
        }
        phases = None
        if is_model and phase_acc:
            per = {k: round(v / args.steps, 4) for k, v in phase_acc.items()}
            lib = {k: round(v[1] * 1e-3 / args.steps, 4) for k, v in ksum.items()}
            phases = {
                "per_step_s": {
                    "calibration_forward_incl_hessian": per.get("forward_s"),
                    "hessian_kernels": lib.get("hessian_accum"),
                    "exchange_reduce": per.get("exchange_s", 0.0),
                    "prepare_permute": round(lib.get("prepare", 0.0) + lib.get("permute", 0.0), 4),
                    "inverse": lib.get("inv_chol"), "quantize": lib.get("gptq_quantize"),
                    "pack": lib.get("pack"), "share_broadcast": per.get("share_s", 0.0),
                    "host_waiting_for_chains": per.get("host_wait_s", 0.0),
                    "host_enqueueing_forward": per.get("host_enqueue_forward_s"),
                    "host_enqueueing_chains": per.get("host_enqueue_chains_s"),
                    "host_setup": per.get("host_setup_s"),
                    "host_capture_of_first_block_inputs": per.get("host_capture_s"),
                    "host_replay_check": per.get("host_replay_check_s"),
                    "host_collecting_last_blocks": per.get("host_tail_collect_s"),
                    "host_final_sync": per.get("host_final_sync_s"),
                    "quantize_model_total": per.get("total_s")},
                "note": "rank 0; forward is measured on the main stream, the chain phases on side "
                        "streams that run beside it, collectives from issue to completion",
                "hessian_tflops_executed": achieved,
            }
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            v, cores, sample = cpu_reference_sample(args.workload, variant, CPU_BASELINE_SCALE)
            cpu = {"value": v, "unit": unit, "cores": cores, "kind": "port", "sample": sample}
        if is_model:
            config = {"workload": wl.describe(),
                      "l2": "one block's calibration activations (>= 0.5 GB per pass) exceed L2; no flush",
                      "parallelism": par, "calibration_batch": spec["batch"],
                      "e2e_note": "weights start on the device (the model is resident, as in the "
                                  "reference's flow); token ids come from pinned host memory and the "
                                  "packed tensors go back to it"}
        else:
            config = {"workload": "layer sweep (3 bf16 linear layers 4096x4096, 11008x4096, 4096x11008; "
                                  "128x2048 calibration tokens each; {4,3}-bit g128 x act-order {off,on}; "
                                  "12 GPTQ runs per step)",
                      "l2": "inputs larger than L2 (2.1-5.8 GB of activations per layer), no flush needed",
                      "parallelism": par,
                      "e2e_note": "weights start on the device; activations come from pinned host memory"}
        out = {
            "metric": metric, "value": ms_step / 1e3, "unit": unit, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16"
            if not is_model or spec["dtype"] == "bf16" else "f32",
            "data": "synthetic", "config": config, "clocks": clocks, "e2e": e2e,
            "gpu_launches": int(lt[0]), "roofline": roofline, "cpu_baseline": cpu}
        if phases:
            out["phases"] = phases
        if is_model and args.linear_check:
            out["linear_check"] = linear_check(spec, device, False) + linear_check(spec, device, True)
        emit(out)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
