#!/usr/bin/env python
"""Benchmark of the GPTQ quantization path on B200.

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the CPU restatement of the reference, timed

Workload ("layer sweep"): three bf16 linear layers (N_out x K) 4096x4096, 11008x4096 and
4096x11008 with weights ~N(0, 0.02); per layer 128 calibration sequences x 2048 tokens of
activations ~N(0,1) with 1 % of the channels scaled by 20; each layer is quantized four
times (4-bit and 3-bit, group 128, act-order off and on, blocksize 128, percdamp 0.01).
One step = the 12 independent GPTQ runs, each: Hessian accumulation over all tokens ->
damped inverse factor -> blockwise quantization -> packing.  The Hessians of all runs are
accumulated first; the 12 chains inverse -> quantization -> packing then run on six side
streams beside each other (with host inputs on one GPU a chain starts as soon as its
Hessian is complete and fills the time the accumulation waits for PCIe).  All inputs are synthetic and
seeded.  Activations (2.1 - 5.8 GB per layer) are far larger than L2, so no flush is needed
between iterations.

`value` is seconds per sweep with activations already resident in HBM; `e2e` is the same
with activations starting in pinned host memory (copied inside the timed region) and the
packed results copied back to the host.  At N > 1 the sequences of every run are split
over the ranks (data-parallel calibration), partial Hessians are reduced to the rank that
owns the run, and the 12 runs are spread over the ranks (layer-parallel quantization):
total work is fixed, i.e. strong scaling.
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

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYERS = [("4096x4096", 4096, 4096), ("11008x4096", 11008, 4096), ("4096x11008", 4096, 11008)]
SETTINGS = [(4, False), (4, True), (3, False), (3, True)]   # (bits, act-order)
NSEQ, SEQ = 128, 2048
GROUP, BLOCK, PERCDAMP = 128, 128, 0.01
CHUNK_SEQS = 32          # sequences per add_batch call
HESS_TILE = 256


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


# ----------------------------------------------------------------------------- synthetic data
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


# ----------------------------------------------------------------------------- the step
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
    def __init__(self, rank: int, world: int, device):
        from distributed_gptq_b200 import _C  # noqa: F401  (fails loudly without the library)
        self.rank, self.world, self.device = rank, world, device
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
        only enqueued here, on one of the pool's side streams; `_collect` waits for it."""
        from distributed_gptq_b200 import _C
        ri, q, work = item
        if work is not None:
            work.wait()
        if self.owner[ri] != self.rank:
            q.free_hessian()
            return None
        bits = self.runs[ri][1]
        fmt = _C.FMT_BYTES_LO_FIRST if bits == 4 else _C.FMT_INT32_LE

        def chain():
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
        # The chains of the runs this rank owns (damped inverse, block quantization, packing:
        # long sequences of short dependent kernels that leave most SMs idle) are spread over
        # six side streams and run beside each other (2 / 4 / 6 / 12 streams: 240 / 225 / 220 /
        # 220 ms per step; enqueueing all chains costs the host 18-30 ms, hidden under phase A).
        pool = self.pool
        # ---- phase A: data-parallel Hessian accumulation, reduce to the owner
        for ri, (li, bits, act) in enumerate(self.runs):
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
            # Host inputs on one GPU: the accumulation waits for PCIe most of the time, so a
            # run's chain is enqueued at once and fills the gaps between the Hessian kernels.
            # Device-resident inputs: the Hessian kernels saturate the GPU (tensor pipe and power
            # cap), chains enqueued beside them only slowed both down in measurements, so they
            # follow in phase B.  Several GPUs:
            # every reduce is a meeting point of all ranks, so all Hessians are accumulated and
            # reduced first.
            if self.world == 1 and from_host:
                jobs.append(self._launch(pending.pop(0), from_host, pool))
        # ---- phase B: layer-parallel quantization of whatever has not been enqueued yet, the
        # longest chains first (enqueueing a chain costs the host a few milliseconds, so the
        # long ones should be on their way while the short ones are still being enqueued)
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


def hessian_flops(K: int, T: int):
    P = -(-K // HESS_TILE)
    executed = (P * (P + 1) // 2) * 2.0 * HESS_TILE * HESS_TILE * T
    return executed, 2.0 * T * K * K


# ----------------------------------------------------------------------------- CPU baseline
def cpu_reference_sample(scale: float = 1.0):
    """Times the CPU restatement of the reference (oracle/) on a bounded sample of the sweep
    with all host threads and extrapolates to seconds per sweep.

    Sample: Hessian X^T X (fp32) at K=4096 and K=11008 on a subset of the tokens; the
    Cholesky -> inverse -> Cholesky chain at both K in full; the block / column loop at
    K=4096 on a subset of rows (rows are independent: scaled by N_out / rows and by
    (K/4096)^2 for K=11008).
    """
    from oracle import oracle_gptq as O
    torch.set_num_threads(os.cpu_count() or 1)
    cores = torch.get_num_threads()
    g = torch.Generator().manual_seed(0)
    t_all0 = time.perf_counter()
    tok4, tok11 = int(49152 * scale), int(6144 * scale)
    per_token, H_of = {}, {}
    for K, tok in ((4096, tok4), (11008, tok11)):
        H, chunk = None, 2048
        t0 = time.perf_counter()
        for s0 in range(0, tok, chunk):
            x = torch.randn(min(chunk, tok - s0), K, generator=g)
            H, _ = O.hessian_add_batch(H, 0, x)
        per_token[K] = (time.perf_counter() - t0) / tok   # includes drawing the sample
        H_of[K] = H + torch.eye(K) * float(H.diagonal().mean())
    inv = {}
    for K in (4096, 11008):
        t0 = time.perf_counter()
        O.damped_inv_chol(H_of[K], PERCDAMP)
        inv[K] = time.perf_counter() - t0
    rows = max(16, int(512 * scale))
    W = torch.randn(rows, 4096, generator=g) * 0.02
    t0 = time.perf_counter()
    O.gptq_quantize(W, H_of[4096], 4, 4, GROUP, BLOCK, PERCDAMP, True)
    loop4 = max(time.perf_counter() - t0 - inv[4096], 1e-3)
    total = 0.0
    T = NSEQ * SEQ
    for _, N_out, K in LAYERS:
        hess = per_token[K] * T
        loop = loop4 * (N_out / rows) * (K / 4096) ** 2
        total += len(SETTINGS) * (hess + inv[K] + loop)
    sample = (f"oracle port, torch fp32 CPU, {cores} threads: X^T X on {tok4} tokens (K=4096) and "
              f"{tok11} tokens (K=11008), Cholesky->inverse->Cholesky at K=4096 and K=11008 in "
              f"full, column loop on {rows} rows at K=4096; extrapolated linearly in tokens and "
              f"rows and with K^2 for the loop; {time.perf_counter() - t_all0:.1f} s of CPU work")
    return total, cores, sample


# ----------------------------------------------------------------------------- main
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
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-input pass")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    metric, unit = "gptq_wall_clock_s_per_model", "s/model"
    config = {"workload": "layer sweep (3 bf16 linear layers 4096x4096, 11008x4096, 4096x11008; "
                          "128x2048 calibration tokens each; {4,3}-bit g128 x act-order {off,on}; "
                          "12 GPTQ runs per step)",
              "l2": "inputs larger than L2 (2.1-5.8 GB of activations per layer), no flush needed",
              "parallelism": f"dp{world} calibration + layer-parallel quantization"
              if world > 1 else "single GPU"}

    if args.impl == "reference":
        if rank != 0:
            return
        times = []
        for i in range(args.warmup + args.steps):
            t, cores, sample = cpu_reference_sample(scale=0.5)
            if i >= args.warmup:
                times.append(t)
        v = sum(times) / len(times)
        emit(({
            "impl": "reference", "metric": metric, "value": v, "unit": unit, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": v * 1e3,
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": config,
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
        dist.init_process_group("nccl", device_id=device)
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

    sweep = Sweep(rank, world, device)
    sweep.load_device_inputs()
    for _ in range(args.warmup):
        sweep.step(False)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    timers = _C.KernelTimers()
    _C.set_timers(timers)
    launches0 = _C.launch_count()
    ms_step = timed(lambda: sweep.step(False), args.steps, "device-resident")
    launches = _C.launch_count() - launches0
    _C.set_timers(None)
    clocks = sampler.stop() if rank == 0 else None
    ksum = timers.summary()
    lt = torch.tensor([float(launches)], device=device)
    if world > 1:
        dist.all_reduce(lt)

    e2e = None
    if not args.no_e2e:
        sweep.load_host_inputs()
        sweep.X_dev = None
        torch.cuda.empty_cache()
        for _ in range(min(2, max(1, args.warmup))):   # allocator warm-up for the host path
            sweep.step(True)
        ms_e2e = timed(lambda: sweep.step(True), max(1, args.steps), "host inputs")
        bt = torch.tensor([float(sweep.h2d_bytes), float(sweep.d2h_bytes)], device=device)
        if world > 1:
            dist.all_reduce(bt)
        e2e = {"value": ms_e2e / 1e3, "unit": unit, "h2d_bytes_per_step": int(bt[0]),
               "d2h_bytes_per_step": int(bt[1])}

    if rank == 0:
        pk = peaks()
        # roofline of the flop-dominant kernel (Hessian), from the events recorded live
        # around every dgq_hessian_accum call of the timed region on this rank
        n_calls, hess_ms = ksum.get("hessian_accum", (0, 0.0))
        ex = al = 0.0
        my_tokens_per_call = min(CHUNK_SEQS, len(sweep.my_seqs)) * SEQ
        for (li, _, _) in sweep.runs:
            K = LAYERS[li][2]
            e, a_ = hessian_flops(K, len(sweep.my_seqs) * SEQ)
            ex += e
            al += a_
        ex *= args.steps
        al *= args.steps
        achieved = ex / (hess_ms * 1e-3) / 1e12 if hess_ms > 0 else None
        total_ms = sum(v[1] for v in ksum.values()) or 1.0
        kernels = {k: {"calls": v[0], "ms": round(v[1], 3), "share": round(v[1] / total_ms, 4)}
                   for k, v in sorted(ksum.items(), key=lambda kv: -kv[1][1])}
        roofline = {
            "kernel": "hessian_syrk_kernel (dgq_hessian_accum)", "bound": "tensor",
            "achieved": achieved, "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
            "frac": achieved / pk["bf16_tflops_sustained"] if achieved else None,
            "peak_source": f"{pk['source']} sustained cuBLAS bf16 (burst {pk['bf16_tflops']})",
            "flops_counted": "executed (upper-triangle 256x256 tiles); the algorithmic 2*T*K^2 rate is "
                             f"{al / (hess_ms * 1e-3) / 1e12:.1f} TFLOP/s" if hess_ms > 0 else "",
            "launches": n_calls, "avg_launch_ms": hess_ms / n_calls if n_calls else None,
            "tokens_per_launch": my_tokens_per_call,
            "traffic": None,
            "kernels_by_time": kernels,
        }
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            # the sample is sized for 10-30 s of CPU work: a fast host gets a larger one
            t0 = time.perf_counter()
            v, cores, sample = cpu_reference_sample()
            spent = time.perf_counter() - t0
            if spent < 10.0:
                v, cores, sample = cpu_reference_sample(scale=min(4.0, 15.0 / max(spent, 1.0)))
            cpu = {"value": v, "unit": unit, "cores": cores, "kind": "port", "sample": sample}
        emit(({
            "metric": metric, "value": ms_step / 1e3, "unit": unit, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": config, "clocks": clocks, "e2e": e2e,
            "gpu_launches": int(lt[0]), "roofline": roofline, "cpu_baseline": cpu}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
