"""Runs one kernel of the library a few times on a small seeded case, for profilers.

    python profile_case.py hessian   --K 4096 --T 32768
    python profile_case.py inv_chol  --K 4096
    python profile_case.py quantize  --K 4096 --N 4096
    python profile_case.py pack      --K 8192 --N 16384
    python profile_case.py dequant   --K 8192 --N 16384
    python profile_case.py qlinear   --K 5120 --N 5120 --M 16
    python profile_case.py gemm      --K 4096 --N 4096 --T 4096     (m = T, n = N, k = K)

Prints the CUDA-event time of each repetition and the derived rate (algorithmic flops
or bytes over time).  Sizes default to a few hundred MB so that a profiler capture ends
quickly while the inputs still exceed the L2 cache.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from distributed_gptq_b200 import _C  # noqa: E402


def _time(fn, reps):
    out = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b))
    return out


def _time_raw(call, reps, inner=50):
    """Average time of `inner` back-to-back raw library calls (no Python wrapper work in
    between, so kernels of a few microseconds are not hidden behind host overhead)."""
    out = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(inner):
            call()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b) / inner)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["hessian", "inv_chol", "quantize", "pack", "dequant", "qlinear", "gemm"])
    ap.add_argument("--K", type=int, default=4096)
    ap.add_argument("--N", type=int, default=4096)
    ap.add_argument("--T", type=int, default=32768)
    ap.add_argument("--M", type=int, default=16)
    ap.add_argument("--bits", type=int, default=4)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--beta", type=float, default=0.0, help="gemm: C = A B^T + beta C")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"], help="qlinear: activation type")
    ap.add_argument("--upper", action="store_true",
                    help="hessian: update only the part on and above the diagonal")
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    _C.device_check()
    g = torch.Generator(device=dev).manual_seed(0)
    K, N, T = a.K, a.N, a.T
    if a.case == "hessian":
        X = torch.randn(T, K, generator=g, device=dev).to(torch.bfloat16)
        H = torch.zeros((K, K), dtype=torch.float32, device=dev)
        ts = _time(lambda: _C.hessian_accum(X, H, 1.0, a.splits, upper_only=a.upper), a.reps)
        P = -(-K // 256)
        ex = (P * (P + 1) // 2) * 2.0 * 256 * 256 * T
        for t in ts:
            print(f"hessian K={K} T={T}: {t:.3f} ms  executed {ex / t / 1e9:.1f} TFLOP/s  "
                  f"algorithmic {2.0 * T * K * K / t / 1e9:.1f} TFLOP/s")
    elif a.case == "gemm":
        m = T
        A = torch.randn(m, K, generator=g, device=dev)
        B = torch.randn(N, K, generator=g, device=dev)
        C0 = torch.randn(m, N, generator=g, device=dev)
        C = C0.clone()
        want = A.double() @ B.double().t() + a.beta * C0.double()

        def run():
            C.copy_(C0)
            _C.gemm_f32(A, B, C, False, beta=a.beta)
        run()
        err = float((C.double() - want).norm() / want.norm())
        for t in _time(lambda: _C.gemm_f32(A, B, C, False, beta=a.beta), a.reps):
            print(f"gemm_f32 m={m} n={N} k={K}: {t:.3f} ms  {2.0 * m * N * K / t / 1e9:.1f} TFLOP/s "
                  f"fp32-equivalent  rel. error vs fp64 {err:.2e}")
    elif a.case in ("inv_chol", "quantize"):
        X = torch.randn(2 * K, K, generator=g, device=dev).to(torch.bfloat16)
        H = torch.zeros((K, K), dtype=torch.float32, device=dev)
        _C.hessian_accum(X, H)
        Hp, _ = _C.hessian_prepare(H, 1.0, 0.01, None)
        if a.case == "inv_chol":
            A = Hp.clone()

            def f():
                A.copy_(Hp)
                _C.inv_chol_upper(A)
            for t in _time(f, a.reps):
                print(f"inv_chol K={K}: {t:.3f} ms (incl. one K^2 copy)  {2 * K ** 3 / 3 / t / 1e9:.2f} TFLOP/s")
        else:
            U = _C.inv_chol_upper(Hp)
            W0 = torch.randn(N, K, generator=g, device=dev) * 0.02
            W = W0.clone()

            def f():
                W.copy_(W0)
                _C.gptq_quantize(W, U, a.bits, 128, 128)
            for t in _time(f, a.reps):
                print(f"gptq_quantize N={N} K={K}: {t:.3f} ms  trailing update "
                      f"{N * K * (K - 128) / t / 1e9:.2f} TFLOP/s")
    elif a.case in ("pack", "dequant"):
        codes = torch.randint(0, 2 ** a.bits, (N, K), generator=g, device=dev, dtype=torch.uint8)
        import ctypes
        P = lambda t: ctypes.c_void_p(t.data_ptr())
        L = _C.lib()
        if a.case == "pack":
            outp = _C.pack(codes, a.bits, _C.FMT_BYTES_LO_FIRST)
            call = lambda: L.dgq_pack(P(codes), N, K, a.bits, _C.FMT_BYTES_LO_FIRST, P(outp), None)
            for t in _time_raw(call, a.reps):
                nbytes = N * K * (1 + a.bits / 8)
                print(f"pack N={N} K={K} bits={a.bits}: {t:.3f} ms  {nbytes / t / 1e6:.1f} GB/s")
        else:
            packed = _C.pack(codes, a.bits, _C.FMT_BYTES_LO_FIRST)
            ng = K // 128
            s = torch.rand(N, ng, generator=g, device=dev).half()
            z = torch.randint(0, 2 ** a.bits, (N, ng), generator=g, device=dev).half()
            outd = torch.empty((N, K), dtype=torch.bfloat16, device=dev)
            call = lambda: L.dgq_unpack_dequant(P(packed), P(s), P(z), None, N, K, ng, a.bits, 128,
                                                _C.FMT_BYTES_LO_FIRST, _C.F16, _C.BF16, P(outd), None)
            for t in _time_raw(call, a.reps):
                nbytes = N * K * (a.bits / 8 + 2) + 4 * N * ng
                print(f"unpack_dequant N={N} K={K} bits={a.bits}: {t:.3f} ms  {nbytes / t / 1e6:.1f} GB/s")
    else:
        codes = torch.randint(0, 16, (N, K), generator=g, device=dev, dtype=torch.uint8)
        qw = _C.pack(codes, 4, _C.FMT_BYTES_LO_FIRST)
        ng = K // 128
        s = torch.rand(N, ng, generator=g, device=dev).half() * 0.01
        z = torch.randint(0, 16, (N, ng), generator=g, device=dev).half()
        tdt, cdt = (torch.bfloat16, _C.BF16) if a.dtype == "bf16" else (torch.float16, _C.F16)
        x = torch.randn(a.M, K, generator=g, device=dev).to(tdt)
        import ctypes
        P = lambda t: ctypes.c_void_p(t.data_ptr())
        y = torch.empty((a.M, N), dtype=tdt, device=dev)
        L = _C.lib()
        call = lambda: L.dgq_qlinear_forward(P(x), cdt, a.M, P(qw), P(s), P(z), None, None, 0, N, K,
                                             ng, 4, 128, P(y), None)
        for t in _time_raw(call, a.reps):
            nbytes = N * K / 2 + 4 * N * ng + 2 * a.M * (K + N)
            print(f"qlinear {a.dtype} M={a.M} N={N} K={K}: {t * 1e3:.1f} us  {nbytes / t / 1e6:.1f} GB/s  "
                  f"{2.0 * a.M * N * K / t / 1e9:.1f} TFLOP/s")


if __name__ == "__main__":
    main()
