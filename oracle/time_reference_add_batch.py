"""Times the reference's own ``GPTQ.add_batch`` (core/gptq.py:63-89, loaded by file path) next to
the oracle's restatement of it, on the host cores of the machine it is run on.
TEST INFRASTRUCTURE; needs the reference checkout (see ref_shim.py).

    python oracle/time_reference_add_batch.py [tokens_per_call] [calls]

Prints seconds per call and GFLOP/s (2*T*K^2 per call) for the two input widths of the
Llama-2-7B layers.  The reference's ``quantize()`` raises on every input, so the Hessian stage
is the only part of the path that can be timed on the reference itself.
"""
import logging
import os
import sys
import time

import torch
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from oracle import oracle_gptq as O  # noqa: E402
from oracle import ref_shim  # noqa: E402


def main():
    T = int(sys.argv[1]) if len(sys.argv) > 1 else 2048
    calls = int(sys.argv[2]) if len(sys.argv) > 2 else 4
    torch.set_num_threads(os.cpu_count() or 1)
    logging.disable(logging.CRITICAL)
    G = ref_shim.load_gptq()
    g = torch.Generator().manual_seed(0)
    for K in (4096, 11008):
        x = torch.randn(1, T, K, generator=g)
        q = G.GPTQ(nn.Linear(K, 8, bias=False), device=torch.device("cpu"))
        q.add_batch(x, None)                      # allocation and warm-up
        t0 = time.perf_counter()
        for _ in range(calls):
            q.add_batch(x, None)
        t_ref = (time.perf_counter() - t0) / calls
        H, n = O.hessian_add_batch(None, 0, x)
        t0 = time.perf_counter()
        for _ in range(calls):
            H, n = O.hessian_add_batch(H, n, x)
        t_or = (time.perf_counter() - t0) / calls
        flop = 2.0 * T * K * K
        print(f"K={K} T={T}: reference add_batch {t_ref:.3f} s/call ({flop / t_ref / 1e9:.0f} GFLOP/s), "
              f"oracle {t_or:.3f} s/call ({flop / t_or / 1e9:.0f} GFLOP/s), "
              f"{torch.get_num_threads()} threads")


if __name__ == "__main__":
    main()
