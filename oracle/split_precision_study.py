"""How many GPTQ codes change when the trailing update ``W[:, i2:] -= Err @ U[i1:i2, i2:]`` is
computed with a cheaper split of its fp32 operands.  TEST INFRASTRUCTURE (CPU study).

    python oracle/split_precision_study.py

The column loop is the oracle's (``oracle_gptq.gptq_quantize``: scale/zero, quantize, error
feedback inside a block); only the product of the lazy update is replaced by an emulation of a
tensor-core product: each operand is split into 1, 2 or 3 terms of the narrow type
(bf16 or tf32, round to nearest), the products of the terms are exact, their sum is wide.

    tf32x1 / bf16x1   one product of the rounded operands
    tf32x3 / bf16x3   hi*hi + hi*lo + lo*hi          (two terms per operand)
    bf16x6            three terms per operand, the six products of order <= 2

Printed per case: share of codes equal to the fp32 product's codes, the largest code
difference, and the ratio of the reconstruction errors.  The numbers this study gave are in
the design notes; tf32x3 is what the library's kernel (csrc/tgemm.cu) computes.
"""
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from oracle import oracle_gptq as O
torch.set_num_threads(8)

def rt(x, kind):
    if kind == "bf16": return x.bfloat16().float()
    if kind == "tf32":  # round to 10 explicit mantissa bits (rna)
        i = x.view(torch.int32)
        i = (i + 0x1000) & ~0x1FFF
        return i.view(torch.float32)
def split(x, kind, terms):
    out, r = [], x.clone()
    for _ in range(terms):
        h = rt(r, kind); out.append(h); r = r - h
    return out
def prod(A, B, mode):
    if mode == "fp32": return A @ B
    kind, n = mode.split("x"); n = int(n)
    terms = {1: 1, 3: 2, 6: 3}[n]
    a, b = split(A, kind, terms), split(B, kind, terms)
    acc = torch.zeros(A.shape[0], B.shape[1], dtype=torch.float64)
    for i in range(terms):
        for j in range(terms):
            if i + j < terms:
                acc += a[i].double() @ b[j].double()   # products exact, accumulation wide
    return acc.float()

def quantize(W, U, bits, g, mode, blocksize=128):
    W = W.clone(); N, K = W.shape; maxq = 2**bits - 1
    codes = torch.zeros((N, K), dtype=torch.uint8); Q = torch.zeros_like(W)
    scale = torch.zeros(N, K // g); zero = torch.zeros(N, K // g)
    for i1 in range(0, K, blocksize):
        i2 = min(i1 + blocksize, K)
        W1 = W[:, i1:i2].clone(); Err = torch.zeros_like(W1)
        for j in range(i2 - i1):
            c = i1 + j
            if c % g == 0:
                s, z = O.find_params(W[:, c:c + g], maxq); scale[:, c // g] = s; zero[:, c // g] = z
            s, z = scale[:, c // g], zero[:, c // g]
            w = W1[:, j]; q, wh = O.quantize_column(w, s, z, maxq)
            e = (w - wh) / U[c, c]
            W1[:, j + 1:] -= e.unsqueeze(1) * U[c, c + 1:i2].unsqueeze(0)
            Err[:, j] = e; codes[:, c] = q.to(torch.uint8); Q[:, c] = wh
        if i2 < K:
            W[:, i2:] -= prod(Err, U[i1:i2, i2:], mode)
    return codes, Q

for K, T in ((2048, 8192), (4096, 16384)):
    g = torch.Generator().manual_seed(K)
    X = torch.randn(T, K, generator=g); X[:, ::97] *= 20
    H = X.t() @ X
    W = (torch.randn(128, K, generator=g) * 0.02)
    Hn = H * (2.0 / 8)
    U = O.damped_inv_chol(Hn, 0.01)
    for bits in (4, 3):
        base, Qb = quantize(W, U, bits, 128, "fp32")
        rb = O.recon_error(W, Qb, H)
        for mode in ("tf32x3", "bf16x6", "bf16x3", "tf32x1", "bf16x1"):
            t0 = time.time()
            c, Q = quantize(W, U, bits, 128, mode)
            d = (c.int() - base.int()).abs()
            print(f"K={K} bits={bits} {mode}: match {float((d==0).float().mean())*100:.4f}% maxdiff {int(d.max())} "
                  f"recon ratio {O.recon_error(W, Q, H)/rb:.5f} ({time.time()-t0:.0f}s)", flush=True)
