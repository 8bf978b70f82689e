"""Generates the golden fixtures in this directory.

Run from the repository root in a container that has the reference tree:

    python tests/golden/make_golden.py

* ``ref_pins.npz``     - inputs and outputs of the reference's own runnable code
  (``GPTQ.add_batch``, ``GPTQ.pack_weights``, ``QuantizedLinear.pack_weights`` /
  ``unpack_weights``, ``GPTQDequantizer._unpack_4bit``) plus the reference's
  scalar expressions for scale/zero and quantize/dequantize
  (``core/gptq.py:165-169,175,179``) evaluated on fixed inputs.
* ``oracle_cases.npz`` - small GPTQ cases (inputs and every output of
  ``oracle.oracle_gptq.gptq_quantize``), so the GPU tests can also compare with
  committed numbers instead of only with an oracle that runs beside them.

The reference tree is only needed for ``ref_pins.npz``.
"""
from __future__ import annotations

import logging
import os
import sys

import numpy as np
import torch
import torch.nn as nn

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import oracle_gptq as O  # noqa: E402
from oracle import ref_shim  # noqa: E402


def make_ref_pins(path: str) -> None:
    logging.disable(logging.CRITICAL)
    G = ref_shim.load_gptq()
    D = ref_shim.load_dequantizer()
    L = ref_shim.load_layers()
    out = {}
    gen = torch.Generator().manual_seed(1234)
    cpu = torch.device("cpu")

    # --- GPTQ.add_batch: 3-D and 2-D inputs (core/gptq.py:63-89)
    K, N = 24, 16
    lin = nn.Linear(K, N, bias=False)
    q = G.GPTQ(lin, bits=4, group_size=8, blocksize=8, device=cpu)
    x3 = torch.randn(3, 10, K, generator=gen)
    x2 = torch.randn(7, K, generator=gen)
    q.add_batch(x3, None)
    out["ab_x3"], out["ab_H1"], out["ab_n1"] = x3.numpy(), q.H.clone().numpy(), np.int64(q.nsamples)
    q.add_batch(x2, None)
    out["ab_x2"], out["ab_H2"], out["ab_n2"] = x2.numpy(), q.H.clone().numpy(), np.int64(q.nsamples)
    # bf16 activations are upcast before the product (core/gptq.py:88)
    lin = nn.Linear(K, N, bias=False)
    q = G.GPTQ(lin, device=cpu)
    xb = torch.randn(2, 12, K, generator=gen).bfloat16()
    q.add_batch(xb, None)
    out["ab_xb"], out["ab_Hb"] = xb.float().numpy(), q.H.clone().numpy()

    # --- tripwire: GPTQ.quantize raises (core/gptq.py:175-176)
    raised = []
    for (i, o) in ((64, 64), (64, 128), (128, 64)):
        lin = nn.Linear(i, o, bias=False)
        q = G.GPTQ(lin, bits=4, group_size=16, blocksize=32, device=cpu)
        q.add_batch(torch.randn(2, 32, i, generator=gen), None)
        try:
            q.quantize()
            raised.append(0)
        except RuntimeError:
            raised.append(1)
    out["quantize_raises"] = np.array(raised, dtype=np.int64)

    # --- GPTQ.pack_weights on hand-set integer codes, format F1 (core/gptq.py:216-266).
    # pack_weights transposes an nn.Linear weight, so a square layer holding codes.t()
    # packs `codes` itself.
    n = 16
    for bits in (2, 3, 4, 8):
        codes = torch.randint(0, 2 ** bits, (n, n), generator=gen)
        lin = nn.Linear(n, n, bias=False)
        lin.weight.data = codes.t().float().contiguous()
        q = G.GPTQ(lin, bits=bits, device=cpu)
        p = q.pack_weights()["packed_weights"]
        out[f"f1_codes_{bits}"] = codes.numpy().astype(np.uint8)
        out[f"f1_packed_{bits}"] = p.numpy()

    # --- QuantizedLinear pack/unpack, format F2 and groupwise dequant (models/layers.py:67-138)
    for tag, (rows, cols, g) in {"even": (6, 32, 8), "odd": (5, 27, 8)}.items():
        for bits in (4, 8, 3):
            codes = torch.randint(0, 2 ** bits, (rows, cols), generator=gen).to(torch.uint8)
            ng = -(-cols // g)
            scales = (torch.rand(rows, ng, generator=gen) * 0.1 + 0.01).half()
            zeros = torch.randint(0, 2 ** bits, (rows, ng), generator=gen).half()
            ql = L.QuantizedLinear(bits=bits, group_size=g, in_features=cols, out_features=rows, bias=False)
            ql.pack_weights(codes, scales, zeros)
            out[f"f2_{tag}_codes_{bits}"] = codes.numpy()
            out[f"f2_{tag}_scales_{bits}"] = scales.numpy()
            out[f"f2_{tag}_zeros_{bits}"] = zeros.numpy()
            out[f"f2_{tag}_qweight_{bits}"] = ql.qweight.numpy()
            out[f"f2_{tag}_deq_{bits}"] = ql.unpack_weights().numpy()
            if bits == 4 and cols % 2 == 0:
                out[f"f2_{tag}_unpack4"] = D.GPTQDequantizer(4, g)._unpack_4bit(ql.qweight).numpy()
    out["f2_group_size"] = np.int64(8)

    # --- the reference's scalar expressions on fixed inputs (core/gptq.py:165-169,175,179)
    for bits in (2, 3, 4, 8):
        maxq = 2 ** bits - 1
        w_group = torch.randn(32, 16, generator=gen) * 0.02
        w_max = w_group.max(dim=1, keepdim=True)[0]
        w_min = w_group.min(dim=1, keepdim=True)[0]
        scale = (w_max - w_min).squeeze() / maxq
        zero = torch.round(-w_min.squeeze() / scale)
        w = w_group[:, 3]
        qq = torch.clamp(torch.round(w / scale + zero), 0, maxq)
        w_hat = (qq - zero) * scale
        out[f"sf_wgroup_{bits}"] = w_group.numpy()
        out[f"sf_scale_{bits}"] = scale.numpy()
        out[f"sf_zero_{bits}"] = zero.numpy()
        out[f"sf_q_{bits}"] = qq.numpy()
        out[f"sf_what_{bits}"] = w_hat.numpy()
    np.savez_compressed(path, **out)
    print("wrote", path, f"{os.path.getsize(path)} bytes")


ORACLE_CASES = {
    # name: (N_out, K, T, bits, group_size, blocksize, actorder)
    "b4_g32": (24, 96, 256, 4, 32, 32, False),
    "b4_g32_act": (24, 96, 256, 4, 32, 32, True),
    "b3_g128": (40, 256, 512, 3, 128, 128, False),
    "b2_g64_act": (33, 256, 512, 2, 64, 128, True),
    "b8_perchannel": (17, 192, 384, 8, -1, 128, False),
    "b4_g128_ragged": (19, 320, 640, 4, 128, 128, True),
}


def synth_layer(N_out: int, K: int, T: int, seed: int):
    """Weights ~N(0, 0.02); activations ~N(0,1) with 1 % of channels (at least one)
    scaled by 20, rounded to bf16 - the value distributions of the layer-sweep
    workload."""
    gen = torch.Generator().manual_seed(seed)
    W = torch.randn(N_out, K, generator=gen) * 0.02
    X = torch.randn(T, K, generator=gen)
    n_out = max(1, -(-K // 100))
    idx = torch.randperm(K, generator=gen)[:n_out]
    X[:, idx] *= 20
    return W, X.bfloat16().float()


def make_oracle_cases(path: str) -> None:
    out = {}
    for i, (name, (N_out, K, T, bits, g, B, act)) in enumerate(ORACLE_CASES.items()):
        W, X = synth_layer(N_out, K, T, 100 + i)
        nseq = 4
        H = X.t() @ X
        r = O.gptq_quantize(W, H, nseq, bits=bits, group_size=g, blocksize=B, percdamp=0.01, actorder=act)
        out[f"{name}_W"] = W.numpy()
        out[f"{name}_H"] = H.numpy()
        out[f"{name}_cfg"] = np.array([N_out, K, T, bits, g, B, int(act), nseq], dtype=np.int64)
        out[f"{name}_codes"] = r["codes"].numpy()
        out[f"{name}_scale"] = r["scale"].numpy()
        out[f"{name}_zero"] = r["zero"].numpy()
        out[f"{name}_g_idx"] = r["g_idx"].numpy()
        out[f"{name}_Q"] = r["Q"].numpy()
        out[f"{name}_U"] = r["U"].numpy()
        out[f"{name}_total_error"] = np.float64(r["total_error"])
        out[f"{name}_recon"] = np.float64(O.recon_error(W, r["Q"], H))
    np.savez_compressed(path, **out)
    print("wrote", path, f"{os.path.getsize(path)} bytes")


if __name__ == "__main__":
    torch.manual_seed(0)
    torch.set_num_threads(1)
    if ref_shim.available():
        make_ref_pins(os.path.join(HERE, "ref_pins.npz"))
    else:
        print("reference tree not found: ref_pins.npz left as is")
    make_oracle_cases(os.path.join(HERE, "oracle_cases.npz"))
