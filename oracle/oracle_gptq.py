"""CPU oracle for the GPTQ quantization path.  TEST INFRASTRUCTURE ONLY.

This file restates, on the CPU (torch fp32/fp64, vectorised over weight rows with
one Python loop over columns), the algorithm that the reference implements in
``src/distributed_gptq/core/gptq.py`` and the storage formats of
``src/distributed_gptq/models/layers.py`` / ``core/dequantizer.py`` /
``kernels/triton_kernels.py``.  Only the tests, the smoke check and the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark may import it; the
product package never does.

Pinning status
--------------
* ``hessian_add_batch``  - pinned against the reference's own runnable
  ``GPTQ.add_batch`` (golden vectors ``tests/golden/ref_pins.npz``).
* ``pack_f1``            - pinned against the reference's ``GPTQ.pack_weights``.
* ``pack_f2`` / ``unpack_f2`` / ``dequant`` - pinned against the reference's
  ``QuantizedLinear.pack_weights`` / ``unpack_weights`` and
  ``GPTQDequantizer._unpack_4bit``.
* ``gptq_quantize``      - **parity unpinned**: the reference's ``GPTQ.quantize``
  raises on every input (``core/gptq.py:175-176``) and its tests hold no golden
  vectors, so the column loop follows ``core/gptq.py:91-214`` with the defect
  fixes listed in the function's docstring.  ``find_params`` and
  ``quantize_column`` are pinned by re-evaluating the reference's expressions
  (``core/gptq.py:165-169,175,179``) on the same inputs.
* ``pack_f3``            - parity unpinned: the reference kernel
  (``kernels/triton_kernels.py:186-222``) is never launched.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch

FORMAT_F1 = 1  # bytes, first code in the high bits  (core/gptq.py:229-257)
FORMAT_F2 = 2  # bytes, first code in the low nibble (models/layers.py:76-93)
FORMAT_F3 = 3  # int32 words, first code in the low bits (kernels/triton_kernels.py:203-222)


# --------------------------------------------------------------------------- Hessian
def hessian_add_batch(H: Optional[torch.Tensor], nsamples: int, inp: torch.Tensor
                      ) -> Tuple[torch.Tensor, int]:
    """``H += XᵀX`` in fp32 and ``nsamples += batch`` (core/gptq.py:63-89).

    A 2-D input counts as one sample (``:71-72``); a 3-D ``(b, s, K)`` input adds
    ``b`` and is flattened to ``(b*s, K)`` (``:74-79``).
    """
    if inp.dim() == 2:
        inp = inp.unsqueeze(0)
    batch = inp.shape[0]
    x = inp.reshape(-1, inp.shape[-1]).float()
    if H is None:
        H = torch.zeros((x.shape[1], x.shape[1]), dtype=torch.float32)
    H += x.t() @ x
    return H, nsamples + batch


# --------------------------------------------------------------------------- scalar formulas
def find_params(w_group: torch.Tensor, maxq: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row ``scale = (max-min)/maxq``, ``zero = round(-min/scale)``
    (core/gptq.py:165-169).  A constant row (max == min) takes scale 1, which the
    reference leaves undefined (division by zero)."""
    mx = w_group.max(dim=1)[0]
    mn = w_group.min(dim=1)[0]
    scale = (mx - mn) / maxq
    scale = torch.where(scale == 0, torch.ones_like(scale), scale)
    zero = torch.round(-mn / scale)
    return scale, zero


def quantize_column(w: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor, maxq: int
                    ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``q = clamp(round(w/scale + zero), 0, maxq)``; ``w_hat = (q - zero)*scale``
    (core/gptq.py:175,179).  ``round`` is half-to-even."""
    q = torch.clamp(torch.round(w / scale + zero), 0, maxq)
    return q, (q - zero) * scale


# --------------------------------------------------------------------------- inverse chain
def damped_inv_chol(H: torch.Tensor, percdamp: float) -> torch.Tensor:
    """Damp (core/gptq.py:116-119), then Cholesky -> inverse (``:122``) -> upper
    Cholesky, returning ``U`` with ``H⁻¹ = UᵀU``."""
    H = H.clone()
    d = torch.diagonal(H)
    d += percdamp * d.mean()
    L = torch.linalg.cholesky(H)
    Hinv = torch.cholesky_inverse(L)
    return torch.linalg.cholesky(Hinv, upper=True)


def n_groups(K: int, group_size: int) -> int:
    return 1 if group_size <= 0 or group_size >= K else math.ceil(K / group_size)


# --------------------------------------------------------------------------- the column loop
def gptq_quantize(W: torch.Tensor, H_raw: torch.Tensor, nsamples: int, bits: int = 4,
                  group_size: int = 128, blocksize: int = 128, percdamp: float = 0.01,
                  actorder: bool = False, dtype: torch.dtype = torch.float32
                  ) -> Dict[str, object]:
    """GPTQ of one ``(N_out, K)`` weight matrix given the raw Hessian sum.

    Follows ``core/gptq.py:91-214`` with these decisions where the reference is
    broken or silent:

    * ``W`` stays ``(out, in)`` so columns are input features and match ``H``
      (the reference transposes, ``:107-108``, which is dimensionally
      inconsistent for non-square layers).
    * ``H = (2/n)·H_raw`` (the reference divides by ``n`` only, ``:113``; the
      codes do not depend on this scalar because damping is relative).
    * dead columns (``H_ii == 0``): ``H_ii = 1``, ``W[:, i] = 0``.
    * act-order: stable descending sort of ``diag(H)`` (``actorder`` is stored but
      never used by the reference, ``:49``).
    * per column ``d = U[c, c]`` and the row ``U[c, c+1:]`` of the upper Cholesky
      factor of ``H⁻¹`` replace the stale ``H_inv`` rows of ``:142,153,187``.
    * the column's scale/zero are ``(rows,)`` vectors (the reference's
      ``(rows, 1)`` shape is what makes ``:175-176`` raise).
    * group parameters are taken from the outer matrix ``W[:, c:c+g]`` (``:162``),
      i.e. with every earlier block's trailing update and none of the current
      block's in-block updates.
    * after each block ``W[:, i2:] -= Err · U[i1:i2, i2:]`` (``Err`` is filled at
      ``:190`` but never applied by the reference).
    * ``total_error = Σ ((w - w_hat)/d)²`` as at ``:183,191``.
    """
    W = W.detach().to(dtype).clone()
    N_out, K = W.shape
    maxq = 2 ** bits - 1
    H = H_raw.detach().to(dtype) * (2.0 / nsamples)
    dead = torch.diagonal(H) == 0
    H[dead, dead] = 1
    W[:, dead] = 0
    perm = None
    if actorder:
        perm = torch.argsort(torch.diagonal(H), descending=True, stable=True)
        W = W[:, perm]
        H = H[perm][:, perm]
    U = damped_inv_chol(H, percdamp)

    per_channel = group_size <= 0 or group_size >= K
    g = K if per_channel else group_size
    ng = n_groups(K, group_size)
    scale = torch.zeros((N_out, ng), dtype=dtype)
    zero = torch.zeros((N_out, ng), dtype=dtype)
    codes = torch.zeros((N_out, K), dtype=torch.uint8)
    Q = torch.zeros_like(W)
    total_error = 0.0

    for i1 in range(0, K, blocksize):
        i2 = min(i1 + blocksize, K)
        W1 = W[:, i1:i2].clone()
        Err = torch.zeros_like(W1)
        for j in range(i2 - i1):
            c = i1 + j
            if c % g == 0:
                s, z = find_params(W[:, c:min(c + g, K)], maxq)
                scale[:, c // g] = s
                zero[:, c // g] = z
            s = scale[:, c // g]
            z = zero[:, c // g]
            w = W1[:, j]
            q, w_hat = quantize_column(w, s, z, maxq)
            d = U[c, c]
            e = (w - w_hat) / d
            if j < i2 - i1 - 1:
                W1[:, j + 1:] -= e.unsqueeze(1) * U[c, c + 1:i2].unsqueeze(0)
            Err[:, j] = e
            total_error += float((e.double() ** 2).sum())
            codes[:, c] = q.to(torch.uint8)
            Q[:, c] = w_hat
        if i2 < K:
            W[:, i2:] -= Err @ U[i1:i2, i2:]

    g_idx = torch.arange(K, dtype=torch.int32) // g
    if actorder:
        invperm = torch.argsort(perm)
        Q = Q[:, invperm]
        codes = codes[:, invperm]
        g_idx = torch.empty(K, dtype=torch.int32)
        g_idx[perm] = (torch.arange(K, dtype=torch.int32) // g)
    return {
        "codes": codes, "scale": scale, "zero": zero, "g_idx": g_idx, "Q": Q,
        "perm": perm, "U": U, "total_error": total_error,
        "stats": {"bits": bits, "group_size": group_size, "total_error": total_error,
                  "compression_ratio": 32.0 / bits,
                  "scale_shape": tuple(scale.shape), "zero_shape": tuple(zero.shape)},
    }


def recon_error(W0: torch.Tensor, Q: torch.Tensor, H_raw: torch.Tensor) -> float:
    """``‖W X − Q X‖² = tr((W−Q) H_raw (W−Q)ᵀ)`` in fp64."""
    D = (W0.double() - Q.double())
    return float(((D @ H_raw.double()) * D).sum())


# --------------------------------------------------------------------------- storage formats
def pack_f1(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """Byte packing of ``GPTQ.pack_weights`` (core/gptq.py:229-257): 4-bit
    ``c[i]*16 + c[i+1]``; 2-bit ``c0*64 + c1*16 + c2*4 + c3``; 3-bit one code per
    uint8; 8-bit reinterpreted as int8."""
    c = codes.to(torch.int32)
    if bits == 4:
        return (c[:, 0::2] * 16 + c[:, 1::2]).to(torch.uint8)
    if bits == 2:
        return (c[:, 0::4] * 64 + c[:, 1::4] * 16 + c[:, 2::4] * 4 + c[:, 3::4]).to(torch.uint8)
    if bits == 8:
        return codes.to(torch.uint8).view(torch.int8)
    return codes.to(torch.uint8)


def unpack_f1(packed: torch.Tensor, bits: int, cols: int) -> torch.Tensor:
    p = packed.view(torch.uint8).to(torch.int32)
    if bits == 4:
        out = torch.stack([(p >> 4) & 15, p & 15], dim=2).reshape(p.shape[0], -1)
    elif bits == 2:
        out = torch.stack([(p >> 6) & 3, (p >> 4) & 3, (p >> 2) & 3, p & 3], dim=2
                          ).reshape(p.shape[0], -1)
    else:
        out = p
    return out[:, :cols].to(torch.uint8)


def pack_f2(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """``QuantizedLinear.pack_weights`` (models/layers.py:76-93): 4-bit
    ``c[i] | c[i+1] << 4`` with an odd tail column alone in the low nibble; every
    other width keeps one code per uint8."""
    if bits != 4:
        return codes.to(torch.uint8).clone()
    c = codes.to(torch.int32)
    rows, cols = c.shape
    if cols % 2:
        c = torch.cat([c, torch.zeros((rows, 1), dtype=torch.int32)], dim=1)
    return (c[:, 0::2] | (c[:, 1::2] << 4)).to(torch.uint8)


def unpack_f2(packed: torch.Tensor, bits: int, cols: int) -> torch.Tensor:
    """models/layers.py:105-120 and core/dequantizer.py:79-89."""
    if bits != 4:
        return packed.to(torch.uint8)[:, :cols]
    p = packed.to(torch.int32)
    out = torch.stack([p & 15, (p >> 4) & 15], dim=2).reshape(p.shape[0], -1)
    return out[:, :cols].to(torch.uint8)


def codes_per_word(bits: int) -> int:
    return 32 // bits


def pack_f3(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """int32 words, ``word |= code_j << (j*bits)`` for ``j < 32 // bits``
    (kernels/triton_kernels.py:203-222); 3-bit leaves the top two bits zero."""
    per = codes_per_word(bits)
    rows, cols = codes.shape
    nw = math.ceil(cols / per)
    c = torch.zeros((rows, nw * per), dtype=torch.int64)
    c[:, :cols] = codes.to(torch.int64)
    c = c.reshape(rows, nw, per)
    shifts = (torch.arange(per, dtype=torch.int64) * bits).view(1, 1, per)
    w = (c << shifts).sum(dim=2)
    w = torch.where(w >= 2 ** 31, w - 2 ** 32, w)
    return w.to(torch.int32)


def unpack_f3(packed: torch.Tensor, bits: int, cols: int) -> torch.Tensor:
    per = codes_per_word(bits)
    w = packed.to(torch.int64) & 0xFFFFFFFF
    shifts = (torch.arange(per, dtype=torch.int64) * bits).view(1, 1, per)
    c = (w.unsqueeze(2) >> shifts) & (2 ** bits - 1)
    return c.reshape(w.shape[0], -1)[:, :cols].to(torch.uint8)


def pack(codes: torch.Tensor, bits: int, fmt: int) -> torch.Tensor:
    return {FORMAT_F1: pack_f1, FORMAT_F2: pack_f2, FORMAT_F3: pack_f3}[fmt](codes, bits)


def unpack(packed: torch.Tensor, bits: int, cols: int, fmt: int) -> torch.Tensor:
    return {FORMAT_F1: unpack_f1, FORMAT_F2: unpack_f2, FORMAT_F3: unpack_f3}[fmt](packed, bits, cols)


def dequant(codes: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor,
            g_idx: Optional[torch.Tensor] = None, group_size: int = 128) -> torch.Tensor:
    """``(code − zero[r, g(c)])·scale[r, g(c)]`` in fp32 (models/layers.py:122-136).
    ``g(c)`` is ``g_idx[c]`` when given, else ``c // group_size``."""
    K = codes.shape[1]
    if g_idx is None:
        g = K if group_size <= 0 or group_size >= K else group_size
        g_idx = torch.arange(K) // g
    gi = g_idx.long()
    return (codes.float() - zero.float()[:, gi]) * scale.float()[:, gi]


def qlinear_forward(x: torch.Tensor, codes: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor,
                    g_idx: Optional[torch.Tensor], bias: Optional[torch.Tensor],
                    group_size: int = 128) -> torch.Tensor:
    """``QuantizedLinear.forward`` through its dequantize + ``F.linear`` branch
    (models/layers.py:155-157), evaluated in fp32."""
    w = dequant(codes, scale, zero, g_idx, group_size)
    y = x.float() @ w.t()
    if bias is not None:
        y = y + bias.float()
    return y


# --------------------------------------------------------------------------- RTN helpers
def rtn_quantize(x: torch.Tensor, bits: int, group_size: int
                 ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Flat round-to-nearest of ``kernels/triton_kernels.py:377-433``: groups of
    ``group_size`` consecutive elements of the flattened tensor;
    ``scale = (max-min)/maxq``, ``zero = -min/scale`` (unrounded, ``:411``);
    ``q = clamp(round(x/scale + zero), 0, maxq)`` (``:72-73``).  Constant groups
    take scale 1."""
    maxq = 2 ** bits - 1
    flat = x.detach().float().flatten()
    n = flat.numel()
    ng = math.ceil(n / group_size)
    pad = ng * group_size - n
    fp = torch.cat([flat, flat[-1:].expand(pad)]) if pad else flat
    grp = fp.view(ng, group_size)
    mx = grp.max(dim=1)[0]
    mn = grp.min(dim=1)[0]
    scale = (mx - mn) / maxq
    scale = torch.where(scale == 0, torch.ones_like(scale), scale)
    zero = -mn / scale
    q = torch.clamp(torch.round(grp / scale[:, None] + zero[:, None]), 0, maxq)
    q = q.flatten()[:n].to(torch.uint8).reshape(x.shape)
    return q, scale, zero


def rtn_dequantize(q: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor, group_size: int
                   ) -> torch.Tensor:
    """``(q − zero[g])·scale[g]`` with ``g = offset // group_size``
    (kernels/triton_kernels.py:82-123)."""
    flat = q.flatten().float()
    gi = torch.arange(flat.numel()) // group_size
    return ((flat - zero[gi]) * scale[gi]).reshape(q.shape)
