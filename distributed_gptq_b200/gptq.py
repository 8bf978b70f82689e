"""Layer-level GPTQ: the ``GPTQ`` and ``Quantizer`` classes.

Mirrors ``src/distributed_gptq/core/gptq.py`` of the reference (constructor
arguments, ``add_batch`` / ``quantize`` / ``pack_weights``, the ``H`` / ``nsamples`` /
``scale`` / ``zero`` / ``maxq`` attributes and the keys of the returned stats), with
every computation done by the sm_100a kernels behind ``libdgq.so``.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
import torch.nn as nn

from . import _C


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class Quantizer:
    """Scale/zero search and round-to-nearest on their own.

    ``find_params`` evaluates ``scale = (max-min)/maxq``, ``zero = round(-min/scale)``
    per row (reference ``core/gptq.py:165-169``); ``quantize`` evaluates
    ``clamp(round(x/scale + zero), 0, maxq)`` and returns the dequantized values
    ``(q - zero)*scale`` (``core/gptq.py:175,179``).  The integer levels of the last
    call are kept in ``codes``.
    """

    def __init__(self, bits: int = 4):
        self.configure(bits)
        self.scale: Optional[torch.Tensor] = None
        self.zero: Optional[torch.Tensor] = None
        self.codes: Optional[torch.Tensor] = None

    def configure(self, bits: int, **_unused) -> None:
        if bits not in (2, 3, 4, 8):
            raise ValueError(f"bits must be 2, 3, 4 or 8, got {bits}")
        self.bits = bits
        self.maxq = 2 ** bits - 1

    def find_params(self, x: torch.Tensor, weight: bool = True) -> None:
        x2 = x.reshape(x.shape[0], -1) if weight else x.reshape(1, -1)
        self.scale, self.zero = _C.find_params(x2.float().contiguous(), self.bits)

    def quantize(self, x: torch.Tensor) -> torch.Tensor:
        if not self.ready():
            raise RuntimeError("call find_params first")
        x2 = x.reshape(self.scale.numel(), -1).float().contiguous()
        self.codes, xh = _C.quantize_rows(x2, self.scale, self.zero, self.bits)
        self.codes = self.codes.reshape(x.shape)
        return xh.reshape(x.shape).to(x.dtype)

    def ready(self) -> bool:
        return self.scale is not None


class GPTQ:
    """GPTQ of one ``nn.Linear`` / ``nn.Conv2d`` (reference ``core/gptq.py:16-266``).

    ``H`` holds the raw sum ``Σ XᵀX`` in fp32 like the reference's attribute;
    normalisation, damping, act-order and the inverse factor are applied to a copy
    inside :meth:`quantize`.
    """

    def __init__(self, layer: nn.Module, bits: int = 4, group_size: int = 128,
                 actorder: bool = False, percdamp: float = 0.01, blocksize: int = 128,
                 device: Optional[torch.device] = None):
        self.layer = layer
        self.bits = bits
        self.group_size = group_size
        self.actorder = actorder
        self.percdamp = percdamp
        self.blocksize = blocksize
        if device is None:
            device = layer.weight.device if layer.weight.is_cuda else torch.device("cuda")
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("distributed_gptq_b200 has no CPU path: GPTQ needs a CUDA device")
        self.maxq = 2 ** bits - 1
        self.scale: Optional[torch.Tensor] = None
        self.zero: Optional[torch.Tensor] = None
        self.codes: Optional[torch.Tensor] = None
        self.g_idx: Optional[torch.Tensor] = None
        self.perm: Optional[torch.Tensor] = None
        self._Hbuf: Optional[torch.Tensor] = None
        self.nsamples = 0
        self.columns = self._weight_matrix().shape[1]
        self._info = None
        self._pending = None
        # add_batch updates only the part of the Hessian on and above the diagonal (half the
        # reduction traffic of every batch); the lower part is filled in when the matrix is
        # read: by the `H` property and before quantization
        self._lower_stale = False
        # set by a driver that lends this object a Hessian buffer other ranks' kernels
        # accumulate into as well: the buffer is zeroed as soon as quantization has read it
        self._recycle = False

    # ------------------------------------------------------------------ helpers
    def _weight_matrix(self) -> torch.Tensor:
        W = self.layer.weight.data
        if isinstance(self.layer, nn.Conv2d):
            W = W.flatten(1)
        return W

    @property
    def H(self) -> Optional[torch.Tensor]:
        if self._Hbuf is None:
            return None
        self._complete_hessian()
        return self._Hbuf[:self.columns, :self.columns]

    def _complete_hessian(self) -> None:
        if self._lower_stale and self._Hbuf is not None:
            _C.hessian_mirror(self._Hbuf)
            self._lower_stale = False

    @H.setter
    def H(self, value: Optional[torch.Tensor]) -> None:
        if value is None:
            self._Hbuf = None
            return
        K = self.columns
        assert value.shape == (K, K)
        K8 = _round_up(K, 8)
        buf = torch.zeros((K8, K8), dtype=torch.float32, device=self.device)
        buf[:K, :K] = value.to(self.device, torch.float32)
        self._Hbuf = buf
        self._lower_stale = False

    def _tokens(self, inp: torch.Tensor) -> torch.Tensor:
        """Flattens a batch to ``(tokens, columns)`` the way the layer consumes it."""
        if isinstance(self.layer, nn.Conv2d):
            unfold = nn.Unfold(self.layer.kernel_size, dilation=self.layer.dilation,
                               padding=self.layer.padding, stride=self.layer.stride)
            x = unfold(inp)                      # (b, C*kh*kw, L)
            return x.permute(0, 2, 1).reshape(-1, x.shape[1])
        return inp.reshape(-1, inp.shape[-1])

    # ------------------------------------------------------------------ Hessian
    def add_batch(self, inp: torch.Tensor, out: Optional[torch.Tensor] = None) -> None:
        """``H += XᵀX``; ``nsamples += batch`` (reference ``core/gptq.py:63-89``).

        A 2-D input counts as one sample.  ``out`` is accepted and ignored, as in the
        reference.  Activations are taken in bf16 (fp32/fp16 inputs are rounded to
        bf16 first) and accumulated in fp32 on the tensor cores.
        """
        if inp.dim() == 2 and not isinstance(self.layer, nn.Conv2d):
            inp = inp.unsqueeze(0)
        batch = inp.shape[0]
        x = self._tokens(inp.to(self.device, non_blocking=True))
        K = self.columns
        assert x.shape[1] == K, f"expected {K} input features, got {x.shape[1]}"
        K8 = _round_up(K, 8)
        if self._Hbuf is None:
            self._Hbuf = torch.zeros((K8, K8), dtype=torch.float32, device=self.device)
            self._info = _C.new_info(self.device)
        if K8 != K:
            xp = torch.zeros((x.shape[0], K8), dtype=x.dtype, device=self.device)
            xp[:, :K] = x
            x = xp
        xb = _C.to_bf16(x)
        self.nsamples += batch
        if xb.shape[0] > 0:
            _C.hessian_accum(xb, self._Hbuf, 1.0, 0, self._info, upper_only=True)
            self._lower_stale = True

    # ------------------------------------------------------------------ quantize
    def quantize(self) -> Dict[str, Any]:
        """Blockwise GPTQ of the layer's weight (reference ``core/gptq.py:91-214``).

        Writes the dequantized weights back into ``layer.weight`` in its dtype and
        keeps ``codes`` (uint8, ``(out, in)``), ``scale`` / ``zero`` (fp32,
        ``(out, n_groups)``) and ``g_idx`` (int32 group of every input column) on the
        object.  Returns the reference's stats keys plus timings-free extras.
        """
        self.quantize_launch()
        return self.quantize_finish()

    def quantize_launch(self) -> None:
        """First half of :meth:`quantize`: enqueues every kernel of the quantization on the
        current CUDA stream and returns without waiting for the device, so that a caller can
        put the chains of independent layers on different streams (see ``streams.ChainPool``)
        or keep accumulating other Hessians meanwhile.  :meth:`quantize_finish` must follow."""
        quantize_group_launch([self])

    def quantize_finish(self) -> Dict[str, Any]:
        """Second half of :meth:`quantize`: waits for the chain, raises if the Hessian
        accumulation or the damped inverse reported a failure (the layer's weight is then put
        back as it was) and returns the stats."""
        pend = getattr(self, "_pending", None)
        if pend is None:
            raise RuntimeError("call quantize_launch before quantize_finish")
        self._pending = None
        pend["done"].synchronize()
        cur = torch.cuda.current_stream(self.device)
        cur.wait_event(pend["done"])
        for t in (self.codes, self.scale, self.zero, self.g_idx, self.layer.weight.data):
            if t is not None and t.is_cuda:
                t.record_stream(cur)
        status = pend["status"]
        try:
            if status["hessian_info"] is not None:
                _C.raise_on_info(status["hessian_info"], "hessian accumulation")
            _C.raise_on_info(status["info"], "damped inverse")
        except Exception:
            self.layer.weight.data = pend["old_weight"]
            self.codes = self.scale = self.zero = self.g_idx = self.perm = None
            raise
        total_error = float(status["terr"][pend["slot"]].item())
        return {
            "bits": self.bits,
            "group_size": self.group_size,
            "total_error": total_error,
            "compression_ratio": 32.0 / self.bits,
            "scale_shape": self.scale.shape,
            "zero_shape": self.zero.shape,
        }

    def fasterquant(self, blocksize: Optional[int] = None, percdamp: Optional[float] = None,
                    group_size: Optional[int] = None, groupsize: Optional[int] = None,
                    actorder: Optional[bool] = None) -> Dict[str, Any]:
        """Same work as :meth:`quantize`; arguments override the constructor's values."""
        if blocksize is not None:
            self.blocksize = blocksize
        if percdamp is not None:
            self.percdamp = percdamp
        if group_size is None:
            group_size = groupsize
        if group_size is not None:
            self.group_size = group_size
        if actorder is not None:
            self.actorder = actorder
        return self.quantize()

    # ------------------------------------------------------------------ packing
    def pack_weights(self, format: int = _C.FMT_BYTES_HI_FIRST) -> Dict[str, Any]:
        """Packed codes and parameters (reference ``core/gptq.py:216-266``).

        The default format is the reference's byte packing of this method (first
        code in the high bits); pass ``_C.FMT_BYTES_LO_FIRST`` for the
        ``QuantizedLinear`` layout or ``_C.FMT_INT32_LE`` for 32-bit words.
        """
        if self.codes is None:
            raise RuntimeError("call quantize before pack_weights")
        return {
            "packed_weights": _C.pack(self.codes, self.bits, format),
            "scale": self.scale,
            "zero": self.zero,
            "g_idx": self.g_idx,
            "bits": self.bits,
            "group_size": self.group_size,
            "shape": self.codes.shape,
        }

    def free_hessian(self) -> None:
        """Drops the Hessian buffer (its memory returns to torch's caching allocator)."""
        self._Hbuf = None
        self._info = None

    def free(self) -> None:
        self.free_hessian()
        torch.cuda.empty_cache()


def quantize_group_launch(members: List["GPTQ"]) -> Dict[str, torch.Tensor]:
    """Enqueues the quantization of several layers that read the same input tensor (q/k/v or
    gate/up of a decoder block) as one chain on the current stream.

    ``members[0]`` holds the Hessian.  The Hessian fixes the column order, the damped inverse
    factor ``U`` and nothing else, and the rows of a weight matrix are quantized independently
    given ``U`` (reference ``core/gptq.py:131-194`` has no term that couples rows), so the
    members' weights are stacked into one ``(sum N_out, K)`` matrix: one preparation, one
    inverse factor and one pass of the block loop serve all of them, with results equal to
    quantizing each layer by itself.  Every member ends in the state
    :meth:`GPTQ.quantize_launch` leaves it in; :meth:`GPTQ.quantize_finish` must follow for
    each.  Returns device tensors a caller may ship before the host has seen them:
    ``info`` / ``hessian_info`` (2 x int32 status words) and ``terr`` (one double per
    member)."""
    lead = members[0]
    if lead._Hbuf is None or lead.nsamples == 0:
        raise RuntimeError("no calibration data: call add_batch before quantize")
    dev = lead.device
    K = lead.columns
    for m in members[1:]:
        if (m.columns, m.bits, m.group_size, m.actorder, m.percdamp, m.blocksize, m.device) != \
                (K, lead.bits, lead.group_size, lead.actorder, lead.percdamp, lead.blocksize, dev):
            raise ValueError("layers quantized as one group must agree in input width and settings")
    cur = torch.cuda.current_stream(dev)
    # the inputs may have been produced on another stream than the one this chain runs on
    lead._Hbuf.record_stream(cur)
    # the accumulation (and a reduction over ranks) only kept the upper triangle up to date
    _C.hessian_mirror(lead._Hbuf)
    lead._lower_stale = False
    parts, bounds, r = [], [], 0
    for m in members:
        Wm = m._weight_matrix()
        if Wm.is_cuda:
            Wm.record_stream(cur)
        parts.append(Wm.to(dev, torch.float32))
        bounds.append((r, r + Wm.shape[0]))
        r += Wm.shape[0]
    W = torch.cat(parts) if len(parts) > 1 else parts[0].contiguous().clone()
    del parts
    H = lead.H
    scale = float(torch.tensor(2.0 / lead.nsamples, dtype=torch.float32))

    perm = invperm = None
    if lead.actorder:
        perm, invperm = _C.actorder_perm(H, scale)
    Hp, dead = _C.hessian_prepare(H, scale, lead.percdamp, perm)
    if lead._recycle:           # a lent buffer: hand it back empty
        lead._Hbuf.zero_()
    Wp = _C.permute_cols(W, perm, dead)
    del W
    info = _C.new_info(dev)
    U = _C.inv_chol_upper(Hp, info)
    codes, scales, zeros, rerr = _C.gptq_quantize(Wp, U, lead.bits, lead.group_size,
                                                  lead.blocksize, row_error=True)
    g = K if (lead.group_size <= 0 or lead.group_size >= K) else lead.group_size
    if lead.actorder:
        Q = _C.permute_cols(Wp, invperm)
        codes = _C.permute_cols(codes, invperm)
        g_idx = (invperm // g).to(torch.int32)
    else:
        Q = Wp
        g_idx = (torch.arange(K, device=dev, dtype=torch.int32) // g)
    terr = torch.stack([rerr[a:b].sum() for a, b in bounds])

    # the status words and the error sums travel to pinned host memory on this stream, so that
    # quantize_finish only has to wait for this chain, not for the stream it is called on
    def to_host(t):
        h = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
        h.copy_(t, non_blocking=True)
        return h
    hinfo = lead._info
    status = {"info": to_host(info), "terr": to_host(terr),
              "hessian_info": to_host(hinfo) if hinfo is not None else None}
    for slot, (m, (a, b)) in enumerate(zip(members, bounds)):
        old_weight = m.layer.weight.data
        m.codes, m.scale, m.zero, m.g_idx, m.perm = codes[a:b], scales[a:b], zeros[a:b], g_idx, perm
        m.layer.weight.data = Q[a:b].reshape(m.layer.weight.shape).to(
            device=m.layer.weight.device, dtype=m.layer.weight.dtype)
        m._pending = {"status": status, "old_weight": old_weight, "slot": slot}
    done = torch.cuda.Event()
    done.record(cur)
    for m in members:
        m._pending["done"] = done
    return {"info": info, "hessian_info": hinfo if hinfo is not None else torch.zeros_like(info),
            "terr": terr}


def quantize_layer_gptq(layer: nn.Module, calibration_data, bits: int = 4, group_size: int = 128,
                        **kwargs) -> Dict[str, Any]:
    """One-call helper (reference ``core/gptq.py:383-417``): feeds every batch of
    ``calibration_data`` to ``add_batch`` and quantizes."""
    q = GPTQ(layer, bits=bits, group_size=group_size, **kwargs)
    for batch in calibration_data:
        inp = batch[0] if isinstance(batch, (tuple, list)) else batch
        q.add_batch(inp, None)
    return q.quantize()
