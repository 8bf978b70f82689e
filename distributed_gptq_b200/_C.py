"""ctypes binding of ``libdgq.so`` (declared in ``include/dgq.h``) for torch tensors.

The library is the only compute path of this package: there is no CPU or
eager-PyTorch fallback.  Importing this module loads the library (it loads on
machines without a GPU, so symbols can be inspected); calling any compute wrapper
without a CUDA device raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_double, c_float, c_int32, c_int64, c_void_p
from typing import Optional

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libdgq.so")

FMT_BYTES_HI_FIRST, FMT_BYTES_LO_FIRST, FMT_INT32_LE = 1, 2, 3
F32, F16, BF16 = 0, 1, 2
INFO_OK, INFO_NOT_POSDEF, INFO_WAIT_TIMEOUT = 0, 1, 2

_DTYPE_CODE = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}

_P, _I32, _I64, _F, _D = c_void_p, c_int32, c_int64, c_float, c_double

# name -> (restype, argtypes); mirrors include/dgq.h declaration by declaration
SIGNATURES = {
    "dgq_status_string": (ctypes.c_char_p, [_I32]),
    "dgq_version": (_I32, []),
    "dgq_device_check": (_I32, []),
    "dgq_launch_count": (_I64, []),
    "dgq_hessian_accum": (_I32, [_P, _I64, _I32, _I64, _P, _I64, _F, _I32, _P, _P]),
    "dgq_hessian_accum_upper": (_I32, [_P, _I64, _I32, _I64, _P, _I64, _F, _I32, _P, _P]),
    "dgq_hessian_mirror": (_I32, [_P, _I32, _I64, _P]),
    "dgq_cast_f32_to_bf16": (_I32, [_P, _P, _I64, _P]),
    "dgq_cast_f16_to_bf16": (_I32, [_P, _P, _I64, _P]),
    "dgq_actorder_perm": (_I32, [_P, _I32, _I64, _F, _P, _P, _P]),
    "dgq_hessian_prepare_workspace_bytes": (_I64, [_I32]),
    "dgq_hessian_prepare": (_I32, [_P, _I64, _P, _I64, _I32, _F, _F, _P, _P, _P, _I64, _P]),
    "dgq_permute_cols_f32": (_I32, [_P, _I64, _P, _I64, _I32, _I32, _P, _P, _P]),
    "dgq_permute_cols_u8": (_I32, [_P, _I64, _P, _I64, _I32, _I32, _P, _P]),
    "dgq_permute_cols_u16": (_I32, [_P, _I64, _P, _I64, _I32, _I32, _P, _P]),
    "dgq_inv_chol_workspace_bytes": (_I64, [_I32]),
    "dgq_inv_chol_upper": (_I32, [_P, _I32, _I64, _P, _P, _I64, _P]),
    "dgq_gemm_f32": (_I32, [_P, _I64, _P, _I64, _I32, _P, _I64, _I32, _I32, _I32, _F, _F, _I32, _P, _P]),
    "dgq_gptq_quantize_workspace_bytes": (_I64, [_I32, _I32, _I32]),
    "dgq_gptq_quantize": (_I32, [_P, _I64, _P, _I64, _I32, _I32, _I32, _I32, _I32, _P, _I64,
                                 _P, _P, _P, _P, _I64, _P]),
    "dgq_gptq_quantize_rows": (_I32, [_P, _I64, _P, _I64, _I32, _I32, _I32, _I32, _I32, _P, _I64,
                                      _P, _P, _P, _P, _P, _I64, _P]),
    "dgq_gptq_quantize_noalloc_max_rows": (_I32, []),
    "dgq_gptq_quantize_noalloc": (_I32, [_P, _I64, _P, _I64, _I32, _I32, _I32, _I32, _I32, _P, _I64,
                                         _P, _P, _P, _P]),
    "dgq_find_params": (_I32, [_P, _I64, _I32, _I32, _I32, _P, _P, _P]),
    "dgq_quantize_rows": (_I32, [_P, _I64, _I32, _I32, _I32, _P, _P, _P, _I64, _P, _I64, _P]),
    "dgq_packed_row_bytes": (_I64, [_I32, _I32, _I32]),
    "dgq_pack": (_I32, [_P, _I32, _I32, _I32, _I32, _P, _P]),
    "dgq_unpack": (_I32, [_P, _I32, _I32, _I32, _I32, _P, _P]),
    "dgq_unpack_dequant": (_I32, [_P, _P, _P, _P, _I32, _I32, _I32, _I32, _I32, _I32, _I32, _I32,
                                  _P, _P]),
    "dgq_qlinear_forward": (_I32, [_P, _I32, _I32, _P, _P, _P, _P, _P, _I32, _I32, _I32, _I32,
                                   _I32, _I32, _P, _P]),
    "dgq_rtn_find_params": (_I32, [_P, _I64, _I32, _I32, _P, _P, _P]),
    "dgq_rtn_quantize": (_I32, [_P, _I64, _I32, _I32, _P, _P, _P, _P]),
    "dgq_rtn_dequantize": (_I32, [_P, _I64, _I32, _P, _P, _P, _P]),
}

_lib = None


def lib() -> ctypes.CDLL:
    """Loads ``libdgq.so``; raises (never falls back) when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.isfile(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m distributed_gptq_b200.build` "
                "(needs nvcc); this package has no other compute path")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def status_string(code: int) -> str:
    return lib().dgq_status_string(int(code)).decode()


def check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what}: {status_string(code)} (status {code})")


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("distributed_gptq_b200 computes on CUDA tensors only "
                               "(no CPU fallback exists)")


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


class KernelTimers:
    """Collects CUDA-event pairs around library calls, per call name, on the stream the
    call is enqueued on.  Enable with :func:`set_timers`; read with :meth:`summary`."""

    def __init__(self):
        self.events = []

    def summary(self):
        torch.cuda.synchronize()
        out = {}
        for name, a, b in self.events:
            n, ms = out.get(name, (0, 0.0))
            out[name] = (n + 1, ms + a.elapsed_time(b))
        return out


_timers: Optional[KernelTimers] = None


def set_timers(t: Optional[KernelTimers]) -> None:
    global _timers
    _timers = t


class _timed:
    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        if _timers is not None:
            self.a = torch.cuda.Event(enable_timing=True)
            self.a.record()
        return self

    def __exit__(self, *exc):
        if _timers is not None:
            b = torch.cuda.Event(enable_timing=True)
            b.record()
            _timers.events.append((self.name, self.a, b))
        return False


def launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    return int(lib().dgq_launch_count())


def device_check() -> None:
    check(lib().dgq_device_check(), "dgq_device_check")


def new_info(device) -> torch.Tensor:
    return torch.zeros(2, dtype=torch.int32, device=device)


def raise_on_info(info: torch.Tensor, what: str) -> None:
    """Reads the device status words (synchronises) and raises on a device-side condition."""
    code, detail = info.tolist()
    if code == INFO_NOT_POSDEF:
        raise RuntimeError(f"{what}: matrix is not positive definite (pivot {detail})")
    if code == INFO_WAIT_TIMEOUT:
        raise RuntimeError(f"{what}: a bounded wait inside the kernel ran out (wait {detail})")
    if code != INFO_OK:
        raise RuntimeError(f"{what}: unknown device status {code}")


# --------------------------------------------------------------------------- Hessian
def to_bf16(x: torch.Tensor) -> torch.Tensor:
    """bf16 copy of a float tensor through the library's cast kernels."""
    _require_cuda(x)
    if x.dtype == torch.bfloat16:
        return x.contiguous()
    x = x.contiguous()
    out = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
    if x.numel() == 0:
        return out
    with torch.cuda.device(x.device), _timed("cast"):
        if x.dtype == torch.float32:
            check(lib().dgq_cast_f32_to_bf16(_ptr(x), _ptr(out), x.numel(), _stream()), "cast")
        elif x.dtype == torch.float16:
            check(lib().dgq_cast_f16_to_bf16(_ptr(x), _ptr(out), x.numel(), _stream()), "cast")
        else:
            raise TypeError(f"unsupported activation dtype {x.dtype}")
    return out


def hessian_accum(X: torch.Tensor, H: torch.Tensor, alpha: float = 1.0, splits: int = 0,
                  info: Optional[torch.Tensor] = None, upper_only: bool = False) -> None:
    """``H += alpha * XᵀX`` with X ``(T, K)`` bf16 and H ``(K, K)`` fp32, in place.  With
    ``upper_only`` only the part on and above the diagonal is updated (see
    :func:`hessian_mirror`)."""
    _require_cuda(X, H)
    assert X.dim() == 2 and X.dtype == torch.bfloat16 and X.stride(1) == 1
    assert H.dtype == torch.float32 and H.dim() == 2 and H.stride(1) == 1
    T, K = X.shape
    assert H.shape == (K, K)
    fn = lib().dgq_hessian_accum_upper if upper_only else lib().dgq_hessian_accum
    with torch.cuda.device(X.device), _timed("hessian_accum"):
        check(fn(_ptr(X), T, K, X.stride(0), _ptr(H), H.stride(0), alpha, splits, _ptr(info),
                 _stream()), "dgq_hessian_accum")


def hessian_mirror(H: torch.Tensor) -> None:
    """Copies the part of H above the diagonal to below it, in place."""
    _require_cuda(H)
    assert H.dtype == torch.float32 and H.dim() == 2 and H.stride(1) == 1
    with torch.cuda.device(H.device), _timed("prepare"):
        check(lib().dgq_hessian_mirror(_ptr(H), H.shape[0], H.stride(0), _stream()),
              "dgq_hessian_mirror")


# --------------------------------------------------------------------------- preparation
def actorder_perm(H: torch.Tensor, scale: float):
    _require_cuda(H)
    K = H.shape[0]
    perm = torch.empty(K, dtype=torch.int32, device=H.device)
    inv = torch.empty(K, dtype=torch.int32, device=H.device)
    with torch.cuda.device(H.device), _timed("prepare"):
        check(lib().dgq_actorder_perm(_ptr(H), K, H.stride(0), scale, _ptr(perm), _ptr(inv),
                                      _stream()), "dgq_actorder_perm")
    return perm, inv


def hessian_prepare(H: torch.Tensor, scale: float, percdamp: float,
                    perm: Optional[torch.Tensor] = None):
    """Returns ``(Hout, dead)``: the scaled, permuted, damped copy of H and the dead-column mask."""
    _require_cuda(H)
    K = H.shape[0]
    Hout = torch.empty((K, K), dtype=torch.float32, device=H.device)
    dead = torch.empty(K, dtype=torch.uint8, device=H.device)
    nbytes = lib().dgq_hessian_prepare_workspace_bytes(K)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=H.device)
    with torch.cuda.device(H.device), _timed("prepare"):
        check(lib().dgq_hessian_prepare(_ptr(H), H.stride(0), _ptr(Hout), K, K, scale, percdamp,
                                        _ptr(perm), _ptr(dead), _ptr(ws), nbytes, _stream()),
              "dgq_hessian_prepare")
    return Hout, dead


def permute_cols(src: torch.Tensor, perm: Optional[torch.Tensor],
                 dead: Optional[torch.Tensor] = None) -> torch.Tensor:
    _require_cuda(src)
    assert src.dim() == 2 and src.stride(1) == 1
    rows, cols = src.shape
    dst = torch.empty((rows, cols), dtype=src.dtype, device=src.device)
    with torch.cuda.device(src.device), _timed("permute"):
        if src.dtype == torch.float32:
            check(lib().dgq_permute_cols_f32(_ptr(src), src.stride(0), _ptr(dst), cols, rows, cols,
                                             _ptr(perm), _ptr(dead), _stream()), "permute_cols_f32")
        elif src.dtype == torch.uint8:
            check(lib().dgq_permute_cols_u8(_ptr(src), src.stride(0), _ptr(dst), cols, rows, cols,
                                            _ptr(perm), _stream()), "permute_cols_u8")
        elif src.dtype in (torch.float16, torch.bfloat16):
            check(lib().dgq_permute_cols_u16(_ptr(src), src.stride(0), _ptr(dst), cols, rows, cols,
                                             _ptr(perm), _stream()), "permute_cols_u16")
        else:
            raise TypeError(src.dtype)
    return dst


def inv_chol_upper(A: torch.Tensor, info: Optional[torch.Tensor] = None) -> torch.Tensor:
    """In place: symmetric positive definite A -> upper U with A⁻¹ = UᵀU."""
    _require_cuda(A)
    assert A.dtype == torch.float32 and A.dim() == 2 and A.stride(1) == 1
    K = A.shape[0]
    nbytes = lib().dgq_inv_chol_workspace_bytes(K)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=A.device)
    with torch.cuda.device(A.device), _timed("inv_chol"):
        check(lib().dgq_inv_chol_upper(_ptr(A), K, A.stride(0), _ptr(info), _ptr(ws), nbytes,
                                       _stream()), "dgq_inv_chol_upper")
    return A


def gemm_f32(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, b_is_kn: bool, alpha: float = 1.0,
             beta: float = 0.0, lower_only: bool = False,
             info: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``c = alpha * a @ (b if b_is_kn else b.T) + beta * c`` on the tensor cores, fp32-accurate."""
    _require_cuda(a, b, c)
    m, k = a.shape
    n = c.shape[1]
    assert c.shape[0] == m and b.shape == ((k, n) if b_is_kn else (n, k))
    assert a.stride(1) == 1 and b.stride(1) == 1 and c.stride(1) == 1
    with torch.cuda.device(a.device), _timed("gemm_f32"):
        check(lib().dgq_gemm_f32(_ptr(a), a.stride(0), _ptr(b), b.stride(0), int(b_is_kn), _ptr(c),
                                 c.stride(0), m, n, k, alpha, beta, int(lower_only), _ptr(info),
                                 _stream()), "dgq_gemm_f32")
    return c


def gptq_quantize(W: torch.Tensor, U: torch.Tensor, bits: int, group_size: int, blocksize: int,
                  row_error: bool = False, ws_bytes: Optional[int] = None):
    """Quantizes W ``(N_out, K)`` fp32 in place (it becomes the dequantized Q).

    Returns ``(codes uint8, scales fp32, zeros fp32, total_error device double)``; with
    ``row_error=True`` the last element is the ``(N_out,)`` device vector of per-row error
    sums instead.  ``ws_bytes`` overrides the workspace size (tests of small workspaces)."""
    _require_cuda(W, U)
    assert W.dtype == torch.float32 and W.stride(1) == 1 and U.dtype == torch.float32
    N_out, K = W.shape
    per_channel = group_size <= 0 or group_size >= K
    ng = 1 if per_channel else -(-K // group_size)
    codes = torch.empty((N_out, K), dtype=torch.uint8, device=W.device)
    scales = torch.zeros((N_out, ng), dtype=torch.float32, device=W.device)
    zeros = torch.zeros((N_out, ng), dtype=torch.float32, device=W.device)
    terr = torch.zeros(1, dtype=torch.float64, device=W.device)
    nbytes = lib().dgq_gptq_quantize_workspace_bytes(N_out, K, blocksize)
    check(min(nbytes, 0), "dgq_gptq_quantize_workspace_bytes")
    if ws_bytes is not None:
        nbytes = int(ws_bytes)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=W.device)
    rerr = torch.empty(N_out, dtype=torch.float64, device=W.device) if row_error else None
    with torch.cuda.device(W.device), _timed("gptq_quantize"):
        check(lib().dgq_gptq_quantize_rows(_ptr(W), W.stride(0), _ptr(U), U.stride(0), N_out, K,
                                           bits, group_size, blocksize, _ptr(codes), K,
                                           _ptr(scales), _ptr(zeros), _ptr(terr), _ptr(rerr),
                                           _ptr(ws), nbytes, _stream()),
              "dgq_gptq_quantize")
    return codes, scales, zeros, (rerr if row_error else terr)


def find_params(x: torch.Tensor, bits: int):
    _require_cuda(x)
    assert x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1
    rows, cols = x.shape
    scale = torch.empty(rows, dtype=torch.float32, device=x.device)
    zero = torch.empty(rows, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(lib().dgq_find_params(_ptr(x), x.stride(0), rows, cols, bits, _ptr(scale), _ptr(zero),
                                    _stream()), "dgq_find_params")
    return scale, zero


def quantize_rows(x: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor, bits: int):
    _require_cuda(x, scale, zero)
    assert x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1
    rows, cols = x.shape
    q = torch.empty((rows, cols), dtype=torch.uint8, device=x.device)
    xh = torch.empty((rows, cols), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(lib().dgq_quantize_rows(_ptr(x), x.stride(0), rows, cols, bits, _ptr(scale.contiguous()),
                                      _ptr(zero.contiguous()), _ptr(q), cols, _ptr(xh), cols,
                                      _stream()), "dgq_quantize_rows")
    return q, xh


# --------------------------------------------------------------------------- packing
def packed_row_bytes(cols: int, bits: int, fmt: int) -> int:
    n = lib().dgq_packed_row_bytes(cols, bits, fmt)
    check(min(n, 0), "dgq_packed_row_bytes")
    return n


def _packed_tensor(rows: int, cols: int, bits: int, fmt: int, device) -> torch.Tensor:
    nb = packed_row_bytes(cols, bits, fmt)
    if fmt == FMT_INT32_LE:
        return torch.empty((rows, nb // 4), dtype=torch.int32, device=device)
    dt = torch.int8 if (fmt == FMT_BYTES_HI_FIRST and bits == 8) else torch.uint8
    return torch.empty((rows, nb), dtype=dt, device=device)


def pack(codes: torch.Tensor, bits: int, fmt: int) -> torch.Tensor:
    _require_cuda(codes)
    assert codes.dtype == torch.uint8 and codes.dim() == 2
    codes = codes.contiguous()
    rows, cols = codes.shape
    out = _packed_tensor(rows, cols, bits, fmt, codes.device)
    with torch.cuda.device(codes.device), _timed("pack"):
        check(lib().dgq_pack(_ptr(codes), rows, cols, bits, fmt, _ptr(out), _stream()), "dgq_pack")
    return out


def unpack(packed: torch.Tensor, cols: int, bits: int, fmt: int) -> torch.Tensor:
    _require_cuda(packed)
    packed = packed.contiguous()
    rows = packed.shape[0]
    assert packed.shape[1] * packed.element_size() == packed_row_bytes(cols, bits, fmt)
    codes = torch.empty((rows, cols), dtype=torch.uint8, device=packed.device)
    with torch.cuda.device(packed.device):
        check(lib().dgq_unpack(_ptr(packed), rows, cols, bits, fmt, _ptr(codes), _stream()),
              "dgq_unpack")
    return codes


def unpack_dequant(packed: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor,
                   g_idx: Optional[torch.Tensor], cols: int, bits: int, group_size: int, fmt: int,
                   out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    _require_cuda(packed, scales, zeros, g_idx)
    packed = packed.contiguous()
    rows = packed.shape[0]
    assert packed.shape[1] * packed.element_size() == packed_row_bytes(cols, bits, fmt)
    assert scales.dtype == zeros.dtype and scales.dtype in (torch.float32, torch.float16)
    scales, zeros = scales.contiguous(), zeros.contiguous()
    ng = scales.shape[1] if scales.dim() == 2 else 1
    if g_idx is not None:
        g_idx = g_idx.to(torch.int32).contiguous()
    out = torch.empty((rows, cols), dtype=out_dtype, device=packed.device)
    with torch.cuda.device(packed.device):
        check(lib().dgq_unpack_dequant(_ptr(packed), _ptr(scales), _ptr(zeros), _ptr(g_idx), rows,
                                       cols, ng, bits, group_size, fmt, _DTYPE_CODE[scales.dtype],
                                       _DTYPE_CODE[out_dtype], _ptr(out), _stream()),
              "dgq_unpack_dequant")
    return out


def qlinear_forward(x: torch.Tensor, qweight: torch.Tensor, scales: torch.Tensor,
                    zeros: torch.Tensor, g_idx: Optional[torch.Tensor],
                    bias: Optional[torch.Tensor], in_features: int, bits: int,
                    group_size: int) -> torch.Tensor:
    _require_cuda(x, qweight, scales, zeros, g_idx, bias)
    assert x.dtype in _DTYPE_CODE and x.shape[-1] == in_features
    x2 = x.reshape(-1, in_features).contiguous()
    M = x2.shape[0]
    N_out = qweight.shape[0]
    qweight = qweight.contiguous()
    scales = scales.to(torch.float16).contiguous()
    zeros = zeros.to(torch.float16).contiguous()
    ng = scales.shape[1]
    if g_idx is not None:
        g_idx = g_idx.to(torch.int32).contiguous()
    if bias is not None:
        if bias.dtype not in _DTYPE_CODE:
            bias = bias.float()
        bias = bias.contiguous()
    y = torch.empty((M, N_out), dtype=x.dtype, device=x.device)
    if M > 0:
        with torch.cuda.device(x.device):
            check(lib().dgq_qlinear_forward(
                _ptr(x2), _DTYPE_CODE[x.dtype], M, _ptr(qweight), _ptr(scales), _ptr(zeros),
                _ptr(g_idx), _ptr(bias), _DTYPE_CODE[bias.dtype] if bias is not None else 0,
                N_out, in_features, ng, bits, group_size, _ptr(y), _stream()),
                "dgq_qlinear_forward")
    return y.reshape(*x.shape[:-1], N_out)


# --------------------------------------------------------------------------- flat RTN
def rtn_find_params(x: torch.Tensor, bits: int, group_size: int):
    _require_cuda(x)
    flat = x.contiguous().view(-1)
    assert flat.dtype == torch.float32
    n = flat.numel()
    ng = -(-n // group_size)
    scales = torch.empty(ng, dtype=torch.float32, device=x.device)
    zeros = torch.empty(ng, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(lib().dgq_rtn_find_params(_ptr(flat), n, bits, group_size, _ptr(scales), _ptr(zeros),
                                        _stream()), "dgq_rtn_find_params")
    return scales, zeros


def rtn_quantize(x: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor, bits: int,
                 group_size: int) -> torch.Tensor:
    _require_cuda(x, scales, zeros)
    flat = x.contiguous().view(-1)
    q = torch.empty(flat.numel(), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        check(lib().dgq_rtn_quantize(_ptr(flat), flat.numel(), bits, group_size,
                                     _ptr(scales.contiguous()), _ptr(zeros.contiguous()), _ptr(q),
                                     _stream()), "dgq_rtn_quantize")
    return q.view(x.shape)


def rtn_dequantize(q: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor,
                   group_size: int) -> torch.Tensor:
    _require_cuda(q, scales, zeros)
    flat = q.contiguous().view(-1)
    assert flat.dtype == torch.uint8
    out = torch.empty(flat.numel(), dtype=torch.float32, device=q.device)
    with torch.cuda.device(q.device):
        check(lib().dgq_rtn_dequantize(_ptr(flat), flat.numel(), group_size,
                                       _ptr(scales.float().contiguous()),
                                       _ptr(zeros.float().contiguous()), _ptr(out), _stream()),
              "dgq_rtn_dequantize")
    return out.view(q.shape)
