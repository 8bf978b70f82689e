"""The C-ABI library loads without a GPU and exports exactly what include/dgq.h declares."""
import ctypes
import os
import re

from distributed_gptq_b200 import _C

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "dgq.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dgq_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    names = declared_functions()
    assert len(names) >= 25
    assert sorted(_C.SIGNATURES) == names


def test_library_exports_every_declared_symbol():
    L = _C.lib()
    for name in declared_functions():
        assert hasattr(L, name), name
        assert isinstance(getattr(L, name), ctypes._CFuncPtr)


def test_host_only_entry_points():
    L = _C.lib()
    assert L.dgq_version() >= 100
    assert _C.status_string(0) == "ok"
    assert "align" in _C.status_string(-2)
    # packed row lengths (no device needed)
    assert _C.packed_row_bytes(128, 4, _C.FMT_BYTES_HI_FIRST) == 64
    assert _C.packed_row_bytes(27, 4, _C.FMT_BYTES_LO_FIRST) == 14
    assert _C.packed_row_bytes(27, 3, _C.FMT_BYTES_LO_FIRST) == 27
    assert _C.packed_row_bytes(45, 3, _C.FMT_INT32_LE) == 4 * 5
    assert _C.packed_row_bytes(128, 2, _C.FMT_INT32_LE) == 4 * 8
    assert L.dgq_packed_row_bytes(7, 4, _C.FMT_BYTES_HI_FIRST) < 0   # odd column count
    assert L.dgq_packed_row_bytes(8, 5, _C.FMT_BYTES_HI_FIRST) < 0   # bad bit width
    assert L.dgq_inv_chol_workspace_bytes(4096) > 0
    assert L.dgq_gptq_quantize_workspace_bytes(4096, 4096, 128) == 4096 * 256 * 4
    assert L.dgq_gptq_quantize_workspace_bytes(4096, 4096, 256) < 0


def test_argument_validation_needs_no_device():
    L = _C.lib()
    # null pointers / bad sizes are rejected before any CUDA call
    assert L.dgq_pack(None, 4, 8, 4, 1, None, None) == -1
    assert L.dgq_hessian_accum(None, 16, 64, 64, None, 64, 1.0, 0, None, None) == -1
    assert L.dgq_inv_chol_upper(None, 8, 8, None, None, 0, None) == -1


def test_g_idx_classification_is_host_logic():
    """The operator passes a column-to-group map on to the kernels only when it is a general one:
    the reference constructor's default (``range(in_features)``) holds no valid group numbers, and
    the sequential map ``c // group_size`` is what the kernels compute themselves."""
    import torch
    from distributed_gptq_b200 import ops
    K, g = 512, 128
    n_groups = K // g
    seq = (torch.arange(K) // g).to(torch.int32)
    assert ops._classify_g_idx(seq, n_groups) == ops._SEQUENTIAL
    assert ops._classify_g_idx(torch.arange(K, dtype=torch.int32), n_groups) == ops._INVALID
    perm = seq[torch.randperm(K, generator=torch.Generator().manual_seed(0))].contiguous()
    assert ops._classify_g_idx(perm, n_groups) == ops._GENERAL
    assert ops._g_idx_usable(perm, n_groups) and ops._g_idx_usable(seq, n_groups)
    # ragged last group: the operator can only infer ceil(K / n_groups) = 104 columns per group,
    # so the true map (groups of 128) is a general one and is passed on
    K2 = 520
    seq2 = (torch.arange(K2) // 128).to(torch.int32)
    assert ops._classify_g_idx(seq2, 5) == ops._GENERAL
