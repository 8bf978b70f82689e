"""Loads the runnable files of the reference by path.  TEST INFRASTRUCTURE ONLY.

The reference package cannot be imported as a package (its ``__init__`` chain has
import-time failures), but three of its files have no intra-package imports and
load standalone: ``core/gptq.py``, ``core/dequantizer.py``, ``models/layers.py``.
This shim is used by the golden-vector generator and by CPU tests that are
skipped when the reference tree is not present.
"""
from __future__ import annotations

import importlib.util
import os
import sys

# the reference checkout: named by DGQ_REFERENCE_ROOT, else a directory `reference` beside this
# repository; absent on machines that only run the GPU tests (callers check `available()`)
DEFAULT_ROOT = os.environ.get("DGQ_REFERENCE_ROOT") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
_SUB = "src/distributed_gptq"


def available(root: str = DEFAULT_ROOT) -> bool:
    return os.path.isfile(os.path.join(root, _SUB, "core", "gptq.py"))


def _load(alias: str, path: str):
    sys.dont_write_bytecode = True  # the reference tree is read-only
    spec = importlib.util.spec_from_file_location(alias, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def load_gptq(root: str = DEFAULT_ROOT):
    return _load("_ref_gptq", os.path.join(root, _SUB, "core", "gptq.py"))


def load_dequantizer(root: str = DEFAULT_ROOT):
    return _load("_ref_dequantizer", os.path.join(root, _SUB, "core", "dequantizer.py"))


def load_layers(root: str = DEFAULT_ROOT):
    return _load("_ref_layers", os.path.join(root, _SUB, "models", "layers.py"))
