"""Loader of the native pieces: the C-ABI library (ctypes, `capi`) and the
torch operator library `_C.so` that registers the `*_b200` op namespaces.

There is no fallback: a missing or unloadable native library raises.
"""
from __future__ import annotations

from pathlib import Path

import torch

from . import capi

_HERE = Path(__file__).resolve().parent
_EXT = _HERE / "_C.so"
_loaded = False


def load() -> None:
    """Load the operator library once; raises if it was not built."""
    global _loaded
    if _loaded:
        return
    if not _EXT.exists():
        raise RuntimeError(f"{_EXT} is missing: run `python {_HERE.parent.parent / 'build.py'}` "
                           "(this package has no eager or CPU fallback)")
    capi.lib()                      # resolves libflashrt_b200.so first, with a clear error
    torch.ops.load_library(str(_EXT))
    _loaded = True


def make_ops(namespace: str):
    """(ops, add_op_namespace_prefix) pair for one operator namespace, as the
    reference's generated `_ops.py` modules expose them."""
    load()
    ops = getattr(torch.ops, namespace)

    def add_op_namespace_prefix(op_name: str) -> str:
        return f"{namespace}::{op_name}"

    return ops, add_op_namespace_prefix


def sfa_size_bytes(rows: int, dim: int) -> int:
    if rows <= 0 or dim <= 0 or dim % 16 != 0:
        raise ValueError("rows must be positive and dim must be positive/divisible by 16")
    return ((rows + 127) // 128) * ((dim // 16 + 3) // 4) * 512


def alloc_fp4(rows: int, dim: int, device):
    """packed [rows, dim/2] + zero-filled swizzled scale buffer (padding bytes
    of the scale layout are not written by the producers)."""
    return (torch.empty((rows, dim // 2), device=device, dtype=torch.uint8),
            torch.zeros((sfa_size_bytes(rows, dim),), device=device, dtype=torch.uint8))
