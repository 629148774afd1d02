"""Helpers shared by the GPU tests: the C-ABI library through ctypes, the
reference's own CUDA kernels (oracle/_ref, when built), seeded inputs."""
from __future__ import annotations

import ctypes as C
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "flashrt-hf-kernels_b200" / "torch-ext"))

from flashrt_b200_core import capi  # noqa: E402
from oracle import nvfp4_oracle as O  # noqa: E402

DEV = "cuda"


def sf_bytes(rows, dim):
    return int(capi.lib().frt_nvfp4_sf_swizzled_bytes(rows, dim))


def alloc_fp4(rows, dim, fill=0):
    packed = torch.full((rows, dim // 2), fill, dtype=torch.uint8, device=DEV)
    sf = torch.full((sf_bytes(rows, dim),), fill, dtype=torch.uint8, device=DEV)
    return packed, sf


def quantize(x, packed=None, sf=None):
    rows, dim = x.shape
    if packed is None:
        packed, sf = alloc_fp4(rows, dim)
    dt = 0 if x.dtype == torch.bfloat16 else 1
    capi.check(capi.lib().frt_nvfp4_quantize(capi.ptr(x), dt, capi.ptr(packed), capi.ptr(sf), rows, dim,
                                             capi.stream_ptr()), "quantize")
    return packed, sf


def gemm(a, sfa, b, sfb, M, N, K, alpha=1.0, bias=None, c=None, beta=0.0, out=None):
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=DEV)
    capi.check(capi.lib().frt_nvfp4_gemm_bf16(capi.ptr(a), capi.ptr(sfa), capi.ptr(b), capi.ptr(sfb),
                                              capi.ptr(bias), capi.ptr(c), capi.ptr(out), M, N, K,
                                              float(alpha), float(beta), capi.stream_ptr()), "gemm")
    return out


def device_status():
    v = C.c_uint(0)
    capi.check(capi.lib().frt_device_status(capi.stream_ptr(), C.byref(v)))
    return v.value


def sf_linear(sf_swizzled, rows, dim):
    return O.sf_swizzled_to_linear(sf_swizzled.cpu().numpy(), rows, dim)


def bits(t):
    return O.torch_bf16_to_bits(t)


def randn_bf16(shape, seed, scale=1.0, offset=0.0):
    g = torch.Generator().manual_seed(seed)
    return (offset + scale * torch.randn(shape, generator=g)).to(torch.bfloat16)


# ---- the reference's own CUDA kernels ------------------------------------
_REF = None


def ref_lib():
    """oracle/_ref/libflashrt_ref.so or None when it was not built."""
    global _REF
    if _REF is None:
        path = ROOT / "oracle" / "_ref" / "libflashrt_ref.so"
        if not path.exists():
            _REF = False
        else:
            _REF = C.CDLL(str(path))
    return _REF or None
