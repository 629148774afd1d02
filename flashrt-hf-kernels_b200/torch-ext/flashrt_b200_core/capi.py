"""ctypes binding of the C ABI declared in include/flashrt_b200.h.

The library is the product: if it is missing this module raises, it never
falls back to another implementation.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_PKG = Path(__file__).resolve().parent.parent.parent       # flashrt-hf-kernels_b200/
LIB_PATH = _PKG / "lib" / "libflashrt_b200.so"

_P, _I, _F, _L, _U = C.c_void_p, C.c_int, C.c_float, C.c_int64, C.c_uint

# name -> (restype, argtypes); must list every symbol of include/flashrt_b200.h
SIGNATURES = {
    "frt_error_string": (C.c_char_p, [_I]),
    "frt_nvfp4_sf_swizzled_bytes": (_L, [_I, _I]),
    "frt_nvfp4_sf_offset": (_L, [_I, _I, _I]),
    "frt_nvfp4_sf_linear_to_swizzled": (_I, [_P, _P, _I, _I, _P]),
    "frt_nvfp4_quantize": (_I, [_P, _I, _P, _P, _I, _I, _P]),
    "frt_nvfp4_quantize_mse": (_I, [_P, _I, _P, _P, _I, _I, _P]),
    "frt_nvfp4_dequantize_fp16": (_I, [_P, _P, _P, _I, _I, _P]),
    "frt_rms_norm_bf16": (_I, [_P, _P, _P, _I, _I, _F, _P]),
    "frt_rms_norm_heads_bf16": (_I, [_P, _I, _I, _I, _I, _P, _I, _P, _F, _P]),
    "frt_residual_add_rms_norm_bf16": (_I, [_P, _P, _P, _P, _I, _I, _F, _P]),
    "frt_norm_quant_nvfp4": (_I, [_P, _P, _P, _F, _F, _P, _P, _P, _I, _I, _U, _P]),
    "frt_norm_quant_nvfp4_bcast": (_I, [_P, _P, _P, _F, _F, _P, _P, C.POINTER(_P), C.POINTER(_P), _I, _I, _I, _I, _U, _P,
                                         C.POINTER(_P), _I, _I, _U, _P]),
    "frt_peer_wait": (_I, [_P, _I, _U, _P]),
    "frt_nvfp4_gemm_bf16": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _F, _F, _P]),
    "frt_nvfp4_repack_interleaved": (_I, [_P, _P, _I, _I, _P]),
    "frt_nvfp4_gemv_interleaved_bf16": (_I, [_P, _P, _P, _P, _P, _I, _I, _F, _P]),
    "frt_nvfp4_gemm_plan": (_I, [_I, _I, _I, C.POINTER(_I), C.POINTER(_I)]),
    "frt_router_topk_bf16": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "frt_router_topk_softmax_bf16": (_I, [_P, _P, _P, _P, _I, _I, _I, _P]),
    "frt_moe_quantize_scatter_nvfp4": (_I, [_P, _P, _P, _P, _I, _I, _I, _P]),
    "frt_moe_route_plan": (_I, [_P, _I, _I, _I, _P, _P, _P, _P]),
    "frt_moe_gather_nvfp4": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _P]),
    "frt_moe_weighted_sum_bf16": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "frt_residual_norm_quant_nvfp4_fp16": (_I, [_P, _P, _F, _P, _P, _I, _I, _P]),
    "frt_layer_norm_bf16": (_I, [_P, _P, _P, _P, _I, _I, _F, _P]),
    "frt_rms_norm_quant_fp8": (_I, [_P, _P, _P, _P, _P, _I, _I, _F, _P]),
    "frt_silu_mul_quant_nvfp4": (_I, [_P, _P, _P, _I, _I, _P]),
    "frt_nvfp4_gemm_swiglu_nvfp4": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _F, _P]),
    "frt_nvfp4_grouped_gemm_workspace_bytes": (_L, [_I, _I]),
    "frt_nvfp4_grouped_gemm_bf16": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _L, _L, _P, _P]),
    "frt_nvfp4_grouped_gemm_bf16_noalloc": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _L, _L, _P]),
    "frt_device_status": (_I, [_P, C.POINTER(_U)]),
    "frt_launch_count": (_L, []),
    "frt_set_option": (_I, [_I, _I]),
}

_lib = None


def lib():
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python {_PKG / 'build.py'}` (there is no fallback path)")
        handle = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(rc: int, what: str = "flashrt_b200"):
    if rc != 0:
        raise RuntimeError(f"{what} failed: rc={rc} ({lib().frt_error_string(rc).decode()})")


def ptr(t):
    """device pointer of a torch tensor (None -> NULL)"""
    return None if t is None else C.c_void_p(t.data_ptr())


def stream_ptr(stream=None):
    import torch
    s = torch.cuda.current_stream() if stream is None else stream
    return C.c_void_p(s.cuda_stream)
