"""Fused (residual-add +) RMSNorm -> NVFP4 producers (B200 build), with the
reference package's function names and return conventions
(fp4-fused-ops/torch-ext/fp4_fused_ops/__init__.py:10-21,291-306,458-473,722-737)."""
from __future__ import annotations

import torch

from flashrt_b200_core import alloc_fp4 as _alloc_fp4

from ._ops import add_op_namespace_prefix, ops


def sfa_size_bytes(rows: int, dim: int, is_sfb: bool = False, device=None) -> int:
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    anchor = torch.empty((1,), device=device, dtype=torch.uint8)
    return int(ops.sfa_size_bytes_for(anchor, int(rows), int(dim), bool(is_sfb)))


def _check_producer(x, packed, sfa):
    if x.dim() != 2 or x.shape[1] % 16 != 0:
        raise RuntimeError("x must have shape (rows, dim), dim divisible by 16")
    if packed.shape != (x.shape[0], x.shape[1] // 2) or sfa.dim() != 1:
        raise RuntimeError("packed must have shape (rows, dim / 2) and sfa must be flat")


@torch.library.register_fake(add_op_namespace_prefix("sfa_size_bytes_for"))
def _sfa_size_fake(anchor, rows, dim, is_sfb=False) -> int:
    return ((rows + 127) // 128) * ((dim // 16 + 3) // 4) * 512


@torch.library.register_fake(add_op_namespace_prefix("rms_norm_quantize_fp4_sfa_bf16"))
def _rms_norm_quantize_fake(x, weight, eps, normed, packed, sfa) -> None:
    _check_producer(x, packed, sfa)
    if normed.shape != x.shape:
        raise RuntimeError("normed must have the shape of x")
    return None


@torch.library.register_fake(add_op_namespace_prefix("residual_add_rms_norm_nvfp4_bf16"))
def _residual_add_rms_norm_nvfp4_fake(residual, x, inv_s, eps, packed, sfa) -> None:
    _check_producer(x, packed, sfa)
    return None


@torch.library.register_fake(add_op_namespace_prefix("residual_add_rms_norm_quant_nvfp4_swizzled_bf16"))
def _residual_add_rms_norm_quant_fake(residual, x, weight, eps, packed, sfa) -> None:
    _check_producer(x, packed, sfa)
    if residual.shape != x.shape:
        raise RuntimeError("residual and x must have the same 2D shape")
    return None


@torch.library.register_fake(add_op_namespace_prefix("residual_add_rms_norm_quant_nvfp4_ex"))
def _residual_add_rms_norm_quant_ex_fake(residual, x, weight, eps, inv_global_scale, normed, packed, sfa) -> None:
    _check_producer(x, packed, sfa)
    return None


@torch.library.register_fake(add_op_namespace_prefix("dequantize_fp4_sfa_fp16"))
def _dequantize_fake(packed, sfa, out) -> None:
    return None


@torch.library.register_fake(add_op_namespace_prefix("silu_mul_quantize_fp4_sfa_bf16"))
def _silu_mul_quantize_fake(merged, packed, sfa) -> None:
    if merged.dim() != 2 or merged.shape[1] % 32 != 0:
        raise RuntimeError("merged must have shape (rows, 2 * hidden), hidden divisible by 16")
    rows, twice_hidden = merged.shape
    if packed.shape != (rows, twice_hidden // 4) or sfa.dim() != 1:
        raise RuntimeError("packed/SFA output shape contract failed")
    return None


def silu_mul_quantize_fp4_sfa_bf16(merged, *, packed=None, sfa=None):
    """SiLU(gate) * up of ``merged = [gate | up]`` in fp32, rounded to bf16 and quantised to
    NVFP4 (fp4-fused-ops/torch-ext/fp4_fused_ops/__init__.py:276-288)."""
    rows, twice_hidden = merged.shape
    if packed is None or sfa is None:
        packed, sfa = _alloc_fp4(rows, twice_hidden // 2, merged.device)
    ops.silu_mul_quantize_fp4_sfa_bf16(merged, packed, sfa)
    return packed, sfa


def rms_norm_quantize_fp4_sfa_bf16(x, weight, eps: float = 1e-6, *, normed=None, packed=None, sfa=None):
    """RMSNorm with residual-form weight ``1 + weight``; emits the bf16 `normed`
    tensor and its NVFP4 quantisation."""
    if normed is None:
        normed = torch.empty_like(x)
    if packed is None or sfa is None:
        packed, sfa = _alloc_fp4(x.shape[0], x.shape[1], x.device)
    ops.rms_norm_quantize_fp4_sfa_bf16(x, weight, float(eps), normed, packed, sfa)
    return normed, packed, sfa


def residual_add_rms_norm_nvfp4_bf16(residual, x, inv_s=None, eps: float = 1e-6, *, packed=None, sfa=None):
    """Update a BF16 residual, RMS-normalise and produce NVFP4 (hardware
    round-to-nearest-even element codes)."""
    if packed is None or sfa is None:
        packed, sfa = _alloc_fp4(x.shape[0], x.shape[1], x.device)
    ops.residual_add_rms_norm_nvfp4_bf16(residual, x, inv_s, float(eps), packed, sfa)
    return residual, packed, sfa


def residual_add_rms_norm_quant_nvfp4_swizzled_bf16(residual, x, weight, eps: float = 1e-6, *, packed=None,
                                                    sfa=None):
    """``residual += x`` in place, weighted RMSNorm of the fp32 sum, NVFP4 with
    swizzled UE4M3 scales: the activation producer of the low-bit linear path."""
    if packed is None or sfa is None:
        packed, sfa = _alloc_fp4(x.shape[0], x.shape[1], x.device)
    ops.residual_add_rms_norm_quant_nvfp4_swizzled_bf16(residual, x, weight, float(eps), packed, sfa)
    return packed, sfa


def residual_add_rms_norm_quant_nvfp4(residual, x, weight, eps: float = 1e-6, *, inv_global_scale: float = 1.0,
                                      normed=None, packed=None, sfa=None):
    """Additive variant: optional per-tensor second-level scale (the norm result
    is multiplied by `inv_global_scale` before quantisation; fold the matching
    global scale into the GEMM's alpha) and optional bf16 copy of the
    quantiser input."""
    if packed is None or sfa is None:
        packed, sfa = _alloc_fp4(x.shape[0], x.shape[1], x.device)
    ops.residual_add_rms_norm_quant_nvfp4_ex(residual, x, weight, float(eps), float(inv_global_scale), normed,
                                             packed, sfa)
    return packed, sfa


@torch.library.register_fake(add_op_namespace_prefix("rms_norm_quant_nvfp4_ex"))
def _rms_norm_quant_ex_fake(x, weight, eps, normed, packed, sfa, one_plus_weight=False, round_bf16=True) -> None:
    _check_producer(x, packed, sfa)
    return None


def rms_norm_quant_nvfp4(x, weight, eps: float = 1e-6, *, one_plus_weight: bool = False, round_bf16: bool = True,
                         normed=None, packed=None, sfa=None):
    """Additive variant without a residual: RMSNorm with a plain (or ``1 + weight``) weight,
    NVFP4 of the result and, when `normed` is given, its bf16 copy in the same pass."""
    if packed is None or sfa is None:
        packed, sfa = _alloc_fp4(x.shape[0], x.shape[1], x.device)
    ops.rms_norm_quant_nvfp4_ex(x, weight, float(eps), normed, packed, sfa, bool(one_plus_weight), bool(round_bf16))
    return packed, sfa


@torch.library.register_fake(add_op_namespace_prefix("residual_add_rms_norm_fp4_sfa_v2_fp16"))
def _residual_add_rms_norm_fp16_fake(residual, x, packed, sfa) -> None:
    _check_producer(x, packed, sfa)
    if residual.shape != x.shape:
        raise RuntimeError("residual and x must have the same 2D shape")
    return None


def residual_add_rms_norm_fp4_sfa_v2_fp16(residual, x, *, packed=None, sfa=None):
    """FP16 ``residual += x`` in place, unweighted RMSNorm (eps 1e-6) of the fp32 sum, NVFP4 with swizzled
    scales (fp4-fused-ops/torch-ext/fp4_fused_ops/__init__.py: residual_add_rms_norm_fp4_sfa_v2_fp16)."""
    if packed is None or sfa is None:
        packed, sfa = _alloc_fp4(x.shape[0], x.shape[1], x.device)
    ops.residual_add_rms_norm_fp4_sfa_v2_fp16(residual, x, packed, sfa)
    return packed, sfa


def dequantize_fp4_sfa_fp16(packed, sfa, out=None):
    if out is None:
        out = torch.empty((packed.shape[0], packed.shape[1] * 2), device=packed.device, dtype=torch.float16)
    ops.dequantize_fp4_sfa_fp16(packed, sfa, out)
    return out


__all__ = ["sfa_size_bytes", "rms_norm_quantize_fp4_sfa_bf16", "residual_add_rms_norm_nvfp4_bf16",
           "residual_add_rms_norm_quant_nvfp4_swizzled_bf16", "residual_add_rms_norm_quant_nvfp4",
           "dequantize_fp4_sfa_fp16", "silu_mul_quantize_fp4_sfa_bf16", "rms_norm_quant_nvfp4", "residual_add_rms_norm_fp4_sfa_v2_fp16"]
