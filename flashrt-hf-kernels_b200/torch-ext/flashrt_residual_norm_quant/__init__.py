"""The norm package (B200 build): BF16 RMSNorm / residual RMSNorm, LayerNorm and the static-scale
FP8 variants, with the reference package's function names and schemas
(flashrt-residual-norm-quant/torch-ext/flashrt_residual_norm_quant/__init__.py:97-175)."""
from __future__ import annotations

import torch

from ._ops import add_op_namespace_prefix, ops


def _check(x, other, name):
    if x.dim() != 2 or other.shape != x.shape:
        raise RuntimeError(f"{name} and x must have the same 2D shape")


@torch.library.register_fake(add_op_namespace_prefix("rms_norm_bf16"))
def _rms_norm_fake(x, weight, eps, out) -> None:
    _check(x, out, "out")
    if weight.shape != (x.shape[1],):
        raise RuntimeError("weight must have shape (x.shape[1],)")
    return None


@torch.library.register_fake(add_op_namespace_prefix("residual_add_rms_norm_bf16"))
def _residual_add_rms_norm_fake(residual, x, weight, eps, out) -> None:
    if residual.shape != x.shape:
        raise RuntimeError("residual and x must have the same shape")
    _check(x, out, "out")
    if weight.shape != (x.shape[1],):
        raise RuntimeError("weight must have shape (x.shape[1],)")
    return None


@torch.library.register_fake(add_op_namespace_prefix("layer_norm_bf16"))
def _layer_norm_fake(x, weight, bias, eps, out) -> None:
    _check(x, out, "out")
    if weight.shape != (x.shape[1],) or bias.shape != (x.shape[1],):
        raise RuntimeError("weight and bias must have shape (x.shape[1],)")
    return None


@torch.library.register_fake(add_op_namespace_prefix("rms_norm_quant_fp8_static_bf16"))
def _rms_norm_fp8_fake(x, weight, scale, eps, out) -> None:
    _check(x, out, "out")
    if weight.shape != (x.shape[1],):
        raise RuntimeError("weight must have shape (x.shape[1],)")
    return None


@torch.library.register_fake(add_op_namespace_prefix("residual_add_rms_norm_quant_fp8_static_bf16"))
def _residual_add_rms_norm_fp8_fake(residual, x, weight, scale, eps, out) -> None:
    if residual.shape != x.shape:
        raise RuntimeError("residual and x must have the same shape")
    _check(x, out, "out")
    return None


def layer_norm_bf16(x, weight, bias, eps: float = 1e-5, out=None):
    """BF16 LayerNorm with affine weight and bias."""
    if out is None:
        out = torch.empty_like(x, dtype=torch.bfloat16)
    ops.layer_norm_bf16(x, weight, bias, float(eps), out)
    return out


def rms_norm_quant_fp8_static_bf16(x, weight, scale, eps: float = 1e-6, out=None):
    """BF16 RMSNorm followed by static-scale FP8 E4M3 quantization."""
    if out is None:
        out = torch.empty_like(x, dtype=torch.float8_e4m3fn)
    ops.rms_norm_quant_fp8_static_bf16(x, weight, scale, float(eps), out)
    return out


def residual_add_rms_norm_quant_fp8_static_bf16(residual, x, weight, scale, eps: float = 1e-6, out=None):
    """In-place ``residual += x`` then RMSNorm and static FP8 quantization."""
    if out is None:
        out = torch.empty_like(x, dtype=torch.float8_e4m3fn)
    ops.residual_add_rms_norm_quant_fp8_static_bf16(residual, x, weight, scale, float(eps), out)
    return out


def rms_norm_bf16(x, weight, eps: float = 1e-6, out=None):
    """BF16 RMSNorm with affine weight."""
    if out is None:
        out = torch.empty_like(x, dtype=torch.bfloat16)
    ops.rms_norm_bf16(x, weight, float(eps), out)
    return out


def residual_add_rms_norm_bf16(residual, x, weight, eps: float = 1e-6, out=None):
    """In-place ``residual += x`` followed by weighted BF16 RMSNorm."""
    if out is None:
        out = torch.empty_like(x, dtype=torch.bfloat16)
    ops.residual_add_rms_norm_bf16(residual, x, weight, float(eps), out)
    return out


@torch.library.register_fake(add_op_namespace_prefix("rms_norm_heads_bf16_"))
def _rms_norm_heads_fake(x, weight_a, heads_a, weight_b, heads_b, head_dim, eps) -> None:
    if x.dim() != 2 or (heads_a + heads_b) * head_dim > x.shape[1]:
        raise RuntimeError("x must be (tokens, width) with room for the heads")
    return None


def rms_norm_heads_bf16_(x, weight_a, heads_a: int, weight_b=None, heads_b: int = 0, head_dim: int = 128,
                         eps: float = 1e-6):
    """Per-head RMSNorm in place over the leading heads of every row of `x` (tokens, width; unit inner stride): the q
    and k heads of a stacked q/k/v projection output in one launch.  Extension of this build."""
    ops.rms_norm_heads_bf16_(x, weight_a, int(heads_a), weight_b, int(heads_b), int(head_dim), float(eps))
    return x


__all__ = ["rms_norm_heads_bf16_", "layer_norm_bf16", "residual_add_rms_norm_quant_fp8_static_bf16", "rms_norm_quant_fp8_static_bf16",
           "rms_norm_bf16", "residual_add_rms_norm_bf16"]
