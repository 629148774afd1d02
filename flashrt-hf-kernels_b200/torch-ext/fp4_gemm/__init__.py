"""NVFP4 A4W4 GEMM and quantise helpers (B200 build) with the reference
package's function names (fp4-gemm/torch-ext/fp4_gemm/__init__.py).  Only the
members on the NVFP4 linear path are provided; `variant`, `warps` and `stages`
are accepted for call compatibility and do not select kernels: the tile
configuration follows from the shape."""
from __future__ import annotations

from typing import Optional

import torch

from flashrt_b200_core import alloc_fp4 as _alloc_fp4, sfa_size_bytes

from ._ops import add_op_namespace_prefix, ops


def capabilities() -> dict:
    """Facts about this build (mirrors the reference's capabilities() dict)."""
    return {
        "arch": "sm_100a",
        "device": "NVIDIA B200",
        "gemm": "tcgen05.mma kind::mxf4nvf4 (block 16, UE4M3), TMEM accumulators, TMA-fed, persistent",
        "outputs": ("bf16",),
        "epilogues": ("alpha", "bias", "residual", "bias+residual"),
        "k_alignment": 32,
        "n_alignment": 8,
        "small_m_max": 64,
        "quantizer_rule": "thresholds, ties to the smaller magnitude; scale = e4m3_rn(max(amax/6, 1e-12))",
        "graph_safe": True,
        "errors": "exceptions",
    }


def _gemm_fake_check(a, b, out):
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[1]:
        raise RuntimeError("a_packed and b_packed must be (M, K/2) and (N, K/2)")
    if out.shape != (a.shape[0], b.shape[0]):
        raise RuntimeError("out must have shape (M, N)")


@torch.library.register_fake(add_op_namespace_prefix("nvfp4_gemm_bf16"))
def _gemm_fake(a_packed, b_packed, sfa, sfb, out, alpha=1.0, variant=-1) -> None:
    _gemm_fake_check(a_packed, b_packed, out)
    return None


@torch.library.register_fake(add_op_namespace_prefix("fp4_w4a16_linear_bf16"))
def _linear_fake(a_packed, b_packed, sfa, sfb, out, alpha=1.0, variant=-1) -> None:
    _gemm_fake_check(a_packed, b_packed, out)
    return None


@torch.library.register_fake(add_op_namespace_prefix("nvfp4_gemm_bias_bf16"))
def _bias_fake(a, b, sfa, sfb, bias, out) -> None:
    _gemm_fake_check(a, b, out)
    return None


@torch.library.register_fake(add_op_namespace_prefix("nvfp4_gemm_bias_residual_bf16"))
def _bias_residual_fake(a, b, sfa, sfb, bias, residual, out) -> None:
    _gemm_fake_check(a, b, out)
    return None


@torch.library.register_fake(add_op_namespace_prefix("nvfp4_gemm_residual_bf16"))
def _residual_fake(a, b, sfa, sfb, residual, out, alpha=1.0) -> None:
    _gemm_fake_check(a, b, out)
    return None


@torch.library.register_fake(add_op_namespace_prefix("fp4_w4a4_gemv_warpsplit_bf16"))
def _gemv_fake(a, b, sfa, sfb, out, alpha=1.0, warps=4, stages=4) -> None:
    return None


@torch.library.register_fake(add_op_namespace_prefix("fp4_w4a4_gemm_warpsplit_mrows_bf16"))
def _mrows_fake(a, b, sfa, sfb, out, alpha=1.0, warps=2, stages=6) -> None:
    return None


@torch.library.register_fake(add_op_namespace_prefix("quantize_fp4_sfa_fp16"))
def _quantize_fp16_fake(x, packed, sfa, is_sfb=False) -> None:
    return None


@torch.library.register_fake(add_op_namespace_prefix("quantize_fp4_sfa_bf16"))
def _quantize_bf16_fake(x, packed, sfa, is_sfb=False) -> None:
    return None


@torch.library.register_fake(add_op_namespace_prefix("dequantize_fp4_sfa_fp16"))
def _dequantize_fake(packed, sfa, out, is_sfb=False) -> None:
    return None


def quantize_fp4_sfa_fp16(x, packed=None, sfa=None, is_sfb: bool = False):
    if packed is None or sfa is None:
        packed, sfa = _alloc_fp4(x.shape[0], x.shape[1], x.device)
    ops.quantize_fp4_sfa_fp16(x, packed, sfa, bool(is_sfb))
    return packed, sfa


def quantize_fp4_sfa_bf16(x, packed=None, sfa=None, is_sfb: bool = False):
    if packed is None or sfa is None:
        packed, sfa = _alloc_fp4(x.shape[0], x.shape[1], x.device)
    ops.quantize_fp4_sfa_bf16(x, packed, sfa, bool(is_sfb))
    return packed, sfa


@torch.library.register_fake(add_op_namespace_prefix("quantize_fp4_sfa_bf16_pdl"))
def _quantize_bf16_pdl_fake(x, packed, sfa, is_sfb=False) -> None:
    return None


@torch.library.register_fake(add_op_namespace_prefix("fp4_w4a4_gemm_warpsplit_mrows_pdl_bf16"))
def _mrows_pdl_fake(a, b, sfa, sfb, out, alpha=1.0, warps=2, stages=6) -> None:
    _gemm_fake_check(a, b, out)
    return None


def quantize_fp4_sfa_bf16_pdl(x, packed=None, sfa=None, is_sfb: bool = False):
    """PDL-enabled twin of :func:`quantize_fp4_sfa_bf16` (every launch of this build is one already)."""
    if packed is None or sfa is None:
        packed, sfa = _alloc_fp4(x.shape[0], x.shape[1], x.device)
    ops.quantize_fp4_sfa_bf16_pdl(x, packed, sfa, bool(is_sfb))
    return packed, sfa


def dequantize_fp4_sfa_fp16(packed, sfa, out=None, is_sfb: bool = False):
    if out is None:
        out = torch.empty((packed.shape[0], packed.shape[1] * 2), device=packed.device, dtype=torch.float16)
    ops.dequantize_fp4_sfa_fp16(packed, sfa, out, bool(is_sfb))
    return out


def _out_like(a_packed, b_packed):
    return torch.empty((a_packed.shape[0], b_packed.shape[0]), device=a_packed.device, dtype=torch.bfloat16)


def nvfp4_gemm_bf16(a_packed, b_packed, sfa, sfb, alpha: float = 1.0, out=None, variant: int = -1):
    """out[M,N] = bf16(alpha * A . B^T) for packed NVFP4 A [M,K/2], B [N,K/2]."""
    if out is None:
        out = _out_like(a_packed, b_packed)
    ops.nvfp4_gemm_bf16(a_packed, b_packed, sfa, sfb, out, float(alpha), int(variant))
    return out


@torch.library.register_fake(add_op_namespace_prefix("nvfp4_gemm_swiglu_nvfp4_bf16"))
def _gemm_swiglu_fake(a_packed, b_packed, sfa, sfb, out_packed, out_sfa, alpha=1.0) -> None:
    if a_packed.dim() != 2 or b_packed.dim() != 2 or a_packed.shape[1] != b_packed.shape[1]:
        raise RuntimeError("a_packed and b_packed must be matrices with the same packed K")
    if b_packed.shape[0] % 256 != 0:
        raise RuntimeError("stacked gate/up N must be divisible by 256")
    if out_packed.shape != (a_packed.shape[0], b_packed.shape[0] // 4) or out_sfa.dim() != 1:
        raise RuntimeError("out_packed must have shape (M, N / 4) and out_sfa must be flat")
    return None


def nvfp4_gemm_swiglu_nvfp4_bf16(a_packed, b_packed, sfa, sfb, alpha: float = 1.0, *, out_packed=None,
                                 out_sfa=None):
    """gate/up projection with the SwiGLU -> NVFP4 producer as the GEMM epilogue.

    ``b_packed`` is the stacked ``[gate ; up]`` weight (2 * hidden rows).  Returns the NVFP4
    tensor ``(out_packed [M, hidden / 2], out_sfa)`` that
    ``silu_mul_quantize_fp4_sfa_bf16(nvfp4_gemm_bf16(a, b))`` would produce, bit for bit,
    without writing the (M, 2 * hidden) bf16 intermediate.  Additive: the reference's
    FP4-output epilogues (nvfp4_gemm_nvfp4, nvfp4_gemm_geglu_nvfp4_fp16,
    fp4-gemm/torch-ext/fp4_gemm/__init__.py:591-620) are SM110-only and need a weight repack."""
    if out_packed is None or out_sfa is None:
        out_packed, out_sfa = _alloc_fp4(a_packed.shape[0], b_packed.shape[0] // 2, a_packed.device)
    ops.nvfp4_gemm_swiglu_nvfp4_bf16(a_packed, b_packed, sfa, sfb, out_packed, out_sfa, float(alpha))
    return out_packed, out_sfa


def fp4_w4a16_linear_bf16(a_packed, b_packed, sfa, sfb, alpha: float = 1.0, out=None, variant: int = -1):
    """Compatibility alias for :func:`nvfp4_gemm_bf16`."""
    return nvfp4_gemm_bf16(a_packed, b_packed, sfa, sfb, alpha=alpha, out=out, variant=variant)


def nvfp4_gemm_bias_bf16(a_packed, b_packed, sfa, sfb, bias, *, out=None):
    if out is None:
        out = _out_like(a_packed, b_packed)
    ops.nvfp4_gemm_bias_bf16(a_packed, b_packed, sfa, sfb, bias, out)
    return out


def nvfp4_gemm_bias_residual_bf16(a_packed, b_packed, sfa, sfb, bias, residual, *, out=None):
    if out is None:
        out = torch.empty_like(residual)
    ops.nvfp4_gemm_bias_residual_bf16(a_packed, b_packed, sfa, sfb, bias, residual, out)
    return out


def nvfp4_gemm_residual_bf16(a_packed, b_packed, sfa, sfb, residual, alpha: float = 1.0, out=None):
    if out is None:
        out = torch.empty_like(residual)
    ops.nvfp4_gemm_residual_bf16(a_packed, b_packed, sfa, sfb, residual, out, float(alpha))
    return out


def fp4_w4a4_gemv_warpsplit_bf16(a_packed, b_packed, sfa, sfb, *, alpha: float = 1.0, warps: int = 4,
                                 stages: int = 4, out: Optional[torch.Tensor] = None):
    """M = 1 decode row (weight-streaming configuration of the same GEMM)."""
    if out is None:
        out = torch.empty((1, b_packed.shape[0]), device=a_packed.device, dtype=torch.bfloat16)
    ops.fp4_w4a4_gemv_warpsplit_bf16(a_packed, b_packed, sfa, sfb, out, float(alpha), int(warps), int(stages))
    return out


@torch.library.register_fake(add_op_namespace_prefix("fp4_repack_b_interleaved_sm120"))
def _repack_b_interleaved_fake(b_packed, b_interleaved) -> None:
    if b_interleaved.shape != b_packed.shape:
        raise RuntimeError("b_interleaved must have the same shape as b_packed")
    return None


@torch.library.register_fake(add_op_namespace_prefix("fp4_w4a4_gemv_warpsplit_interleaved_bf16"))
def _gemv_warpsplit_interleaved_fake(a_packed, b_interleaved, sfa, sfb, out, alpha=1.0, warps=4, stages=4) -> None:
    if a_packed.shape[0] != 1:
        raise RuntimeError("interleaved warp-split GEMV serves M=1 only")
    if out.shape != (1, b_interleaved.shape[0]):
        raise RuntimeError("out must have shape (1, N)")
    return None


def fp4_repack_b_interleaved_sm120(b_packed: torch.Tensor, *, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Bind-time repack of a dense row-major packed weight into the M = 1 GEMV layout
    ([N/8][K/64][8][32 B]; fp4-gemm/torch-ext/fp4_gemm/__init__.py:760-773).  The name is the reference's;
    on B200 the layout is read through a 4-D tensor map by the same weight-streaming kernel."""
    if out is None:
        out = torch.empty_like(b_packed)
    ops.fp4_repack_b_interleaved_sm120(b_packed, out)
    return out


def fp4_w4a4_gemv_warpsplit_interleaved_bf16(a_packed, b_interleaved, sfa, sfb, *, alpha: float = 1.0, warps: int = 8,
                                             stages: int = 3, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """M = 1 GEMV over a weight repacked by fp4_repack_b_interleaved_sm120 (bit-equal to the plain-layout GEMV)."""
    if out is None:
        out = torch.empty((1, b_interleaved.shape[0]), device=a_packed.device, dtype=torch.bfloat16)
    ops.fp4_w4a4_gemv_warpsplit_interleaved_bf16(a_packed, b_interleaved, sfa, sfb, out, float(alpha), int(warps),
                                                 int(stages))
    return out


def fp4_w4a4_gemm_warpsplit_mrows_bf16(a_packed, b_packed, sfa, sfb, *, alpha: float = 1.0, warps: int = 2,
                                       stages: int = 6, out: Optional[torch.Tensor] = None):
    """1..16 rows riding one weight stream."""
    if out is None:
        out = _out_like(a_packed, b_packed)
    ops.fp4_w4a4_gemm_warpsplit_mrows_bf16(a_packed, b_packed, sfa, sfb, out, float(alpha), int(warps),
                                           int(stages))
    return out


@torch.library.register_fake(add_op_namespace_prefix("quantize_fp4_sfa_mse_fp16"))
def _quant_mse_fake(x, packed, sfa, is_sfb: bool = False) -> None:
    return None


@torch.library.register_fake(add_op_namespace_prefix("quantize_fp4_sfa_mse_bf16"))
def _quant_mse_bf16_fake(x, packed, sfa, is_sfb: bool = False) -> None:
    return None


def quantize_fp4_sfa_mse_fp16(x, packed=None, sfa=None, is_sfb: bool = False):
    """Pack FP16 weights using per-block reconstruction-MSE scale search."""
    if packed is None or sfa is None:
        packed, sfa = _alloc_fp4(x.shape[0], x.shape[1], x.device)
    ops.quantize_fp4_sfa_mse_fp16(x, packed, sfa, bool(is_sfb))
    return packed, sfa


def quantize_fp4_sfa_mse_bf16(x, packed=None, sfa=None, is_sfb: bool = False):
    """Pack BF16 weights using per-block reconstruction-MSE scale search."""
    if packed is None or sfa is None:
        packed, sfa = _alloc_fp4(x.shape[0], x.shape[1], x.device)
    ops.quantize_fp4_sfa_mse_bf16(x, packed, sfa, bool(is_sfb))
    return packed, sfa


def aligned_fp4_dim(dim: int, alignment: int = 32) -> int:
    """Physical FP4 GEMM dimension of a logical dimension (fp4-gemm/torch-ext/fp4_gemm/__init__.py:342-346)."""
    if dim <= 0 or alignment <= 0 or alignment % 16 != 0:
        raise ValueError("dim must be positive and alignment divisible by 16")
    return ((dim + alignment - 1) // alignment) * alignment


def quantize_fp4_sfa_padded_bf16(x, *, alignment: int = 32, is_sfb: bool = False):
    """Bind-time BF16 pack with zero padding of the last dimension; returns
    (packed, sfa, logical_dim).  Allocates: not a hot-path op."""
    if x.ndim != 2 or x.dtype != torch.bfloat16:
        raise ValueError("x must be a 2-D BF16 tensor")
    logical_dim = int(x.shape[1])
    physical_dim = aligned_fp4_dim(logical_dim, alignment)
    if physical_dim == logical_dim:
        padded = x.contiguous()
    else:
        padded = torch.zeros((x.shape[0], physical_dim), device=x.device, dtype=x.dtype)
        padded[:, :logical_dim].copy_(x)
    packed, sfa = quantize_fp4_sfa_bf16(padded, is_sfb=is_sfb)
    return packed, sfa, logical_dim


def pack_nvfp4_weight_bf16(weight: torch.Tensor, bias: Optional[torch.Tensor] = None, *, alignment: int = 32,
                           mse: bool = False):
    """Bind-time packing of a logical ``(N, K)`` BF16 weight: zero-pads both dimensions to
    `alignment` (4304 -> 4320 and the like), quantises (optionally with the MSE scale search)
    and returns ``(packed, sfb, padded_bias, (logical_n, logical_k))``
    (fp4-gemm/torch-ext/fp4_gemm/__init__.py:376-411)."""
    if weight.ndim != 2 or weight.dtype != torch.bfloat16:
        raise ValueError("weight must be a 2-D BF16 tensor")
    logical_n, logical_k = map(int, weight.shape)
    physical_n = aligned_fp4_dim(logical_n, alignment)
    physical_k = aligned_fp4_dim(logical_k, alignment)
    padded_weight = torch.zeros((physical_n, physical_k), device=weight.device, dtype=weight.dtype)
    padded_weight[:logical_n, :logical_k].copy_(weight)
    quantize = quantize_fp4_sfa_mse_bf16 if mse else quantize_fp4_sfa_bf16
    packed, sfb = quantize(padded_weight, is_sfb=True)
    padded_bias = None
    if bias is not None:
        if bias.ndim != 1 or bias.numel() != logical_n:
            raise ValueError("bias must have shape (N,)")
        if bias.dtype != torch.bfloat16 or bias.device != weight.device:
            raise ValueError("bias must match the weight dtype and device")
        padded_bias = torch.zeros((physical_n,), device=bias.device, dtype=bias.dtype)
        padded_bias[:logical_n].copy_(bias)
    return packed, sfb, padded_bias, (logical_n, logical_k)


def adopt_modelopt_nvfp4_weight(weight_packed: torch.Tensor, weight_scale: torch.Tensor,
                                weight_scale_2: torch.Tensor):
    """Bind-time adoption of a standard ModelOpt NVFP4 (two-level) weight for the A4W4 GEMM.

    Inputs: ``weight[N, K/2]`` uint8 (two e2m1 codes per byte, low nibble first, the layout
    this path uses), ``weight_scale[N, K/16]`` float8_e4m3fn (or its uint8 bytes) in row-major
    order, and the scalar per-tensor ``weight_scale_2``.  Returns ``(b_packed, sfb, alpha)``:
    the packed weight unchanged, the block scales re-laid into the swizzled buffer the tensor
    cores read, and the global scale as a float to multiply into the GEMM's ``alpha``
    (together with the activation's global scale, when it has one).  The dequantisation this
    reproduces is the one the reference's oracle uses for such weights
    (fp4-gemm/tests/test_fp4_gemm.py:1150-1164)."""
    import flashrt_nvfp4
    if weight_packed.dtype != torch.uint8 or weight_packed.ndim != 2:
        raise ValueError("weight_packed must be uint8 with shape (N, K / 2)")
    n, k = weight_packed.shape[0], weight_packed.shape[1] * 2
    if k % 32 != 0:
        raise ValueError("K must be divisible by 32")
    if tuple(weight_scale.shape) != (n, k // 16):
        raise ValueError("weight_scale must have shape (N, K / 16)")
    if weight_scale_2.numel() != 1:
        raise ValueError("weight_scale_2 must contain one global scale")
    scale_bytes = weight_scale.contiguous().view(torch.uint8)
    if bool((scale_bytes & 0x80).any()):
        raise ValueError("block scales must be non-negative (UE4M3)")
    sfb = flashrt_nvfp4.nvfp4_sf_linear_to_swizzled(scale_bytes, is_sfb=True)
    return weight_packed.contiguous(), sfb, float(weight_scale_2.float().item())


__all__ = ["capabilities", "sfa_size_bytes", "quantize_fp4_sfa_fp16", "quantize_fp4_sfa_bf16",
           "dequantize_fp4_sfa_fp16", "nvfp4_gemm_bf16", "nvfp4_gemm_swiglu_nvfp4_bf16", "fp4_w4a16_linear_bf16",
           "nvfp4_gemm_bias_bf16",
           "nvfp4_gemm_bias_residual_bf16", "nvfp4_gemm_residual_bf16", "fp4_w4a4_gemv_warpsplit_bf16",
           "fp4_w4a4_gemm_warpsplit_mrows_bf16", "fp4_repack_b_interleaved_sm120",
           "fp4_w4a4_gemv_warpsplit_interleaved_bf16", "pack_nvfp4_weight_bf16", "quantize_fp4_sfa_mse_fp16",
           "quantize_fp4_sfa_mse_bf16", "quantize_fp4_sfa_bf16_pdl", "aligned_fp4_dim", "quantize_fp4_sfa_padded_bf16", "adopt_modelopt_nvfp4_weight"]
