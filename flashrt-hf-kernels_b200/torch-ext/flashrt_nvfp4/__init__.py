"""NVFP4 scale-factor layout helpers (B200 build).

Same functions as the reference package flashrt_nvfp4
(flashrt-nvfp4/torch-ext/flashrt_nvfp4/__init__.py:24-61)."""
from __future__ import annotations

from typing import Optional

import torch

from ._ops import add_op_namespace_prefix, ops


@torch.library.register_fake(add_op_namespace_prefix("nvfp4_sf_linear_to_swizzled"))
def _nvfp4_sf_linear_to_swizzled_fake(scales, out, D, is_sfb=False) -> None:
    if scales.dim() != 2:
        raise RuntimeError("scales must have shape (rows, D / 16)")
    return None


def nvfp4_sf_swizzled_bytes(rows: int, D: int) -> int:
    """Bytes of the swizzled UE4M3 scale buffer of a [rows, D] NVFP4 tensor."""
    if rows <= 0:
        raise ValueError("rows must be positive")
    if D <= 0 or D % 16 != 0:
        raise ValueError("D must be positive and divisible by 16")
    return ((rows + 127) // 128) * ((D // 16 + 3) // 4) * 512


def nvfp4_sf_linear_to_swizzled(scales: torch.Tensor, *, out: Optional[torch.Tensor] = None,
                                is_sfb: bool = False) -> torch.Tensor:
    """linear [rows, D/16] uint8 scales -> flat swizzled buffer (allocated
    zero-filled when `out` is omitted)."""
    if scales.dim() != 2:
        raise ValueError("scales must have shape (rows, D / 16)")
    rows, D = scales.shape[0], scales.shape[1] * 16
    if out is None:
        out = torch.zeros((nvfp4_sf_swizzled_bytes(rows, D),), device=scales.device, dtype=torch.uint8)
    ops.nvfp4_sf_linear_to_swizzled(scales, out, D, is_sfb)
    return out


__all__ = ["nvfp4_sf_linear_to_swizzled", "nvfp4_sf_swizzled_bytes"]
