"""Grouped NVFP4 MoE GEMM (B200 build).

`grouped_nvfp4_gemm_bf16` keeps the reference's tile_expert signature
(grouped-moe-gemm/torch-ext/grouped_moe_gemm/__init__.py:64-109);
`grouped_nvfp4_gemm_bf16_offsets` is the additive form driven by a per-expert
offsets array over expert-sorted rows."""
from __future__ import annotations

import torch

from ._ops import add_op_namespace_prefix, ops


@torch.library.register_fake(add_op_namespace_prefix("grouped_nvfp4_gemm_bf16_out"))
def _out_fake(input, weight, input_scale, weight_scale, alpha, tile_expert, tile_rows, input_scale_stride,
              weight_stride, weight_scale_stride, output) -> None:
    return None


@torch.library.register_fake(add_op_namespace_prefix("grouped_nvfp4_gemm_bf16_offsets_out"))
def _offsets_out_fake(input, weight, input_scale, weight_scale, alpha, expert_offsets, workspace, output) -> None:
    return None


@torch.library.custom_op(add_op_namespace_prefix("_grouped_nvfp4_gemm_bf16"), mutates_args=(), device_types="cuda")
def _compileable(input: torch.Tensor, weight: torch.Tensor, input_scale: torch.Tensor, weight_scale: torch.Tensor,
                 alpha: torch.Tensor, tile_expert: torch.Tensor, tile_rows: int, input_scale_stride: int,
                 weight_stride: int, weight_scale_stride: int) -> torch.Tensor:
    output = torch.empty((input.shape[0], weight.shape[1]), device=input.device, dtype=torch.bfloat16)
    ops.grouped_nvfp4_gemm_bf16_out(input, weight, input_scale, weight_scale, alpha, tile_expert, tile_rows,
                                    input_scale_stride, weight_stride, weight_scale_stride, output)
    return output


@torch.library.register_fake(add_op_namespace_prefix("_grouped_nvfp4_gemm_bf16"))
def _fake(input, weight, input_scale, weight_scale, alpha, tile_expert, tile_rows, input_scale_stride, weight_stride,
          weight_scale_stride):
    if input.ndim != 2 or weight.ndim != 3:
        raise RuntimeError("invalid grouped GEMM tensor shapes")
    return torch.empty((input.shape[0], weight.shape[1]), device=input.device, dtype=torch.bfloat16)


def grouped_nvfp4_gemm_bf16(input, weight, input_scale, weight_scale, alpha, tile_expert, *, tile_rows,
                            input_scale_stride=0, weight_stride=None, weight_scale_stride=None, out=None):
    """Expert-selected packed NVFP4 GEMM tiles with BF16 output: tile t of
    `tile_rows` rows uses expert tile_expert[t]; negative entries skip the tile."""
    if weight_stride is None:
        weight_stride = weight[0].numel()
    if weight_scale_stride is None:
        weight_scale_stride = weight_scale[0].numel()
    if out is None:
        return _compileable(input, weight, input_scale, weight_scale, alpha, tile_expert, int(tile_rows),
                            int(input_scale_stride), int(weight_stride), int(weight_scale_stride))
    ops.grouped_nvfp4_gemm_bf16_out(input, weight, input_scale, weight_scale, alpha, tile_expert, int(tile_rows),
                                    int(input_scale_stride), int(weight_stride), int(weight_scale_stride), out)
    return out


def grouped_workspace(rows: int, experts: int, device) -> torch.Tensor:
    """Scratch buffer the offsets-driven op needs (allocate once, reuse)."""
    return torch.empty((int(ops.grouped_nvfp4_gemm_workspace_size(int(rows), int(experts))),), device=device,
                       dtype=torch.uint8)


def grouped_nvfp4_gemm_bf16_offsets(input, weight, input_scale, weight_scale, alpha, expert_offsets, *,
                                    workspace=None, out=None):
    """Rows are expert-sorted; expert e owns rows [expert_offsets[e], expert_offsets[e+1])."""
    if out is None:
        out = torch.empty((input.shape[0], weight.shape[1]), device=input.device, dtype=torch.bfloat16)
    if workspace is None:
        workspace = grouped_workspace(input.shape[0], weight.shape[0], input.device)
    ops.grouped_nvfp4_gemm_bf16_offsets_out(input, weight, input_scale, weight_scale, alpha, expert_offsets,
                                            workspace, out)
    return out


@torch.library.register_fake(add_op_namespace_prefix("moe_route_plan"))
def _route_plan_fake(topk_idx, n_experts, expert_offsets, row_of_pair, token_of_row) -> None:
    if topk_idx.dim() != 2 or expert_offsets.numel() != n_experts + 1:
        raise RuntimeError("topk_idx must be (tokens, topk) and expert_offsets must have n_experts + 1 elements")
    return None


@torch.library.register_fake(add_op_namespace_prefix("moe_gather_nvfp4"))
def _gather_fake(packed, sfa, token_of_row, out_packed, out_sfa) -> None:
    if packed.dim() != 2 or out_packed.dim() != 2 or packed.shape[1] != out_packed.shape[1]:
        raise RuntimeError("packed and out_packed must be matrices with the same packed K")
    return None


def moe_route_plan(topk_idx, n_experts: int, *, expert_offsets=None, row_of_pair=None, token_of_row=None):
    """Stable sort of the (token, slot) routing pairs by expert, on the device.

    Returns ``(expert_offsets [n_experts + 1], row_of_pair [tokens, topk], token_of_row [tokens * topk])``:
    the offsets drive :func:`grouped_nvfp4_gemm_bf16_offsets`, ``token_of_row`` the gather into
    expert order, ``row_of_pair`` the weighted un-permute.  (The reference leaves this stage to
    the caller: grouped-moe-gemm/README.md:13-16.)"""
    dev = topk_idx.device
    n = topk_idx.numel()
    if expert_offsets is None:
        expert_offsets = torch.empty((n_experts + 1,), device=dev, dtype=torch.int32)
    if row_of_pair is None:
        row_of_pair = torch.empty(tuple(topk_idx.shape), device=dev, dtype=torch.int32)
    if token_of_row is None:
        token_of_row = torch.empty((n,), device=dev, dtype=torch.int32)
    ops.moe_route_plan(topk_idx, int(n_experts), expert_offsets, row_of_pair, token_of_row)
    return expert_offsets, row_of_pair, token_of_row


def moe_gather_nvfp4(packed, sfa, token_of_row, *, out_packed=None, out_sfa=None):
    """NVFP4 rows (packed + swizzled scales) gathered into expert-sorted order."""
    from flashrt_b200_core import alloc_fp4
    rows = token_of_row.numel()
    if out_packed is None or out_sfa is None:
        out_packed, out_sfa = alloc_fp4(rows, packed.shape[1] * 2, packed.device)
    ops.moe_gather_nvfp4(packed, sfa, token_of_row, out_packed, out_sfa)
    return out_packed, out_sfa


@torch.library.register_fake(add_op_namespace_prefix("moe_quantize_scatter_nvfp4"))
def _quantize_scatter_fake(x, row_of_pair, out_packed, out_sfa) -> None:
    if x.dim() != 2 or row_of_pair.dim() != 2 or row_of_pair.shape[0] != x.shape[0]:
        raise RuntimeError("x must be (tokens, K) and row_of_pair (tokens, topk)")
    return None


def moe_quantize_scatter_nvfp4(x, row_of_pair, *, out_packed=None, out_sfa=None):
    """bf16 token rows quantised to NVFP4 straight into expert-sorted order (quantise + gather in one pass)."""
    from flashrt_b200_core import alloc_fp4
    if out_packed is None or out_sfa is None:
        out_packed, out_sfa = alloc_fp4(row_of_pair.numel(), x.shape[1], x.device)
    ops.moe_quantize_scatter_nvfp4(x, row_of_pair, out_packed, out_sfa)
    return out_packed, out_sfa


__all__ = ["grouped_nvfp4_gemm_bf16", "grouped_nvfp4_gemm_bf16_offsets", "grouped_workspace", "moe_route_plan",
           "moe_gather_nvfp4", "moe_quantize_scatter_nvfp4"]
