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


__all__ = ["grouped_nvfp4_gemm_bf16", "grouped_nvfp4_gemm_bf16_offsets", "grouped_workspace"]
