"""MoE routing members of the reference's transformer-fused-ops package (B200 build): the
exact top-k router and the deterministic weighted un-permute, with the reference's names and
return conventions (transformer-fused-ops/torch-ext/transformer_fused_ops/__init__.py:358-396).
The router also takes a (tokens, n_experts) batch."""
from __future__ import annotations

from typing import Optional

import torch

from ._ops import add_op_namespace_prefix, ops


def _topk_fake(logits, out_idx, out_val, k) -> None:
    if logits.dim() not in (1, 2):
        raise RuntimeError("logits must have shape (n_experts,) or (tokens, n_experts)")
    want = (k,) if logits.dim() == 1 else (logits.shape[0], k)
    if tuple(out_idx.shape) != want or tuple(out_val.shape) != want:
        raise RuntimeError("topk outputs must have shape (k,) or (tokens, k)")
    return None


torch.library.register_fake(add_op_namespace_prefix("nexn2_router_topk_bf16"))(_topk_fake)
torch.library.register_fake(add_op_namespace_prefix("router_topk_bf16"))(_topk_fake)


@torch.library.register_fake(add_op_namespace_prefix("moe_weighted_sum_bf16_to_fp32"))
def _weighted_sum_fake(expert_output, row_indices, router_weight, out) -> None:
    if row_indices.dim() != 2 or router_weight.shape != row_indices.shape:
        raise RuntimeError("row_indices and router_weight must have shape (tokens, topk)")
    if out.dim() != 2 or out.shape[0] != row_indices.shape[0]:
        raise RuntimeError("out must have shape (tokens, hidden)")
    return None


def _alloc_topk(logits, k):
    shape = (k,) if logits.dim() == 1 else (logits.shape[0], k)
    return (torch.empty(shape, device=logits.device, dtype=torch.int32),
            torch.empty(shape, device=logits.device, dtype=torch.float32))


def router_topk_bf16(logits, k: int = 8, *, out_idx=None, out_val=None):
    """Exact top-k expert logits (descending) and indices per routing row; equal logits come
    out in the reference kernel's order."""
    if out_idx is None or out_val is None:
        out_idx, out_val = _alloc_topk(logits, k)
    ops.router_topk_bf16(logits, out_idx, out_val, int(k))
    return out_idx, out_val


@torch.library.register_fake(add_op_namespace_prefix("router_topk_softmax_bf16"))
def _topk_softmax_fake(logits, out_idx, out_val, out_weight, k) -> None:
    if logits.dim() != 2 or tuple(out_idx.shape) != (logits.shape[0], k):
        raise RuntimeError("logits must be (tokens, n_experts) and the outputs (tokens, k)")
    return None


def router_topk_softmax_bf16(logits, k: int = 8):
    """Top-k router that also returns the routing weights (softmax over the k selected logits) from the same
    kernel: ``(idx, val, weight)``, each (tokens, k)."""
    idx, val = _alloc_topk(logits, k)
    weight = torch.empty_like(val)
    ops.router_topk_softmax_bf16(logits, idx, val, weight, int(k))
    return idx, val, weight


def nexn2_router_topk_bf16(logits, k: int = 8, *, out_idx=None, out_val=None):
    if out_idx is None or out_val is None:
        out_idx, out_val = _alloc_topk(logits, k)
    ops.nexn2_router_topk_bf16(logits, out_idx, out_val, int(k))
    return out_idx, out_val


def moe_weighted_sum_bf16_to_fp32(expert_output, row_indices, router_weight, *, hidden: Optional[int] = None,
                                  out: Optional[torch.Tensor] = None):
    """Gather routed BF16 expert rows and reduce them in FP32, slots in order."""
    hidden = expert_output.shape[1] if hidden is None else int(hidden)
    if out is None:
        out = torch.empty((row_indices.shape[0], hidden), device=expert_output.device, dtype=torch.float32)
    ops.moe_weighted_sum_bf16_to_fp32(expert_output, row_indices, router_weight, out)
    return out


__all__ = ["router_topk_bf16", "router_topk_softmax_bf16", "nexn2_router_topk_bf16", "moe_weighted_sum_bf16_to_fp32"]
