"""Layer classes for `kernels.kernelize` / quantisation back-ends.

RMSNorm follows the reference's kernelize layer
(demos/space/transformers-qwen3/flashrt_layers/build/torch-universal/flashrt_layers/layers.py:27-35):
`forward(self, hidden_states)` reads `self.weight` and `self.variance_epsilon`.
FlashRTQuantLinear follows demos/space/transformers-qwen3/flashrt_quantizer.py:30-109
(weights packed once at bind time; forward = quantise activations + A4W4 GEMM).
FusedNormLinear is the seam the B200 build fuses: one producer launch feeds
any number of linears that share the normalised activation."""
from __future__ import annotations

import sys
from pathlib import Path

import torch
from torch import nn

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
import fp4_fused_ops  # noqa: E402
import fp4_gemm  # noqa: E402
import flashrt_residual_norm_quant as _norm  # noqa: E402


class RMSNorm(nn.Module):
    weight: torch.Tensor
    variance_epsilon: float

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        shape = hidden_states.shape
        x = hidden_states.to(torch.bfloat16).contiguous().view(-1, shape[-1])
        out = _norm.rms_norm_bf16(x, self.weight.to(torch.bfloat16).contiguous(), float(self.variance_epsilon))
        return out.view(shape).to(hidden_states.dtype)


class FlashRTQuantLinear(nn.Module):
    """NVFP4 A4W4 linear with bf16 output; weights are packed in `from_linear`."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.register_buffer("w_packed", torch.empty(0, dtype=torch.uint8), persistent=False)
        self.register_buffer("w_sfb", torch.empty(0, dtype=torch.uint8), persistent=False)
        self.register_buffer("bias", None, persistent=False)

    @classmethod
    def from_linear(cls, linear: nn.Linear, *, mse: bool = False) -> "FlashRTQuantLinear":
        mod = cls(linear.in_features, linear.out_features, linear.bias is not None)
        weight = linear.weight.data.to(torch.bfloat16).contiguous()
        bias = None if linear.bias is None else linear.bias.data.to(torch.bfloat16).contiguous()
        packed, sfb, bias, _ = fp4_gemm.pack_nvfp4_weight_bf16(weight, bias, mse=mse)
        mod.w_packed, mod.w_sfb, mod.bias = packed, sfb, bias
        return mod

    def forward_packed(self, a_packed: torch.Tensor, sfa: torch.Tensor) -> torch.Tensor:
        if self.bias is not None:
            out = fp4_gemm.nvfp4_gemm_bias_bf16(a_packed, self.w_packed, sfa, self.w_sfb, self.bias)
        else:
            out = fp4_gemm.nvfp4_gemm_bf16(a_packed, self.w_packed, sfa, self.w_sfb)
        return out[:, :self.out_features] if out.shape[1] != self.out_features else out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).to(torch.bfloat16).contiguous()
        pad = self.w_packed.shape[1] * 2 - x2.shape[1]
        if pad:
            x2 = torch.nn.functional.pad(x2, (0, pad))
        a_packed, sfa = fp4_gemm.quantize_fp4_sfa_bf16(x2)
        return self.forward_packed(a_packed, sfa).view(*shape[:-1], self.out_features)


class FusedSwiGLUFFN(nn.Module):
    """down(silu(gate(x)) * up(x)) on NVFP4 activations: the gate/up projection runs as ONE
    GEMM over the stacked [gate ; up] weight whose epilogue applies SwiGLU and quantises to
    NVFP4, and the down projection consumes that directly.  Intermediate size must be a
    multiple of 128 and the projections bias-free (the Llama / Qwen FFN)."""

    def __init__(self, gate: nn.Linear, up: nn.Linear, down: nn.Linear, *, mse: bool = False):
        super().__init__()
        assert gate.bias is None and up.bias is None, "gate/up projections must be bias-free"
        assert gate.out_features == up.out_features == down.in_features and gate.out_features % 128 == 0
        assert gate.in_features % 32 == 0
        stacked = torch.cat([gate.weight.data, up.weight.data], dim=0).to(torch.bfloat16).contiguous()
        quantize = fp4_gemm.quantize_fp4_sfa_mse_bf16 if mse else fp4_gemm.quantize_fp4_sfa_bf16
        packed, sfb = quantize(stacked, is_sfb=True)
        self.register_buffer("w_gate_up", packed, persistent=False)
        self.register_buffer("w_gate_up_sfb", sfb, persistent=False)
        self.down = FlashRTQuantLinear.from_linear(down, mse=mse)

    def forward_packed(self, a_packed: torch.Tensor, sfa: torch.Tensor) -> torch.Tensor:
        h_packed, h_sfa = fp4_gemm.nvfp4_gemm_swiglu_nvfp4_bf16(a_packed, self.w_gate_up, sfa, self.w_gate_up_sfb)
        return self.down.forward_packed(h_packed, h_sfa)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).to(torch.bfloat16).contiguous()
        a_packed, sfa = fp4_gemm.quantize_fp4_sfa_bf16(x2)
        return self.forward_packed(a_packed, sfa).view(*shape[:-1], self.down.out_features)


class FusedNormLinear(nn.Module):
    """residual += x; RMSNorm; NVFP4-quantise once; feed every linear in `linears`."""

    def __init__(self, norm_weight: torch.Tensor, eps: float, linears):
        super().__init__()
        self.register_buffer("norm_weight", norm_weight.to(torch.bfloat16).contiguous(), persistent=False)
        self.eps = float(eps)
        self.linears = nn.ModuleList(linears)

    def forward(self, residual: torch.Tensor, x: torch.Tensor):
        packed, sfa = fp4_fused_ops.residual_add_rms_norm_quant_nvfp4_swizzled_bf16(
            residual, x, self.norm_weight, self.eps)
        return [lin.forward_packed(packed, sfa) for lin in self.linears]
