"""`transformers` integration of the B200 NVFP4 path.

Two levels, both on the structure of a Llama/Qwen-style decoder (`input_layernorm`, `self_attn.{q,k,v,o}_proj`,
`post_attention_layernorm`, `mlp.{gate,up,down}_proj`):

* `FlashRTConfig` / `FlashRTHfQuantizer`: the quantization-backend entry point of the reference's demo
  (demos/space/transformers-qwen3/flashrt_quantizer.py:140-203): every targeted `nn.Linear` becomes an NVFP4
  linear, loaded through `from_pretrained(..., quantization_config=FlashRTConfig(mode="nvfp4"))`.
* `convert_decoder_model(model, fuse=True)`: the same swap plus the fusions the kernels of this library allow:
  each RMSNorm that feeds projections runs as ONE kernel that writes the bf16 result and its NVFP4 form, q/k/v
  (and gate/up) consume that single quantisation instead of re-quantising their input, and the MLP becomes one
  gate/up GEMM with the SwiGLU -> NVFP4 producer in its epilogue followed by the down GEMM.

The module structure transformers expects is kept (no forward of the model is patched): the norm module remembers
the NVFP4 form of the tensor it returned, and a consumer that is handed that very tensor uses it.
"""
from __future__ import annotations

import sys
from pathlib import Path

import torch
from torch import nn

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
import fp4_fused_ops  # noqa: E402
import fp4_gemm  # noqa: E402

from .layers import FlashRTQuantLinear, FusedSwiGLUFFN  # noqa: E402

TARGET_SUFFIXES = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")


class PackedActivation:
    """NVFP4 form of the last tensor a producer returned, recognised by storage, shape and version."""

    def __init__(self):
        self.key = None
        self.packed = self.sfa = None

    def put(self, t: torch.Tensor, packed, sfa):
        self.key = (t.data_ptr(), tuple(t.shape), t._version)
        self.packed, self.sfa = packed, sfa

    def get(self, t: torch.Tensor):
        if self.key is not None and self.key == (t.data_ptr(), tuple(t.shape), t._version):
            return self.packed, self.sfa
        return None


class NormQuant(nn.Module):
    """RMSNorm (plain weight, fp32 statistics) whose single kernel also emits the NVFP4 form of its output."""

    def __init__(self, weight: torch.Tensor, eps: float):
        super().__init__()
        self.register_buffer("weight", weight.detach().to(torch.bfloat16).contiguous(), persistent=False)
        self.variance_epsilon = float(eps)
        self.produced = PackedActivation()

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        shape = hidden_states.shape
        x = hidden_states.to(torch.bfloat16).contiguous().view(-1, shape[-1])
        normed = torch.empty_like(x)
        packed, sfa = fp4_fused_ops.rms_norm_quant_nvfp4(x, self.weight, self.variance_epsilon, normed=normed)
        out = normed.view(shape)
        self.produced.put(out, packed, sfa)
        return out


class SharedInputLinear(FlashRTQuantLinear):
    """NVFP4 linear that uses the producer's quantisation when it is handed the producer's tensor."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.source = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        hit = self.source.get(x) if self.source is not None else None
        if hit is None or self.w_packed.shape[1] * 2 != x.shape[-1]:
            return super().forward(x)
        out = self.forward_packed(*hit)
        return out.view(*x.shape[:-1], self.out_features)


class SharedInputFFN(FusedSwiGLUFFN):
    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.source = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        hit = self.source.get(x) if self.source is not None else None
        if hit is None:
            return super().forward(x)
        return self.forward_packed(*hit).view(*x.shape[:-1], self.down.out_features)


def _shared_linear(linear: nn.Linear, source, mse: bool) -> SharedInputLinear:
    mod = SharedInputLinear(linear.in_features, linear.out_features, linear.bias is not None)
    weight = linear.weight.data.to(torch.bfloat16).contiguous()
    bias = None if linear.bias is None else linear.bias.data.to(torch.bfloat16).contiguous()
    mod.w_packed, mod.w_sfb, mod.bias, _ = fp4_gemm.pack_nvfp4_weight_bf16(weight, bias, mse=mse)
    mod.source = source
    return mod


@torch.no_grad()
def convert_decoder_model(model: nn.Module, *, fuse: bool = True, mse: bool = False, skip=("lm_head",)) -> int:
    """Swap the projections of every decoder layer of `model` (weights already on the GPU) for NVFP4 ones.

    fuse=False: one NVFP4 linear per `nn.Linear` (what the reference's quantizer does).
    fuse=True : additionally norm+quantise in one kernel, one quantisation shared by q/k/v and by gate/up, and the
                MLP as gate/up GEMM with SwiGLU -> NVFP4 epilogue + down GEMM (intermediate size % 128 == 0, SiLU,
                bias-free; other MLPs keep per-linear modules).
    Returns the number of `nn.Linear` modules replaced."""
    replaced = 0
    for layer in [m for m in model.modules() if hasattr(m, "self_attn") and hasattr(m, "mlp")]:
        attn, mlp = layer.self_attn, layer.mlp
        attn_src = mlp_src = None
        if fuse and hasattr(layer, "input_layernorm") and hasattr(layer.input_layernorm, "weight"):
            n = layer.input_layernorm
            layer.input_layernorm = NormQuant(n.weight.data, getattr(n, "variance_epsilon", getattr(n, "eps", 1e-6)))
            attn_src = layer.input_layernorm.produced
        if fuse and hasattr(layer, "post_attention_layernorm") and hasattr(layer.post_attention_layernorm, "weight"):
            n = layer.post_attention_layernorm
            layer.post_attention_layernorm = NormQuant(n.weight.data,
                                                       getattr(n, "variance_epsilon", getattr(n, "eps", 1e-6)))
            mlp_src = layer.post_attention_layernorm.produced
        for name in ("q_proj", "k_proj", "v_proj", "o_proj"):
            lin = getattr(attn, name, None)
            if isinstance(lin, nn.Linear) and not any(s in name for s in skip):
                setattr(attn, name, _shared_linear(lin, attn_src if name != "o_proj" else None, mse))
                replaced += 1
        gate, up, down = (getattr(mlp, n, None) for n in ("gate_proj", "up_proj", "down_proj"))
        if not all(isinstance(l, nn.Linear) for l in (gate, up, down)):
            continue
        silu = getattr(getattr(mlp, "config", None), "hidden_act", "silu") == "silu"
        if (fuse and silu and gate.bias is None and up.bias is None and gate.out_features % 128 == 0
                and gate.in_features % 32 == 0):
            ffn = SharedInputFFN(gate, up, down, mse=mse)
            ffn.source = mlp_src
            layer.mlp = ffn
        else:
            mlp.gate_proj = _shared_linear(gate, mlp_src, mse)
            mlp.up_proj = _shared_linear(up, mlp_src, mse)
            mlp.down_proj = _shared_linear(down, None, mse)
        replaced += 3
    return replaced


# ---- quantization-backend registration (same entry point as the reference's demo) -----------------------------
try:
    from transformers.quantizers import HfQuantizer
    from transformers.quantizers.auto import (AUTO_QUANTIZATION_CONFIG_MAPPING, register_quantization_config,
                                              register_quantizer)
    from transformers.utils.quantization_config import QuantizationConfigMixin
    _HAVE_TRANSFORMERS = True
except Exception:                                                    # transformers absent: conversion API only
    _HAVE_TRANSFORMERS = False

if _HAVE_TRANSFORMERS and "flashrt" not in AUTO_QUANTIZATION_CONFIG_MAPPING:
    @register_quantization_config("flashrt")
    class FlashRTConfig(QuantizationConfigMixin):
        def __init__(self, mode: str = "nvfp4", modules_to_not_convert=None, fuse: bool = True, mse: bool = False,
                     **kwargs):
            if mode != "nvfp4":
                raise ValueError("this build implements mode='nvfp4' only")
            self.quant_method = "flashrt"
            self.mode = mode
            self.fuse = bool(fuse)
            self.mse = bool(mse)
            self.modules_to_not_convert = modules_to_not_convert or []

        def to_dict(self):
            return {"quant_method": "flashrt", "mode": self.mode, "fuse": self.fuse, "mse": self.mse,
                    "modules_to_not_convert": self.modules_to_not_convert}

    @register_quantizer("flashrt")
    class FlashRTHfQuantizer(HfQuantizer):
        requires_calibration = False

        def validate_environment(self, *args, **kwargs):
            if not torch.cuda.is_available():
                raise RuntimeError("FlashRT NVFP4 quantization requires a CUDA GPU (B200, compute capability 10.x).")

        def update_dtype(self, dtype):
            return torch.bfloat16

        def _process_model_before_weight_loading(self, model, **kwargs):
            return model                                          # weights load into the stock nn.Linear modules

        def _process_model_after_weight_loading(self, model, **kwargs):
            cfg = self.quantization_config
            on_gpu = all(p.device.type == "cuda" for p in model.parameters())
            if on_gpu:
                convert_decoder_model(model, fuse=cfg.fuse, mse=cfg.mse,
                                      skip=tuple(cfg.modules_to_not_convert) + ("lm_head",))
            else:
                model._flashrt_pending = cfg                      # call convert_decoder_model after .to("cuda")
            return model

        def param_needs_quantization(self, model, param_name, **kwargs):
            return False

        @property
        def is_serializable(self):
            return False

        @property
        def is_trainable(self):
            return False
elif _HAVE_TRANSFORMERS:
    FlashRTConfig = AUTO_QUANTIZATION_CONFIG_MAPPING["flashrt"]
