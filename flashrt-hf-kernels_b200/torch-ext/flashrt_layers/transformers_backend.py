"""`transformers` integration of the B200 NVFP4 path.

Two levels, both on the structure of a Llama/Qwen-style decoder (`input_layernorm`, `self_attn.{q,k,v,o}_proj`,
`post_attention_layernorm`, `mlp.{gate,up,down}_proj`):

* `FlashRTConfig` / `FlashRTHfQuantizer`: the quantization-backend entry point of the reference's demo
  (demos/space/transformers-qwen3/flashrt_quantizer.py:140-203): every targeted `nn.Linear` becomes an NVFP4
  linear, loaded through `from_pretrained(..., quantization_config=FlashRTConfig(mode="nvfp4"))`.
* `convert_decoder_model(model, fuse=True)`: the same swap plus the fusions the kernels of this library allow:
  - each RMSNorm that feeds projections runs as ONE kernel that writes the bf16 result and its NVFP4 form, and
    q/k/v (and gate/up) consume that single quantisation instead of re-quantising their input;
  - q, k and v run as ONE GEMM over the stacked weight;
  - the MLP becomes one gate/up GEMM with the SwiGLU -> NVFP4 producer in its epilogue followed by the down GEMM;
  - (`fuse_residual=True`, decoder layers of the Llama / Qwen form) the residual stream is carried beside the
    branch output, so that `residual += branch` happens inside the next norm's kernel (the fused
    residual-add + RMSNorm -> NVFP4 producer) instead of in a separate elementwise kernel: once per
    attention block, once per MLP (added by the next layer's input norm, or by the model's final norm).

The module structure transformers expects is kept: the norm module remembers the NVFP4 form of the tensor it
returned, and a consumer that is handed that very tensor uses it.  With `fuse_residual` the tensor a decoder layer
returns is its MLP output and the residual stream travels in a side object until the next norm adds them; hidden
states captured BETWEEN layers (`output_hidden_states`) are therefore not the residual stream: convert with
`fuse_residual=False` when those are needed.
"""
from __future__ import annotations

import sys
import types
from pathlib import Path

import torch
from torch import nn

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
import fp4_fused_ops  # noqa: E402
import fp4_gemm  # noqa: E402
import flashrt_residual_norm_quant as _norm  # noqa: E402

from .layers import FlashRTQuantLinear, FusedSwiGLUFFN  # noqa: E402

TARGET_SUFFIXES = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")
# decoder layers whose forward is `x + attn(norm(x))` then `x + mlp(norm(x))` (checked by name, the forward is replaced)
RESIDUAL_FUSABLE_LAYERS = ("Qwen3DecoderLayer", "Qwen2DecoderLayer", "LlamaDecoderLayer", "MistralDecoderLayer")


def _same_tensor(a: torch.Tensor, b: torch.Tensor) -> bool:
    return a is b or (a.data_ptr() == b.data_ptr() and a.shape == b.shape and a.stride() == b.stride()
                      and a._version == b._version)


class PackedActivation:
    """NVFP4 form of the last tensor a producer returned.  The tensor itself is held (so its storage cannot be
    handed to another tensor while this entry lives) and a consumer's input is recognised by identity, or by
    storage, shape, strides and version for a re-wrapped view of the same data."""

    def __init__(self):
        self.tensor = None
        self.version = -1
        self.packed = self.sfa = None

    def put(self, t: torch.Tensor, packed, sfa):
        self.tensor, self.version = t, t._version
        self.packed, self.sfa = packed, sfa

    def get(self, t: torch.Tensor):
        if self.tensor is not None and self.version == t._version and _same_tensor(self.tensor, t):
            return self.packed, self.sfa
        return None

    def clear(self):
        self.tensor = self.packed = self.sfa = None


class ResidualCarry:
    """The residual stream between a decoder layer that deferred its last `residual + mlp_out` and the norm that
    performs it.  One object per converted model."""

    def __init__(self):
        self.deferred = self.residual = None

    def clear(self):
        self.deferred = self.residual = None

    def put(self, deferred: torch.Tensor, residual: torch.Tensor):
        self.deferred, self.residual = deferred, residual

    def take(self, t: torch.Tensor):
        """the residual that `t` still has to be added to, or None when `t` is a complete hidden state"""
        if self.deferred is None:
            return None
        deferred, residual = self.deferred, self.residual
        self.clear()
        if not _same_tensor(deferred, t):
            raise RuntimeError("the tensor handed to this layer is not the one the previous fused decoder layer "
                               "returned, so its pending residual cannot be applied; convert the model with "
                               "fuse_residual=False when something rewrites hidden states between layers")
        return residual


class NormQuant(nn.Module):
    """RMSNorm (plain or 1 + weight, fp32 statistics) whose single kernel also emits the NVFP4 form of its output;
    `fused` additionally performs `residual += x` in the same kernel."""

    def __init__(self, weight: torch.Tensor, eps: float, one_plus_weight: bool = False):
        super().__init__()
        self.register_buffer("weight", weight.detach().to(torch.bfloat16).contiguous(), persistent=False)
        self.variance_epsilon = float(eps)
        self.one_plus_weight = bool(one_plus_weight)
        self.produced = PackedActivation()

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        shape = hidden_states.shape
        x = hidden_states.to(torch.bfloat16).contiguous().view(-1, shape[-1])
        normed = torch.empty_like(x)
        packed, sfa = fp4_fused_ops.rms_norm_quant_nvfp4(x, self.weight, self.variance_epsilon, normed=normed,
                                                         one_plus_weight=self.one_plus_weight)
        out = normed.view(shape)
        self.produced.put(out, packed, sfa)
        return out

    def fused(self, residual: torch.Tensor, x: torch.Tensor, shape) -> torch.Tensor:
        """residual (rows, dim) bf16 += x in place; returns norm(residual) viewed as `shape` and remembers its NVFP4
        form.  (The norm is taken from the fp32 sum, the residual is stored rounded to bf16.)"""
        normed = torch.empty_like(residual)
        packed, sfa = fp4_fused_ops.residual_add_rms_norm_quant_nvfp4(residual, x, self.weight, self.variance_epsilon,
                                                                      normed=normed)
        out = normed.view(shape)
        self.produced.put(out, packed, sfa)
        return out


class KernelNorm(nn.Module):
    """A plain (or 1 + weight) RMSNorm over the last dimension as ONE kernel, for the norms that feed no NVFP4
    projection: the per-head q / k norms of Qwen3-style attention.  Eager `transformers` runs such a norm as half
    a dozen elementwise kernels with an fp32 intermediate."""

    def __init__(self, weight: torch.Tensor, eps: float, one_plus_weight: bool = False):
        super().__init__()
        w = weight.detach().float()
        self.register_buffer("weight", (1.0 + w if one_plus_weight else w).to(torch.bfloat16).contiguous(), persistent=False)
        self.variance_epsilon = float(eps)

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        shape = hidden_states.shape
        x = hidden_states.to(torch.bfloat16).contiguous().view(-1, shape[-1])
        return _norm.rms_norm_bf16(x, self.weight, self.variance_epsilon).view(shape)


class StackedHeadNorm(KernelNorm):
    """q_norm / k_norm of an attention whose q, k and v come from one `StackedProjection`: when q_norm is called on
    the q slice of the stacked output, ONE kernel normalises the q heads and the k heads in place in that buffer;
    k_norm, called next on the k slice of the same buffer, returns it as it is.  Any other input (another tensor,
    another order) takes the plain one-kernel norm of `KernelNorm`."""

    def __init__(self, weight, eps, one_plus_weight, stacked, is_q: bool):
        super().__init__(weight, eps, one_plus_weight)
        self.__dict__["stacked"] = stacked                     # not a submodule: it lives at q_proj
        self.is_q = is_q
        self.__dict__["partner"] = None                        # the other norm of the pair

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        st, other = self.stacked, self.partner
        buf = st.last_out
        head_dim = self.weight.numel()
        if self.is_q:
            st.__dict__["heads_normed"] = None
            wq, wk = st.widths[0], st.widths[1]
            if (buf is not None and other is not None and buf.is_contiguous() and hidden_states.shape[-1] == head_dim
                    and hidden_states.data_ptr() == buf.data_ptr() and hidden_states.numel() == buf.numel() // buf.shape[-1] * wq
                    and wq % head_dim == 0 and wk % head_dim == 0 and other.weight.numel() == head_dim
                    and other.variance_epsilon == self.variance_epsilon and head_dim in (64, 128, 256, 512)):
                _norm.rms_norm_heads_bf16_(buf.view(-1, buf.shape[-1]), self.weight, wq // head_dim, other.weight,
                                           wk // head_dim, head_dim, self.variance_epsilon)
                st.__dict__["heads_normed"] = buf
                return hidden_states
            return super().forward(hidden_states)
        done = st.__dict__.get("heads_normed")
        if done is not None and hidden_states.data_ptr() == done.data_ptr() + 2 * st.widths[0]:
            st.__dict__["heads_normed"] = None
            return hidden_states
        return super().forward(hidden_states)


class FinalNorm(nn.Module):
    """The model's last norm: adds the pending residual of the last fused decoder layer in the norm kernel."""

    def __init__(self, weight: torch.Tensor, eps: float, carry: ResidualCarry):
        super().__init__()
        self.register_buffer("weight", weight.detach().to(torch.bfloat16).contiguous(), persistent=False)
        self.variance_epsilon = float(eps)
        self.carry = carry

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        shape = hidden_states.shape
        x = hidden_states.to(torch.bfloat16).contiguous().view(-1, shape[-1])
        residual = self.carry.take(hidden_states)
        if residual is None:
            return _norm.rms_norm_bf16(x, self.weight, self.variance_epsilon).view(shape)
        out = _norm.residual_add_rms_norm_bf16(residual, x, self.weight, self.variance_epsilon)
        return out.view(shape)


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
        return out.reshape(*x.shape[:-1], self.out_features)


class StackedProjection(SharedInputLinear):
    """q, k and v as ONE GEMM over the weights stacked along the output axis.  This module stands where `q_proj`
    was; `k_proj` and `v_proj` become `ProjectionSlice`s that return their columns of the result computed here
    (attention calls q_proj, k_proj, v_proj in that order on one tensor)."""

    def __init__(self, in_features, widths, bias):
        super().__init__(in_features, sum(widths), bias)
        self.widths = tuple(widths)
        self.last_in = None
        self.last_out = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out = super().forward(x)
        self.last_in, self.last_out = x, out
        return out[..., :self.widths[0]]

    def piece(self, x: torch.Tensor, index: int) -> torch.Tensor:
        if self.last_in is None or not _same_tensor(self.last_in, x):
            self.forward(x)                                    # called out of order: compute for this input
        lo = sum(self.widths[:index])
        out = self.last_out[..., lo:lo + self.widths[index]]
        if index == len(self.widths) - 1:
            self.last_in = self.last_out = None
        return out


class ProjectionSlice(nn.Module):
    def __init__(self, stacked: StackedProjection, index: int):
        super().__init__()
        self.__dict__["stacked"] = stacked                     # not a submodule: it already lives at q_proj
        self.index = index
        self.out_features = stacked.widths[index]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.stacked.piece(x, self.index)


class SharedInputFFN(FusedSwiGLUFFN):
    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.source = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        hit = self.source.get(x) if self.source is not None else None
        if hit is None:
            return super().forward(x)
        return self.forward_packed(*hit).reshape(*x.shape[:-1], self.down.out_features)


def _shared_linear(linear: nn.Linear, source, mse: bool) -> SharedInputLinear:
    mod = SharedInputLinear(linear.in_features, linear.out_features, linear.bias is not None)
    weight = linear.weight.data.to(torch.bfloat16).contiguous()
    bias = None if linear.bias is None else linear.bias.data.to(torch.bfloat16).contiguous()
    mod.w_packed, mod.w_sfb, mod.bias, _ = fp4_gemm.pack_nvfp4_weight_bf16(weight, bias, mse=mse)
    mod.source = source
    return mod


def _stacked_qkv(q: nn.Linear, k: nn.Linear, v: nn.Linear, source, mse: bool) -> StackedProjection:
    has_bias = q.bias is not None
    mod = StackedProjection(q.in_features, (q.out_features, k.out_features, v.out_features), has_bias)
    weight = torch.cat([l.weight.data for l in (q, k, v)], dim=0).to(torch.bfloat16).contiguous()
    bias = torch.cat([l.bias.data for l in (q, k, v)]).to(torch.bfloat16).contiguous() if has_bias else None
    mod.w_packed, mod.w_sfb, mod.bias, _ = fp4_gemm.pack_nvfp4_weight_bf16(weight, bias, mse=mse)
    mod.source = source
    return mod


def _norm_semantics(norm: nn.Module):
    """How `norm` uses its weight, found by running it: "plain" (x_hat * w), "one_plus" (x_hat * (1 + w)) or None
    when it is neither (an offset, a bias, another statistic): such a norm is left as it is."""
    w = getattr(norm, "weight", None)
    if w is None or w.dim() != 1:
        return None
    eps = getattr(norm, "variance_epsilon", getattr(norm, "eps", None))
    if eps is None:
        return None
    g = torch.Generator(device=w.device).manual_seed(1)
    x = torch.randn(4, w.numel(), generator=g, device=w.device, dtype=torch.float32)
    xh = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    with torch.no_grad():
        got = norm(x.to(torch.bfloat16)).float()
    xb = x.to(torch.bfloat16).float()
    xh = xb * torch.rsqrt(xb.pow(2).mean(-1, keepdim=True) + eps)
    for name, scale in (("plain", w.detach().float()), ("one_plus", 1.0 + w.detach().float())):
        if (got - xh * scale).abs().max() <= 0.05 * (xh * scale).abs().max().clamp_min(1e-3):
            return name
    return None


def _fused_decoder_forward(self, hidden_states, attention_mask=None, position_ids=None, past_key_values=None,
                           use_cache=False, position_embeddings=None, **kwargs):
    """Forward of a Llama / Qwen decoder layer with both residual additions inside the norm kernels.  Returns the
    MLP output; the residual stream it belongs to waits in `self._frt_carry` for the next norm."""
    carry = self._frt_carry
    shape = hidden_states.shape
    pending = carry.take(hidden_states)
    x = hidden_states.to(torch.bfloat16).contiguous().view(-1, shape[-1])
    if pending is None:
        residual = x.clone()                                   # this layer owns and updates the residual stream
        normed = self.input_layernorm(hidden_states)
    else:
        residual = pending
        normed = self.input_layernorm.fused(residual, x, shape)
    attn_out, _ = self.self_attn(hidden_states=normed, attention_mask=attention_mask, position_ids=position_ids,
                                 past_key_values=past_key_values, use_cache=use_cache,
                                 position_embeddings=position_embeddings, **kwargs)
    a = attn_out.to(torch.bfloat16).contiguous().view(-1, shape[-1])
    normed = self.post_attention_layernorm.fused(residual, a, shape)
    out = self.mlp(normed)
    carry.put(out, residual)
    return out


@torch.no_grad()
def convert_decoder_model(model: nn.Module, *, fuse: bool = True, fuse_residual: bool = True, mse: bool = False,
                          skip=("lm_head",)) -> int:
    """Swap the projections of every decoder layer of `model` (weights already on the GPU) for NVFP4 ones.

    fuse=False: one NVFP4 linear per `nn.Linear` (what the reference's quantizer does).
    fuse=True : additionally norm+quantise in one kernel, one quantisation shared by q/k/v and by gate/up, q/k/v as
                one GEMM, and the MLP as gate/up GEMM with SwiGLU -> NVFP4 epilogue + down GEMM (intermediate size
                % 128 == 0, SiLU, bias-free; other MLPs keep per-linear modules); with fuse_residual the residual
                additions move into the norm kernels (decoder layers of the Llama / Qwen form only).
    `skip`: module names that stay as they are, matched against the qualified name (`model.layers.3.mlp.up_proj`),
    any dotted suffix of it (`mlp.up_proj`, `up_proj`) or a prefix (`model.layers.3`).
    Returns the number of `nn.Linear` modules replaced."""
    names = {id(m): n for n, m in model.named_modules()}

    def skipped(mod) -> bool:
        q = names.get(id(mod), "")
        return any(q == s or q.endswith("." + s) or q.startswith(s + ".") for s in skip)

    replaced = 0
    carry = ResidualCarry()
    fused_layers = []
    for layer in [m for m in model.modules() if hasattr(m, "self_attn") and hasattr(m, "mlp")]:
        attn, mlp = layer.self_attn, layer.mlp
        attn_src = mlp_src = None
        converted_norms = 0
        for attr in ("input_layernorm", "post_attention_layernorm"):
            n = getattr(layer, attr, None)
            kind = _norm_semantics(n) if (fuse and n is not None and not skipped(n)) else None
            if kind is None:
                continue
            nq = NormQuant(n.weight.data, getattr(n, "variance_epsilon", getattr(n, "eps", 1e-6)), kind == "one_plus")
            setattr(layer, attr, nq)
            converted_norms += 1
            if attr == "input_layernorm":
                attn_src = nq.produced
            else:
                mlp_src = nq.produced
        for attr in ("q_norm", "k_norm"):             # per-head norms (Qwen3): one kernel each instead of eager arithmetic
            n = getattr(attn, attr, None)
            kind = _norm_semantics(n) if (fuse and n is not None and not skipped(n)) else None
            if kind is not None and n.weight.numel() % 16 == 0:
                setattr(attn, attr, KernelNorm(n.weight.data, getattr(n, "variance_epsilon", getattr(n, "eps", 1e-6)),
                                               kind == "one_plus"))
        q, k, v, o = (getattr(attn, n, None) for n in ("q_proj", "k_proj", "v_proj", "o_proj"))
        qkv_ok = all(isinstance(l, nn.Linear) and not skipped(l) for l in (q, k, v))
        if (fuse and qkv_ok and len({l.bias is None for l in (q, k, v)}) == 1
                and q.in_features == k.in_features == v.in_features):
            attn.q_proj = _stacked_qkv(q, k, v, attn_src, mse)
            attn.k_proj = ProjectionSlice(attn.q_proj, 1)
            attn.v_proj = ProjectionSlice(attn.q_proj, 2)
            replaced += 3
            qn, kn = getattr(attn, "q_norm", None), getattr(attn, "k_norm", None)
            if type(qn) is KernelNorm and type(kn) is KernelNorm:    # one kernel for both head norms
                sq = StackedHeadNorm(qn.weight, qn.variance_epsilon, False, attn.q_proj, True)
                sk = StackedHeadNorm(kn.weight, kn.variance_epsilon, False, attn.q_proj, False)
                sq.__dict__["partner"], sk.__dict__["partner"] = sk, sq
                attn.q_norm, attn.k_norm = sq, sk
        else:
            for name, lin in (("q_proj", q), ("k_proj", k), ("v_proj", v)):
                if isinstance(lin, nn.Linear) and not skipped(lin):
                    setattr(attn, name, _shared_linear(lin, attn_src, mse))
                    replaced += 1
        if isinstance(o, nn.Linear) and not skipped(o):
            attn.o_proj = _shared_linear(o, None, mse)
            replaced += 1
        gate, up, down = (getattr(mlp, n, None) for n in ("gate_proj", "up_proj", "down_proj"))
        if all(isinstance(l, nn.Linear) for l in (gate, up, down)):
            silu = getattr(getattr(mlp, "config", None), "hidden_act", "silu") == "silu"
            none_skipped = not any(skipped(l) for l in (gate, up, down)) and not skipped(mlp)
            if (fuse and silu and none_skipped and gate.bias is None and up.bias is None
                    and gate.out_features % 128 == 0 and gate.in_features % 32 == 0):
                ffn = SharedInputFFN(gate, up, down, mse=mse)
                ffn.source = mlp_src
                layer.mlp = ffn
                replaced += 3
            else:
                for name, lin, src in (("gate_proj", gate, mlp_src), ("up_proj", up, mlp_src), ("down_proj", down, None)):
                    if not skipped(lin) and not skipped(mlp):
                        setattr(mlp, name, _shared_linear(lin, src, mse))
                        replaced += 1
        if (fuse and fuse_residual and converted_norms == 2 and type(layer).__name__ in RESIDUAL_FUSABLE_LAYERS
                and not layer.input_layernorm.one_plus_weight):
            fused_layers.append(layer)
    # The residual stream may only be deferred when the module that runs after the LAST such layer can add it:
    # all layers of one stack are fused and the stack's final norm is a plain RMSNorm right beside them.
    for parent in model.modules():
        stack = getattr(parent, "layers", None)
        final = getattr(parent, "norm", None)
        if not isinstance(stack, nn.ModuleList) or final is None or len(stack) == 0:
            continue
        if not all(any(l is f for f in fused_layers) for l in stack) or _norm_semantics(final) != "plain":
            continue
        parent.norm = FinalNorm(final.weight.data, getattr(final, "variance_epsilon", getattr(final, "eps", 1e-6)), carry)
        for i, l in enumerate(stack):
            l._frt_carry = carry
            l._frt_first = i == 0
            l.forward = types.MethodType(_fused_decoder_forward, l)
        stack[0].register_forward_pre_hook(lambda mod, args: carry.clear())     # a new pass starts clean
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
