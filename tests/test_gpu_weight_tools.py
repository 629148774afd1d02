"""Bind-time weight tools: MSE scale-search packer (bytes equal to the reference's CUDA kernel and
to the CPU oracle), padded packing, and the layer modules built on them."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from tests.gpu_common import DEV, O, alloc_fp4, capi, randn_bf16, ref_lib, sf_linear  # noqa: E402

P = capi.ptr


def st():
    return capi.stream_ptr()


@pytest.mark.parametrize("rows,dim,scale,dtype", [(64, 256, 0.02, torch.bfloat16), (130, 4096, 1.0, torch.bfloat16),
                                                   (7, 512, 0.5, torch.float16), (257, 1024, 3.0, torch.float16)])
def test_mse_packer_bit_exact(rows, dim, scale, dtype):
    g = torch.Generator().manual_seed(rows + dim)
    x = (torch.randn(rows, dim, generator=g) * scale).to(dtype)
    x[0, :16] = 0
    x[0, 16:32] = 2.0 ** -13
    dx = x.to(DEV)
    packed, sf = alloc_fp4(rows, dim)
    capi.check(capi.lib().frt_nvfp4_quantize_mse(P(dx), 0 if dtype == torch.bfloat16 else 1, P(packed), P(sf), rows,
                                                 dim, st()))
    ref = ref_lib()
    if ref is not None:
        rp, rs = alloc_fp4(rows, dim)
        fn = ref.ref_quantize_mse_bf16 if dtype == torch.bfloat16 else ref.ref_quantize_mse_fp16
        assert fn(P(dx), P(rp), P(rs), rows, dim, st()) == 0
        torch.cuda.synchronize()
        assert torch.equal(rp, packed) and torch.equal(rs, sf)
    want_p, want_s = O.quantize_nvfp4_mse(x.float().numpy())
    np.testing.assert_array_equal(sf_linear(sf, rows, dim), want_s)
    np.testing.assert_array_equal(packed.cpu().numpy(), want_p)
    # the reference's acceptance check (fp4-gemm/tests/test_fp4_gemm.py:1624-1643): never worse than round-to-nearest
    rtn_p, rtn_s = O.quantize_nvfp4(x.float().numpy())
    err = lambda p, s: float(((O.dequantize_nvfp4(p, s) - x.float().numpy()) ** 2).mean())
    assert err(want_p, want_s) <= err(rtn_p, rtn_s) + 1e-8


def test_padded_pack_and_layers():
    import fp4_gemm
    from flashrt_layers import FlashRTQuantLinear, FusedSwiGLUFFN
    assert fp4_gemm.aligned_fp4_dim(4304) == 4320          # fp4-gemm/tests/test_fp4_gemm.py:1703-1711
    w = randn_bf16((72, 4304), 5, 0.05).to(DEV)
    b = randn_bf16((72,), 6).to(DEV)
    packed, sfb, bias, (n, k) = fp4_gemm.pack_nvfp4_weight_bf16(w, b, mse=True)
    assert packed.shape == (96, 2160) and bias.shape == (96,) and (n, k) == (72, 4304)
    assert torch.equal(bias[:72], b) and not bias[72:].any()
    p2, s2, logical = fp4_gemm.quantize_fp4_sfa_padded_bf16(w)
    assert p2.shape == (72, 2160) and logical == 4304

    torch.manual_seed(0)
    lin = torch.nn.Linear(4304, 72, bias=True, device=DEV, dtype=torch.bfloat16)
    q = FlashRTQuantLinear.from_linear(lin)
    x = randn_bf16((33, 4304), 8).to(DEV)
    got, ref = q(x), lin(x)
    rel = ((got.float() - ref.float()).norm() / ref.float().norm()).item()
    assert got.shape == ref.shape and rel < 0.2        # A4W4 against the unquantised layer (about 0.14 expected)

    gate = torch.nn.Linear(256, 384, bias=False, device=DEV, dtype=torch.bfloat16)
    up = torch.nn.Linear(256, 384, bias=False, device=DEV, dtype=torch.bfloat16)
    down = torch.nn.Linear(384, 256, bias=False, device=DEV, dtype=torch.bfloat16)
    ffn = FusedSwiGLUFFN(gate, up, down)
    x = randn_bf16((200, 256), 9).to(DEV)
    got = ffn(x)
    # the same chain with separate kernels gives the same bytes
    a_p, a_s = fp4_gemm.quantize_fp4_sfa_bf16(x)
    import fp4_fused_ops
    merged = fp4_gemm.nvfp4_gemm_bf16(a_p, ffn.w_gate_up, a_s, ffn.w_gate_up_sfb)
    h_p, h_s = fp4_fused_ops.silu_mul_quantize_fp4_sfa_bf16(merged)
    want = ffn.down.forward_packed(h_p, h_s)
    assert torch.equal(got, want)
    ref = down(torch.nn.functional.silu(gate(x).float()).to(torch.bfloat16) * up(x))
    cos = torch.nn.functional.cosine_similarity(got.float().flatten(), ref.float().flatten(), dim=0).item()
    assert cos > 0.95


def test_adopt_modelopt_two_level_weight():
    """A ModelOpt-style two-level NVFP4 weight (block scales relative to a per-tensor scale)
    runs through the A4W4 GEMM with the global scale folded into alpha and matches the
    dequantise-then-matmul oracle of such weights (fp4-gemm/tests/test_fp4_gemm.py:1150-1164)."""
    import fp4_gemm
    n, k, m = 256, 512, 96
    w = randn_bf16((n, k), 21, 0.02).float()
    global_scale = w.abs().max() / (6.0 * 448.0)                       # weight_scale_2
    packed_np, sf_np = O.quantize_nvfp4((w / global_scale).numpy())   # level 1 on the rescaled tensor
    weight = torch.from_numpy(packed_np).to(DEV)
    weight_scale = torch.from_numpy(sf_np).view(torch.float8_e4m3fn).to(DEV)
    b_packed, sfb, alpha = fp4_gemm.adopt_modelopt_nvfp4_weight(weight, weight_scale, global_scale.to(DEV))
    x = randn_bf16((m, k), 22).to(DEV)
    a_packed, sfa = fp4_gemm.quantize_fp4_sfa_bf16(x)
    out = fp4_gemm.nvfp4_gemm_bf16(a_packed, b_packed, sfa, sfb, alpha=alpha)
    w_deq = torch.from_numpy(O.dequantize_nvfp4(packed_np, sf_np)) * global_scale
    a_deq = torch.from_numpy(O.dequantize_nvfp4(a_packed.cpu().numpy(), sf_linear(sfa, m, k)))
    want = (a_deq @ w_deq.T).to(torch.bfloat16)
    rel, cos = O.gemm_error_metrics(out.cpu(), want)
    assert rel <= 1e-2 and cos >= 0.999, (rel, cos)
    with pytest.raises(ValueError, match="one global scale"):
        fp4_gemm.adopt_modelopt_nvfp4_weight(weight, weight_scale, torch.ones(2))


def test_transformers_decoder_conversion():
    """A small random Qwen3 through `convert_decoder_model`: the fused conversion (norm+quant in one kernel, shared
    activations, one q/k/v GEMM, SwiGLU epilogue, residual additions inside the norm kernels) agrees with the
    per-linear conversion, and both stay close to the bf16 model."""
    transformers = pytest.importorskip("transformers")
    from flashrt_layers.transformers_backend import (FinalNorm, NormQuant, ProjectionSlice, SharedInputFFN,
                                                     StackedProjection, convert_decoder_model)
    cfg = transformers.Qwen3Config(hidden_size=256, intermediate_size=512, num_hidden_layers=3, num_attention_heads=4,
                                   num_key_value_heads=2, head_dim=64, vocab_size=512, max_position_embeddings=256)
    torch.manual_seed(0)
    base = transformers.Qwen3ForCausalLM(cfg).to(DEV, torch.bfloat16).eval()
    ids = torch.randint(0, 512, (2, 48), device=DEV)
    import copy
    with torch.no_grad():
        ref = base(ids).logits.float()
        plain = copy.deepcopy(base)
        assert convert_decoder_model(plain, fuse=False) == 21
        fused = copy.deepcopy(base)
        assert convert_decoder_model(fused, fuse=True, fuse_residual=False) == 21
        carried = copy.deepcopy(base)
        assert convert_decoder_model(carried, fuse=True) == 21
        layer = fused.model.layers[0]
        assert isinstance(layer.mlp, SharedInputFFN) and isinstance(layer.input_layernorm, NormQuant)
        assert isinstance(layer.self_attn.q_proj, StackedProjection) and isinstance(layer.self_attn.k_proj, ProjectionSlice)
        assert isinstance(carried.model.norm, FinalNorm) and not isinstance(fused.model.norm, FinalNorm)
        out_plain = plain(ids).logits.float()
        out_fused = fused(ids).logits.float()
        out_carried = carried(ids).logits.float()
        again = carried(ids).logits.float()                 # a second pass starts from a clean residual carry
    cos = lambda a, b: torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item()
    # A4W4 on every projection of a random-weight model: about 0.95 against bf16 (each linear alone is ~0.99)
    for out in (out_plain, out_fused, out_carried):
        assert cos(out, ref) > 0.9, cos(out, ref)
    # the fused norm multiplies by the weight in fp32 (transformers rounds to bf16 first): a few codes flip
    assert cos(out_fused, out_plain) > 0.98, cos(out_fused, out_plain)
    # residual additions inside the norm kernels: the norm sees the fp32 sum instead of its bf16 rounding
    assert cos(out_carried, out_fused) > 0.98, cos(out_carried, out_fused)
    assert torch.equal(again, out_carried)
    assert carried.model.layers[0]._frt_carry.deferred is None
    # the shared quantisation was used: one producer call per norm, no per-linear quantise of that tensor
    assert layer.self_attn.q_proj.source is layer.input_layernorm.produced


def test_conversion_skip_names_and_norm_detection():
    """`skip` matches qualified module names; a norm that scales by (1 + weight) is detected by running it, and a
    norm of another form is left alone"""
    transformers = pytest.importorskip("transformers")
    from torch import nn
    from flashrt_layers.transformers_backend import SharedInputLinear, _norm_semantics, convert_decoder_model
    cfg = transformers.Qwen3Config(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, head_dim=64, vocab_size=512, max_position_embeddings=256)
    torch.manual_seed(1)
    model = transformers.Qwen3ForCausalLM(cfg).to(DEV, torch.bfloat16).eval()
    n = convert_decoder_model(model, fuse=True, skip=("lm_head", "model.layers.1.mlp", "layers.0.self_attn.o_proj"))
    assert n == 6 + 4                                        # layer 0 keeps its o_proj, layer 1 its MLP
    assert isinstance(model.model.layers[0].self_attn.o_proj, nn.Linear)
    assert isinstance(model.model.layers[1].self_attn.o_proj, SharedInputLinear)
    assert isinstance(model.model.layers[1].mlp.gate_proj, nn.Linear)
    with torch.no_grad():
        assert torch.isfinite(model(torch.randint(0, 512, (1, 16), device=DEV)).logits.float()).all()

    class OnePlus(nn.Module):
        def __init__(self):
            super().__init__()
            self.weight = nn.Parameter(torch.randn(256, device=DEV) * 0.1)
            self.eps = 1e-6

        def forward(self, x):
            xf = x.float()
            return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps) * (1 + self.weight.float())).to(x.dtype)

    class Shifted(OnePlus):
        def forward(self, x):
            return super().forward(x) + 1.0

    assert _norm_semantics(OnePlus()) == "one_plus"
    assert _norm_semantics(Shifted()) is None
    assert _norm_semantics(transformers.models.qwen3.modeling_qwen3.Qwen3RMSNorm(256).to(DEV)) == "plain"
