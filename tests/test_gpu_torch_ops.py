"""The torch operator layer (reference names and signatures) on a GPU: every op
routes to the C ABI, outputs equal the direct C-ABI results / the oracle, the
ops trace under torch.compile(fullgraph=True) and replay bit-stably in a CUDA
graph (fp4-gemm/tests/test_fp4_gemm.py:873-898,1419-1442)."""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "flashrt-hf-kernels_b200" / "torch-ext"))

from oracle import nvfp4_oracle as O  # noqa: E402

DEV = "cuda"


def bf16(shape, seed, scale=1.0, offset=0.0):
    g = torch.Generator().manual_seed(seed)
    return (offset + scale * torch.randn(shape, generator=g)).to(torch.bfloat16).to(DEV)


def test_layout_package():
    import flashrt_nvfp4 as pkg
    lin = torch.randint(0, 256, (129, 256), dtype=torch.uint8)
    out = pkg.nvfp4_sf_linear_to_swizzled(lin.to(DEV))
    assert out.numel() == pkg.nvfp4_sf_swizzled_bytes(129, 4096) == 65536
    np.testing.assert_array_equal(out.cpu().numpy(), O.sf_linear_to_swizzled(lin.numpy()))
    reuse = torch.zeros_like(out)
    assert pkg.nvfp4_sf_linear_to_swizzled(lin.to(DEV), out=reuse) is reuse and torch.equal(reuse, out)
    with pytest.raises(ValueError):
        pkg.nvfp4_sf_swizzled_bytes(0, 64)
    with pytest.raises(ValueError):
        pkg.nvfp4_sf_swizzled_bytes(4, 40)


def test_norm_package_and_rejections():
    import flashrt_residual_norm_quant as pkg
    x, r, w = bf16((63, 2048), 1), bf16((63, 2048), 2), bf16((2048,), 3, 0.1, 1.0)
    y = pkg.rms_norm_bf16(x, w, 1e-6)
    np.testing.assert_array_equal(O.torch_bf16_to_bits(y), O.rms_norm_bf16(O.torch_bf16_to_bits(x), O.torch_bf16_to_bits(w), 1e-6))
    res = r.clone()
    y2 = pkg.residual_add_rms_norm_bf16(res, x, w, 1e-6)
    wr, wy = O.residual_add_rms_norm_bf16(O.torch_bf16_to_bits(r), O.torch_bf16_to_bits(x), O.torch_bf16_to_bits(w), 1e-6)
    np.testing.assert_array_equal(O.torch_bf16_to_bits(res), wr)
    np.testing.assert_array_equal(O.torch_bf16_to_bits(y2), wy)
    with pytest.raises(RuntimeError):
        pkg.rms_norm_bf16(x[:, :2040].contiguous(), w[:2040].contiguous())      # dim % 16
    with pytest.raises(RuntimeError):
        pkg.rms_norm_bf16(x.t(), w)                                             # non-contiguous
    with pytest.raises(RuntimeError):
        pkg.rms_norm_bf16(x, w[:100].contiguous())                              # shape mismatch


def test_fused_producer_feeds_gemm_end_to_end():
    """config-1 shaped: residual/hidden [128,4096], weight 4096x4096 N(0,.02)."""
    import fp4_fused_ops, fp4_gemm
    m, h, n = 128, 4096, 4096
    x, r, w = bf16((m, h), 23), bf16((m, h), 24), bf16((h,), 25, 0.1, 1.0)
    weight = bf16((n, h), 26, 0.02)
    wp, wsf = fp4_gemm.quantize_fp4_sfa_bf16(weight, is_sfb=True)
    res = r.clone()
    ap, sfa = fp4_fused_ops.residual_add_rms_norm_quant_nvfp4_swizzled_bf16(res, x, w, 1e-6)
    out = fp4_gemm.nvfp4_gemm_bf16(ap, wp, sfa, wsf)
    want = O.fused_norm_quant(O.torch_bf16_to_bits(x), O.torch_bf16_to_bits(w), 1e-6, res_bits=O.torch_bf16_to_bits(r))
    np.testing.assert_array_equal(ap.cpu().numpy(), want["packed"])
    np.testing.assert_array_equal(sfa.cpu().numpy(), O.sf_linear_to_swizzled(want["sf_linear"]))
    wq_p, wq_s = O.quantize_nvfp4(weight.float().cpu().numpy())
    np.testing.assert_array_equal(wp.cpu().numpy(), wq_p)
    ref = O.gemm_bf16(want["packed"], want["sf_linear"], wq_p, wq_s)
    rel, cos = O.gemm_error_metrics(out.cpu(), ref)
    assert rel <= 1e-2 and cos >= 0.999
    # two-level variant: g = amax/(6*448); quantise v/g; GEMM alpha = g
    amax = np.abs(O.bf16_bits_to_f32(want["normed"])).max()
    g = float(np.float32(amax) / np.float32(6 * 448))
    res2 = r.clone()
    ap2, sfa2 = fp4_fused_ops.residual_add_rms_norm_quant_nvfp4(res2, x, w, 1e-6, inv_global_scale=1.0 / g)
    out2 = fp4_gemm.nvfp4_gemm_bf16(ap2, wp, sfa2, wsf, alpha=g)
    rel, cos = O.gemm_error_metrics(out2.cpu(), ref)
    assert rel <= 0.2 and cos >= 0.98          # differs from one-level by quantisation noise only


def test_other_producers_and_dequant():
    import fp4_fused_ops, fp4_gemm
    x, w = bf16((257, 4096), 7, 0.2), bf16((4096,), 8, 0.05)
    normed, packed, sfa = fp4_fused_ops.rms_norm_quantize_fp4_sfa_bf16(x, w, 1e-6)
    qp, qs = fp4_gemm.quantize_fp4_sfa_bf16(normed)
    assert torch.equal(qp, packed) and torch.equal(qs, sfa)
    deq = fp4_fused_ops.dequantize_fp4_sfa_fp16(packed, sfa)
    deq2 = fp4_gemm.dequantize_fp4_sfa_fp16(packed, sfa)
    assert torch.equal(deq, deq2)
    lin = O.sf_swizzled_to_linear(sfa.cpu().numpy(), 257, 4096)
    np.testing.assert_array_equal(deq.float().cpu().numpy(), O.dequantize_nvfp4(packed.cpu().numpy(), lin))
    r = bf16((257, 4096), 9)
    res, p2, s2 = fp4_fused_ops.residual_add_rms_norm_nvfp4_bf16(r.clone(), x, None, 1e-6)
    want = O.fused_norm_quant(O.torch_bf16_to_bits(x), None if False else O.torch_bf16_to_bits(torch.ones(4096).bfloat16()),
                              1e-6, res_bits=O.torch_bf16_to_bits(r), flags=2 | 4 | 8)
    np.testing.assert_array_equal(p2.cpu().numpy(), want["packed"])
    assert fp4_fused_ops.sfa_size_bytes(257, 4096) == 3 * 64 * 512
    # bf16 and fp16 quantisers agree byte for byte on values both represent
    xs = bf16((8, 5120), 10, 1.5)
    a = fp4_gemm.quantize_fp4_sfa_bf16(xs)
    b = fp4_gemm.quantize_fp4_sfa_fp16(xs.half())
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


def test_gemm_ops_epilogues_smallm_and_errors():
    import fp4_gemm
    m, n, k = 64, 512, 512
    a, b = bf16((m, k), 11, 0.25), bf16((n, k), 12, 0.25)
    ap, sfa = fp4_gemm.quantize_fp4_sfa_bf16(a)
    bp, sfb = fp4_gemm.quantize_fp4_sfa_bf16(b, is_sfb=True)
    A, B = ap.cpu().numpy(), bp.cpu().numpy()
    la, lb = O.sf_swizzled_to_linear(sfa.cpu().numpy(), m, k), O.sf_swizzled_to_linear(sfb.cpu().numpy(), n, k)
    bias, res = bf16((n,), 13, 0.02), bf16((m, n), 14)

    def close(got, **kw):
        rel, cos = O.gemm_error_metrics(got.cpu(), O.gemm_bf16(A, la, B, lb, **kw))
        assert rel <= 1e-2 and cos >= 0.999

    close(fp4_gemm.nvfp4_gemm_bf16(ap, bp, sfa, sfb, alpha=0.5, variant=1), alpha=0.5)
    close(fp4_gemm.fp4_w4a16_linear_bf16(ap, bp, sfa, sfb, variant=2))
    close(fp4_gemm.nvfp4_gemm_bias_bf16(ap, bp, sfa, sfb, bias), bias_bits=O.torch_bf16_to_bits(bias))
    close(fp4_gemm.nvfp4_gemm_residual_bf16(ap, bp, sfa, sfb, res, alpha=2.0), alpha=2.0,
          residual_bits=O.torch_bf16_to_bits(res))
    close(fp4_gemm.nvfp4_gemm_bias_residual_bf16(ap, bp, sfa, sfb, bias, res), bias_bits=O.torch_bf16_to_bits(bias),
          residual_bits=O.torch_bf16_to_bits(res))
    # small-M entry points: per-row GEMV equals the multi-row op bit for bit
    ap16, sfa16 = fp4_gemm.quantize_fp4_sfa_bf16(a[:16].contiguous())
    rows16 = fp4_gemm.fp4_w4a4_gemm_warpsplit_mrows_bf16(ap16, bp, sfa16, sfb)
    for i in (0, 7, 15):
        api, sfai = fp4_gemm.quantize_fp4_sfa_bf16(a[i:i + 1].contiguous())
        assert torch.equal(fp4_gemm.fp4_w4a4_gemv_warpsplit_bf16(api, bp, sfai, sfb)[0], rows16[i])
    ap17, sfa17 = fp4_gemm.quantize_fp4_sfa_bf16(a[:17].contiguous())
    with pytest.raises(RuntimeError, match="1..16 rows"):
        fp4_gemm.fp4_w4a4_gemm_warpsplit_mrows_bf16(ap17, bp, sfa17, sfb)
    with pytest.raises(RuntimeError):
        fp4_gemm.nvfp4_gemm_bf16(ap, bp[:, :128].contiguous(), sfa, sfb)
    with pytest.raises(RuntimeError):
        fp4_gemm.nvfp4_gemm_bf16(ap, bp, sfa[:100], sfb)
    with pytest.raises(RuntimeError):
        fp4_gemm.nvfp4_gemm_bf16(ap, bp, sfa, sfb, out=torch.empty(m, n, device=DEV, dtype=torch.float16))


def test_compile_and_graph_replay():
    import fp4_fused_ops, fp4_gemm
    m, h, n = 256, 2048, 1024
    x, r, w = bf16((m, h), 31), bf16((m, h), 32), bf16((h,), 33, 0.1, 1.0)
    wp, wsf = fp4_gemm.quantize_fp4_sfa_bf16(bf16((n, h), 34, 0.02), is_sfb=True)

    def step(res, xx):
        ap, sfa = fp4_fused_ops.residual_add_rms_norm_quant_nvfp4_swizzled_bf16(res, xx, w, 1e-6)
        return fp4_gemm.nvfp4_gemm_bf16(ap, wp, sfa, wsf)

    eager = step(r.clone(), x)
    compiled = torch.compile(step, fullgraph=True)
    assert torch.equal(compiled(r.clone(), x), eager)
    res_g, packed, sfa = r.clone(), *fp4_fused_ops._alloc_fp4(m, h, DEV)
    out = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            fp4_fused_ops.residual_add_rms_norm_quant_nvfp4_swizzled_bf16(res_g, x, w, 1e-6, packed=packed, sfa=sfa)
            fp4_gemm.nvfp4_gemm_bf16(packed, wp, sfa, wsf, out=out)
    res_g.copy_(r); graph.replay(); torch.cuda.synchronize()
    first = out.clone()
    res_g.copy_(r); graph.replay(); torch.cuda.synchronize()
    assert torch.equal(first, out) and torch.equal(first, eager)


def test_hub_and_layers():
    from flashrt_b200_core.hub import get_kernel, kernelize
    from flashrt_layers import FlashRTQuantLinear, FusedNormLinear
    assert get_kernel("flashrt/fp4-gemm", version=1, trust_remote_code=True).nvfp4_gemm_bf16 is not None

    class TinyRMSNorm(torch.nn.Module):
        def __init__(self, dim):
            super().__init__()
            self.weight = torch.nn.Parameter(torch.ones(dim) + 0.1 * torch.randn(dim))
            self.variance_epsilon = 1e-6

        def forward(self, h):
            v = h.float().pow(2).mean(-1, keepdim=True)
            return (self.weight * (h.float() * torch.rsqrt(v + self.variance_epsilon))).to(h.dtype)

    class Tiny(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.norm = TinyRMSNorm(512)
            self.proj = torch.nn.Linear(512, 264, bias=True)

        def forward(self, h):
            return self.proj(self.norm(h))

    torch.manual_seed(0)
    model = Tiny().to(DEV).to(torch.bfloat16)
    h = torch.randn(4, 33, 512, device=DEV, dtype=torch.bfloat16)
    ref = model(h)
    kernelize(model)
    got_norm = model.norm(h)
    assert (got_norm.float() - TinyRMSNorm.forward(model.norm, h).float()).abs().max() <= 2 ** -5
    model.proj = FlashRTQuantLinear.from_linear(model.proj)
    got = model(h)
    assert got.shape == ref.shape
    cos = torch.nn.functional.cosine_similarity(got.float().flatten(), ref.float().flatten(), dim=0)
    assert cos > 0.98                                       # A4W4 against the unquantised linear
    lin_a = FlashRTQuantLinear.from_linear(torch.nn.Linear(512, 256, bias=False).to(DEV).to(torch.bfloat16))
    lin_b = FlashRTQuantLinear.from_linear(torch.nn.Linear(512, 128, bias=False).to(DEV).to(torch.bfloat16))
    fused = FusedNormLinear(model.norm.weight.data, 1e-6, [lin_a, lin_b])
    res = torch.randn(66, 512, device=DEV, dtype=torch.bfloat16)
    xa = torch.randn(66, 512, device=DEV, dtype=torch.bfloat16)
    oa, ob = fused(res, xa)
    assert oa.shape == (66, 256) and ob.shape == (66, 128)


@pytest.mark.parametrize("K", [4096, 12288, 2048])
def test_decode_matvec_known_answer(K):
    """the reference's constant-input check of its M=1 matvec
    (flashrt-smallm-gemm/tests/test_nvfp4_w4a4_decode_matvec.py:33-52): nibbles 0x11 (0.5), scales 0x38 (1.0)
    give K * 0.25 * alpha in every output"""
    import flashrt_nvfp4
    import flashrt_smallm_gemm
    N, alpha = 16, 0.5
    a_packed = torch.full((K // 2,), 0x11, device=DEV, dtype=torch.uint8)
    b_packed = torch.full((N, K // 2), 0x11, device=DEV, dtype=torch.uint8)
    sfa = flashrt_nvfp4.nvfp4_sf_linear_to_swizzled(torch.full((1, K // 16), 0x38, dtype=torch.uint8, device=DEV))
    sfb = flashrt_nvfp4.nvfp4_sf_linear_to_swizzled(torch.full((N, K // 16), 0x38, dtype=torch.uint8, device=DEV))
    out = flashrt_smallm_gemm.nvfp4_w4a4_decode_matvec_bf16out(a_packed, b_packed, sfa, sfb, alpha=alpha)
    expected = torch.full((N,), K * 0.25 * alpha, device=DEV, dtype=torch.bfloat16)
    torch.testing.assert_close(out, expected)
    again = flashrt_smallm_gemm.nvfp4_w4a4_decode_matvec_bf16out(a_packed.view(1, -1), b_packed, sfa, sfb, alpha=alpha,
                                                                 out=out)
    assert again.data_ptr() == out.data_ptr() and torch.equal(again, expected)
    with pytest.raises(RuntimeError, match=r"\(K / 2,\) or \(1, K / 2\)"):
        flashrt_smallm_gemm.nvfp4_w4a4_decode_matvec_bf16out(b_packed[:2], b_packed, sfa, sfb)
