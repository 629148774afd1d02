"""GPU parity of the SwiGLU -> NVFP4 producer: the stand-alone kernel against the
reference's production-chain definition and its own CUDA kernel, and the GEMM-epilogue
form against the chain (GEMM -> stand-alone kernel) it replaces, byte for byte."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from tests.gpu_common import (DEV, O, alloc_fp4, bits, capi, device_status, gemm, quantize, randn_bf16,  # noqa: E402
                              ref_lib, sf_linear)

P = capi.ptr


def st():
    return capi.stream_ptr()


def silu_mul_quant(merged, encoder=0):
    rows, hidden = merged.shape[0], merged.shape[1] // 2
    packed, sf = alloc_fp4(rows, hidden)
    prev = capi.lib().frt_set_option(1, encoder)
    try:
        capi.check(capi.lib().frt_silu_mul_quant_nvfp4(P(merged), P(packed), P(sf), rows, hidden, st()))
    finally:
        capi.lib().frt_set_option(1, prev)
    return packed, sf


@pytest.mark.parametrize("encoder", [0, 1])
@pytest.mark.parametrize("rows,hidden,scale", [(1, 1024, 0.2), (7, 1024, 0.2), (257, 1024, 0.2), (63, 12288, 1.0),
                                               (130, 48, 3.0)])
def test_silu_mul_quant_production_chain(rows, hidden, scale, encoder):
    """The reference's own check of this op (fp4-fused-ops/tests/test_fp4_fused_ops.py:483-495):
    stage silu(gate) * up in fp32 with torch on the GPU, round to bf16, quantise with the
    reference quantiser; the fused op must give the same bytes."""
    merged = randn_bf16((rows, 2 * hidden), 2026081700 + rows, scale).to(DEV)
    merged[0, :8] = torch.tensor([-100.0, -20.0, -0.0, 0.0, 20.0, 100.0, -88.5, 3e38], dtype=torch.bfloat16)
    packed, sf = silu_mul_quant(merged, encoder)
    staged = (torch.nn.functional.silu(merged[:, :hidden].float()) * merged[:, hidden:].float()).bfloat16()
    want_p, want_s = O.quantize_nvfp4(staged.float().cpu().numpy())
    np.testing.assert_array_equal(packed.cpu().numpy(), want_p)
    np.testing.assert_array_equal(sf_linear(sf, rows, hidden), want_s)
    ref = ref_lib()
    if ref is not None:
        rp, rs = alloc_fp4(rows, hidden)
        assert ref.ref_silu_mul_quantize_bf16(P(merged), P(rp), P(rs), rows, hidden, st()) == 0
        torch.cuda.synchronize()
        assert torch.equal(rp, packed) and torch.equal(rs, sf)
    # the all-CPU oracle differs only where the host and device exponentials round apart
    cpu = O.silu_mul_quantize(bits(merged))
    assert (cpu["staged"] != bits(staged)).mean() < 2e-3
    assert (O.unpack_codes(cpu["packed"]) != O.unpack_codes(want_p)).mean() < 5e-3


def make_operands(M, N2, K, seed):
    x = randn_bf16((M, K), seed, 1.0).to(DEV)
    w = randn_bf16((N2, K), seed + 1, 0.05).to(DEV)
    a, sfa = quantize(x)
    b, sfb = quantize(w)
    return a, sfa, b, sfb


@pytest.mark.parametrize("M,hidden,K,alpha", [(256, 128, 256, 1.0), (300, 384, 512, 0.5), (37, 256, 128, 2.0),
                                              (1, 128, 64, 1.0), (2048, 1536, 2048, 1.0), (4096, 1024, 1024, 0.75),
                                              (1000, 12288, 512, 1.0)])
def test_gemm_swiglu_epilogue_equals_chain(M, hidden, K, alpha):
    """GEMM with the producer as its epilogue == bf16 GEMM followed by the stand-alone producer."""
    N2 = 2 * hidden
    a, sfa, b, sfb = make_operands(M, N2, K, 4000 + M + hidden)
    prev = capi.lib().frt_set_option(2, 4)            # the chain's GEMM on the same tile family
    try:
        merged = gemm(a, sfa, b, sfb, M, N2, K, alpha=alpha)
    finally:
        capi.lib().frt_set_option(2, prev)
    want_p, want_s = silu_mul_quant(merged)
    got_p, got_s = alloc_fp4(M, hidden)
    capi.check(capi.lib().frt_nvfp4_gemm_swiglu_nvfp4(P(a), P(sfa), P(b), P(sfb), P(got_p), P(got_s), M, N2, K,
                                                      float(alpha), st()))
    torch.cuda.synchronize()
    assert device_status() == 0
    assert torch.equal(got_p, want_p)
    np.testing.assert_array_equal(sf_linear(got_s, M, hidden), sf_linear(want_s, M, hidden))


def test_gemm_swiglu_against_oracle():
    """End to end against the CPU oracle (dequantise, fp32 matmul, bf16, SwiGLU, quantise): the
    result dequantises to the oracle's within the GEMM tolerance."""
    M, hidden, K = 192, 256, 512
    N2 = 2 * hidden
    x = randn_bf16((M, K), 51, 1.0)
    w = randn_bf16((N2, K), 52, 0.05)
    a, sfa = quantize(x.to(DEV))
    b, sfb = quantize(w.to(DEV))
    got_p, got_s = alloc_fp4(M, hidden)
    capi.check(capi.lib().frt_nvfp4_gemm_swiglu_nvfp4(P(a), P(sfa), P(b), P(sfb), P(got_p), P(got_s), M, N2, K,
                                                      1.0, st()))
    torch.cuda.synchronize()
    merged = O.gemm_bf16(a.cpu().numpy(), sf_linear(sfa, M, K), b.cpu().numpy(), sf_linear(sfb, N2, K))
    want = O.silu_mul_quantize(bits(merged))
    got = O.dequantize_nvfp4(got_p.cpu().numpy(), sf_linear(got_s, M, hidden))
    ref = O.dequantize_nvfp4(want["packed"], want["sf_linear"])
    rel, cos = O.gemm_error_metrics(torch.from_numpy(got), torch.from_numpy(ref))
    assert rel <= 1e-2 and cos >= 0.999, (rel, cos)          # tolerance of the GEMM contract
    assert (O.unpack_codes(got_p.cpu().numpy()) != O.unpack_codes(want["packed"])).mean() < 5e-3


def test_swiglu_argument_errors():
    L = capi.lib()
    a, sfa, b, sfb = make_operands(128, 256, 64, 9)
    p, s = alloc_fp4(128, 128)
    assert L.frt_nvfp4_gemm_swiglu_nvfp4(None, P(sfa), P(b), P(sfb), P(p), P(s), 128, 256, 64, 1.0, st()) == -1
    assert L.frt_nvfp4_gemm_swiglu_nvfp4(P(a), P(sfa), P(b), P(sfb), P(p), P(s), 128, 192, 64, 1.0, st()) < 0
    assert L.frt_nvfp4_gemm_swiglu_nvfp4(P(a), P(sfa), P(b), P(sfb), P(p), P(s), 128, 256, 48, 1.0, st()) < 0
    m = randn_bf16((4, 64), 1).to(DEV)
    assert L.frt_silu_mul_quant_nvfp4(P(m), P(p), P(s), 4, 24, st()) < 0
    assert L.frt_silu_mul_quant_nvfp4(P(m), None, P(s), 4, 32, st()) == -1


def test_torch_ops_swiglu():
    import fp4_fused_ops
    import fp4_gemm
    M, hidden, K = 512, 256, 256
    a, sfa, b, sfb = make_operands(M, 2 * hidden, K, 77)
    merged = fp4_gemm.nvfp4_gemm_bf16(a, b, sfa, sfb)
    p1, s1 = fp4_fused_ops.silu_mul_quantize_fp4_sfa_bf16(merged)
    p2, s2 = fp4_gemm.nvfp4_gemm_swiglu_nvfp4_bf16(a, b, sfa, sfb)
    assert torch.equal(p1, p2)
    np.testing.assert_array_equal(sf_linear(s1, M, hidden), sf_linear(s2, M, hidden))
    with pytest.raises(RuntimeError, match="divisible by 256"):
        fp4_gemm.nvfp4_gemm_swiglu_nvfp4_bf16(a, b[:384], sfa, sfb, out_packed=p2, out_sfa=s2)
    with pytest.raises(RuntimeError, match="divisible by 32"):
        fp4_fused_ops.silu_mul_quantize_fp4_sfa_bf16(merged[:, :48].contiguous(), packed=p1, sfa=s1)


def test_swiglu_ops_compile_and_graph():
    """the new ops trace under torch.compile(fullgraph=True) and replay bit-stably in a CUDA graph"""
    import fp4_gemm
    import transformer_fused_ops
    M, hidden, K = 256, 256, 256
    a, sfa, b, sfb = make_operands(M, 2 * hidden, K, 99)
    p_eager, s_eager = fp4_gemm.nvfp4_gemm_swiglu_nvfp4_bf16(a, b, sfa, sfb)

    def step(aa):
        return fp4_gemm.nvfp4_gemm_swiglu_nvfp4_bf16(aa, b, sfa, sfb)

    p_c, s_c = torch.compile(step, fullgraph=True)(a)
    assert torch.equal(p_c, p_eager) and torch.equal(s_c, s_eager)
    logits = randn_bf16((64, 128), 5).to(DEV)
    idx_e, val_e = transformer_fused_ops.router_topk_bf16(logits, 8)
    idx_c, val_c = torch.compile(lambda l: transformer_fused_ops.router_topk_bf16(l, 8), fullgraph=True)(logits)
    assert torch.equal(idx_c, idx_e) and torch.equal(val_c, val_e)

    op, osf = alloc_fp4(M, hidden)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fp4_gemm.nvfp4_gemm_swiglu_nvfp4_bf16(a, b, sfa, sfb, out_packed=op, out_sfa=osf)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            fp4_gemm.nvfp4_gemm_swiglu_nvfp4_bf16(a, b, sfa, sfb, out_packed=op, out_sfa=osf)
    torch.cuda.synchronize()
    op.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(op, p_eager)
