"""GPU parity of the decode fusion frt_norm_quant_gemm_bf16 (residual add + RMSNorm -> NVFP4 inside the
weight-streaming GEMM, up to 4 token rows).  Oracle: the two-call path of this library, which the other GPU
tests pin against the CPU oracle (frt_norm_quant_nvfp4: bit-exact bytes; frt_nvfp4_gemm_bf16: dequantised
fp32 matmul).  Bar: the fused output equals the two-call output BIT FOR BIT, and residual_out equals the
residual the producer leaves."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from tests.gpu_common import DEV, capi, device_status, quantize, sf_bytes  # noqa: E402

FLAGS = {"none": 0, "one_plus_w+round_bf16": 1 | 2, "rne_e2m1": 4, "norm_from_bf16_residual": 8}


def two_calls(residual, x, weight, eps, flags, bp, sfb, m, n, k):
    L, P, st = capi.lib(), capi.ptr, capi.stream_ptr()
    res = residual.clone() if residual is not None else None
    packed = torch.empty(m, k // 2, dtype=torch.uint8, device=DEV)
    sf = torch.zeros(sf_bytes(m, k), dtype=torch.uint8, device=DEV)
    capi.check(L.frt_norm_quant_nvfp4(P(res), P(x), P(weight), eps, 1.0, None, P(packed), P(sf), m, k, flags, st))
    out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    capi.check(L.frt_nvfp4_gemm_bf16(P(packed), P(sf), P(bp), P(sfb), None, None, P(out), m, n, k, 1.0, 0.0, st))
    torch.cuda.synchronize()
    return out, res


def fused(residual, x, weight, eps, flags, bp, sfb, m, n, k):
    L, P, st = capi.lib(), capi.ptr, capi.stream_ptr()
    res_out = torch.full_like(residual, 7.0) if residual is not None else None
    out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    capi.check(L.frt_norm_quant_gemm_bf16(P(residual), P(res_out), P(x), P(weight), eps, flags, P(bp), P(sfb), None,
                                          P(out), m, n, k, 1.0, st), "fused")
    torch.cuda.synchronize()
    return out, res_out


def make(m, n, k, seed, with_res=True, with_w=True):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16).to(DEV)
    bp, sfb = quantize(w)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    residual = (torch.randn(m, k, generator=g) * 2).to(torch.bfloat16).to(DEV) if with_res else None
    nw = (1.0 + 0.1 * torch.randn(k, generator=g)).to(torch.bfloat16).to(DEV) if with_w else None
    return bp, sfb, x, residual, nw


# Qwen3-8B linears fed by a norm (split-K 4, no split), an o-shaped layer (split-K 8), and small layers whose
# row is one, two and four warps of the producer wide (K = 512, 1024, 2048), N not a multiple of 128
SHAPES = [(6144, 4096), (24576, 4096), (4096, 4096), (264, 512), (1032, 1024), (2048, 2048), (136, 192)]


@pytest.mark.parametrize("n,k", SHAPES)
@pytest.mark.parametrize("m", [1, 2, 3, 4])
def test_fused_equals_two_calls_bitwise(n, k, m):
    bp, sfb, x, residual, nw = make(m, n, k, 5 + n + k + m)
    want, want_res = two_calls(residual, x, nw, 1e-6, 0, bp, sfb, m, n, k)
    got, got_res = fused(residual, x, nw, 1e-6, 0, bp, sfb, m, n, k)
    assert torch.equal(got, want)
    assert torch.equal(got_res, want_res)
    assert device_status() == 0


@pytest.mark.parametrize("flag", sorted(FLAGS))
@pytest.mark.parametrize("with_res,with_w", [(True, True), (False, True), (True, False), (False, False)])
def test_fused_flags_and_optional_inputs(flag, with_res, with_w):
    m, n, k = 3, 1024, 4096
    bp, sfb, x, residual, nw = make(m, n, k, 99, with_res, with_w)
    want, want_res = two_calls(residual, x, nw, 1e-5, FLAGS[flag], bp, sfb, m, n, k)
    got, got_res = fused(residual, x, nw, 1e-5, FLAGS[flag], bp, sfb, m, n, k)
    assert torch.equal(got, want)
    if with_res:
        assert torch.equal(got_res, want_res)
    assert device_status() == 0


def test_fused_in_a_graph_and_repeated():
    """captured in a CUDA graph between two other launches (the programmatic dependent launch path) and replayed"""
    m, n, k = 1, 6144, 4096
    bp, sfb, x, residual, nw = make(m, n, k, 4242)
    want, _ = two_calls(residual, x, nw, 1e-6, 0, bp, sfb, m, n, k)
    L, P = capi.lib(), capi.ptr
    res_out = torch.empty_like(residual)
    out = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            st = capi.stream_ptr()
            for _ in range(3):
                capi.check(L.frt_norm_quant_gemm_bf16(P(residual), P(res_out), P(x), P(nw), 1e-6, 0, P(bp), P(sfb), None,
                                                      P(out), m, n, k, 1.0, st))
    for _ in range(3):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, want)
    assert device_status() == 0


def test_fused_rejections():
    L, P, st = capi.lib(), capi.ptr, capi.stream_ptr()
    bp, sfb, x, residual, nw = make(4, 256, 512, 1)
    out = torch.empty(4, 256, dtype=torch.bfloat16, device=DEV)
    res_out = torch.empty_like(residual)
    call = lambda **kw: L.frt_norm_quant_gemm_bf16(P(kw.get("rin", residual)), P(kw.get("rout", res_out)), P(x), P(nw), 1e-6,
                                                   kw.get("flags", 0), P(bp), P(sfb), None, P(out), kw.get("m", 4), 256,
                                                   kw.get("k", 512), 1.0, st)
    assert call(m=5) == -4
    assert call(k=8192) == -4
    assert call(rout=residual) == -4          # in place: every CTA reads the input
    assert call(rout=None) == -1
    assert call(flags=0x100) == -4
    assert call(k=520) == -2
    assert call() == 0
    torch.cuda.synchronize()
