"""GPU parity of the NVFP4 GEMM through the C ABI.

Oracle: dequantise the exact bytes the kernel consumed, fp32 matmul, bf16
(fp4-gemm/tests/test_fp4_gemm.py:593-636).  Tolerance (stated by the task):
relative Frobenius error <= 1e-2 and cosine >= 0.999; in addition the
reference's own envelope max_abs <= 0.125, mean <= 0.005 on 0.25-scale data.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from tests.gpu_common import DEV, O, alloc_fp4, bits, capi, device_status, gemm, quantize, ref_lib, sf_linear  # noqa: E402

REL_FROB, COSINE = 1e-2, 0.999


def make_quantized(m, n, k, seed, scale=0.25):
    g = torch.Generator().manual_seed(seed)
    a = (torch.randn(m, k, generator=g) * scale).to(torch.bfloat16).to(DEV)
    b = (torch.randn(n, k, generator=g) * scale).to(torch.bfloat16).to(DEV)
    ap, sfa = quantize(a)
    bp, sfb = quantize(b)
    return ap, sfa, bp, sfb


def oracle_out(ap, sfa, bp, sfb, m, n, k, **kw):
    return O.gemm_bf16(ap.cpu().numpy(), sf_linear(sfa, m, k), bp.cpu().numpy(), sf_linear(sfb, n, k), **kw)


def gpu_fp32_reference(ap, sfa, bp, sfb, m, n, k, alpha=1.0):
    """dequantise on the CPU oracle, matmul in fp32 on the GPU (full-size cases)."""
    a = torch.from_numpy(O.dequantize_nvfp4(ap.cpu().numpy(), sf_linear(sfa, m, k))).to(DEV)
    b = torch.from_numpy(O.dequantize_nvfp4(bp.cpu().numpy(), sf_linear(sfb, n, k))).to(DEV)
    return ((a @ b.T) * alpha).to(torch.bfloat16)


def assert_close(got, want, strict=True):
    rel, cos = O.gemm_error_metrics(got.cpu(), want.cpu())
    assert rel <= REL_FROB and cos >= COSINE, (rel, cos)
    if strict:
        d = (got.cpu().float() - want.cpu().float()).abs()
        assert d.max() <= 0.125 and d.mean() <= 0.005, (float(d.max()), float(d.mean()))
    assert device_status() == 0


def test_constant_known_answer():
    # flashrt-smallm-gemm/tests/test_nvfp4_w4a4_decode_matvec.py:32-52 (every output = K*0.25*alpha)
    for m, n, k in [(1, 16, 4096), (128, 256, 12288), (64, 128, 256)]:
        ap = torch.full((m, k // 2), 0x11, dtype=torch.uint8, device=DEV)
        bp = torch.full((n, k // 2), 0x11, dtype=torch.uint8, device=DEV)
        sfa = torch.full((int(capi.lib().frt_nvfp4_sf_swizzled_bytes(m, k)),), 0x38, dtype=torch.uint8, device=DEV)
        sfb = torch.full((int(capi.lib().frt_nvfp4_sf_swizzled_bytes(n, k)),), 0x38, dtype=torch.uint8, device=DEV)
        out = gemm(ap, sfa, bp, sfb, m, n, k, alpha=0.5)
        assert torch.all(out.float() == k * 0.25 * 0.5)
    assert device_status() == 0


SHAPES = [(16, 128, 128), (32, 256, 256), (64, 512, 512),             # the reference's quick grid
          (128, 128, 256), (128, 256, 256), (256, 384, 1024), (129, 136, 320), (300, 1000, 704),
          (1, 4096, 4096), (4, 1024, 2048), (17, 264, 512), (128, 4096, 4096), (576, 2048, 1536)]


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_gemm_vs_oracle(m, n, k):
    ap, sfa, bp, sfb = make_quantized(m, n, k, 7000 + m + n + k)
    out = gemm(ap, sfa, bp, sfb, m, n, k)
    assert_close(out, oracle_out(ap, sfa, bp, sfb, m, n, k))


@pytest.mark.parametrize("cfg", [1, 2, 3, 4, 5, 6])
@pytest.mark.parametrize("m,n,k", [(128, 256, 256), (256, 768, 1024), (300, 1000, 704), (512, 576, 2048)])
def test_every_tile_configuration(m, n, k, cfg):
    ap, sfa, bp, sfb = make_quantized(m, n, k, 9000 + m + n + k)
    prev = capi.lib().frt_set_option(2, cfg)
    try:
        out = gemm(ap, sfa, bp, sfb, m, n, k)
    finally:
        capi.lib().frt_set_option(2, prev)
    assert_close(out, oracle_out(ap, sfa, bp, sfb, m, n, k))


@pytest.mark.parametrize("m", [1, 4, 16, 17, 33, 64])
def test_small_m_random_bytes(m):
    """random codes (all 16 nibbles, -0 included) and random scale bytes:
    grouped-moe-gemm/tests/test_grouped_moe_gemm.py:28-47 style inputs."""
    n, k = 384, 1024
    g = torch.Generator().manual_seed(19 + m)
    ap = torch.randint(0, 256, (m, k // 2), generator=g, dtype=torch.uint8)
    bp = torch.randint(0, 256, (n, k // 2), generator=g, dtype=torch.uint8)
    al = torch.randint(32, 80, (m, k // 16), generator=g, dtype=torch.uint8)
    bl = torch.randint(32, 80, (n, k // 16), generator=g, dtype=torch.uint8)
    sfa = torch.from_numpy(O.sf_linear_to_swizzled(al.numpy())).to(DEV)
    sfb = torch.from_numpy(O.sf_linear_to_swizzled(bl.numpy())).to(DEV)
    out = gemm(ap.to(DEV), sfa, bp.to(DEV), sfb, m, n, k, alpha=2.0 ** -8)
    want = O.gemm_bf16(ap.numpy(), al.numpy(), bp.numpy(), bl.numpy(), alpha=2.0 ** -8)
    assert_close(out, want, strict=False)


def test_epilogues_bias_residual_alpha():
    m, n, k = 200, 520, 768
    ap, sfa, bp, sfb = make_quantized(m, n, k, 41)
    g = torch.Generator().manual_seed(42)
    bias = (torch.randn(n, generator=g) * 0.02).to(torch.bfloat16).to(DEV)
    res = torch.randn(m, n, generator=g).to(torch.bfloat16).to(DEV)
    A, B = ap.cpu().numpy(), bp.cpu().numpy()
    la, lb = sf_linear(sfa, m, k), sf_linear(sfb, n, k)
    out = gemm(ap, sfa, bp, sfb, m, n, k, alpha=0.5, bias=bias)
    assert_close(out, O.gemm_bf16(A, la, B, lb, 0.5, bias_bits=bits(bias)))
    out = gemm(ap, sfa, bp, sfb, m, n, k, c=res, beta=1.0)
    assert_close(out, O.gemm_bf16(A, la, B, lb, 1.0, residual_bits=bits(res)))
    inplace = res.clone()                                  # C may alias D
    gemm(ap, sfa, bp, sfb, m, n, k, bias=bias, c=inplace, beta=1.0, out=inplace)
    assert_close(inplace, O.gemm_bf16(A, la, B, lb, 1.0, bias_bits=bits(bias), residual_bits=bits(res)))
    # small-M (swapped) epilogue
    m2 = 8
    ap2, sfa2 = quantize((torch.randn(m2, k, generator=g) * 0.25).to(torch.bfloat16).to(DEV))
    res2 = torch.randn(m2, n, generator=g).to(torch.bfloat16).to(DEV)
    out = gemm(ap2, sfa2, bp, sfb, m2, n, k, alpha=0.5, bias=bias, c=res2, beta=1.0)
    assert_close(out, O.gemm_bf16(ap2.cpu().numpy(), sf_linear(sfa2, m2, k), B, lb, 0.5, bias_bits=bits(bias),
                                  residual_bits=bits(res2)))


def test_poisoned_padding_and_untouched_output():
    """rows of the last 128-row scale group beyond M/N may hold anything; output
    beyond [M,N] is never written."""
    m, n, k = 70, 200, 512
    ap, sfa, bp, sfb = make_quantized(m, n, k, 77)
    want = oracle_out(ap, sfa, bp, sfb, m, n, k)
    for sf, rows in ((sfa, m), (sfb, n)):
        mask = np.ones(sf.numel(), bool)
        mask[O.sf_offsets(rows, k).reshape(-1)] = False
        sf[torch.from_numpy(mask).to(DEV)] = 0xFF          # NaN pattern in every padding byte
    buf = torch.full((m + 3, n), 7.0, dtype=torch.bfloat16, device=DEV)
    gemm(ap, sfa, bp, sfb, m, n, k, out=buf)
    assert_close(buf[:m], want)
    assert torch.all(buf[m:] == 7.0)


def test_graph_replay_bit_stable():
    m, n, k = 256, 512, 1024
    ap, sfa, bp, sfb = make_quantized(m, n, k, 5)
    eager = gemm(ap, sfa, bp, sfb, m, n, k)
    out = torch.zeros_like(eager)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        gemm(ap, sfa, bp, sfb, m, n, k, out=out)          # warm-up outside capture (attribute set-up)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            gemm(ap, sfa, bp, sfb, m, n, k, out=out)
    out.zero_()
    graph.replay(); torch.cuda.synchronize()
    first = out.clone()
    graph.replay(); torch.cuda.synchronize()
    assert torch.equal(first, out) and torch.equal(first, eager)


def test_rejections():
    L = capi.lib()
    ap, sfa, bp, sfb = make_quantized(16, 128, 128, 1)
    out = torch.empty(16, 128, dtype=torch.bfloat16, device=DEV)
    P, s = capi.ptr, capi.stream_ptr()
    assert L.frt_nvfp4_gemm_bf16(P(ap), P(sfa), P(bp), P(sfb), None, None, P(out), 16, 128, 112, 1.0, 0.0, s) == -2
    assert L.frt_nvfp4_gemm_bf16(P(ap), P(sfa), P(bp), P(sfb), None, None, P(out), 16, 100, 128, 1.0, 0.0, s) == -2
    assert L.frt_nvfp4_gemm_bf16(P(ap), P(sfa), None, P(sfb), None, None, P(out), 16, 128, 128, 1.0, 0.0, s) == -1
    assert L.frt_nvfp4_gemm_bf16(P(ap), P(sfa), P(bp), P(sfb), None, None, P(out), 16, 128, 128, 1.0, 1.0, s) == -1


@pytest.mark.parametrize("name,m,n,k", [("qkv", 4096, 6144, 4096), ("o", 4096, 4096, 4096),
                                        ("gate_up", 4096, 24576, 4096), ("down", 4096, 4096, 12288)])
def test_qwen3_8b_prefill_shapes(name, m, n, k):
    """Full-size Qwen3-8B-shaped linears: the whole output against an fp32 GPU
    matmul of the dequantised bytes, and 64 sampled rows against the CPU oracle."""
    g = torch.Generator().manual_seed(31 + n + k)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16).to(DEV)
    ap, sfa = quantize(a)
    bp, sfb = quantize(w)
    out = gemm(ap, sfa, bp, sfb, m, n, k)
    want = gpu_fp32_reference(ap, sfa, bp, sfb, m, n, k)
    rel, cos = O.gemm_error_metrics(out.cpu(), want.cpu())
    assert rel <= REL_FROB and cos >= COSINE, (rel, cos)
    idx = torch.randperm(m, generator=g)[:64]
    la, lb = sf_linear(sfa, m, k), sf_linear(sfb, n, k)
    sample = O.gemm_bf16(ap.cpu().numpy()[idx], la[idx], bp.cpu().numpy(), lb)
    rel, cos = O.gemm_error_metrics(out.cpu()[idx], sample)
    assert rel <= REL_FROB and cos >= COSINE, (rel, cos)
    assert device_status() == 0


def test_against_reference_cutlass_gemm():
    """The reference's own Sm100 CUTLASS kernel on the same bytes (when oracle/_ref has it)."""
    ref = ref_lib()
    if ref is None or not ref.ref_has_cutlass():
        pytest.skip("oracle/_ref built without the CUTLASS GEMM")
    import ctypes as C
    m, n, k = 512, 1024, 2048
    ap, sfa, bp, sfb = make_quantized(m, n, k, 99)
    out = gemm(ap, sfa, bp, sfb, m, n, k, alpha=0.75)
    rout = torch.zeros_like(out)
    P = capi.ptr
    ref.ref_gemm_sm100_bf16(P(ap), P(bp), P(rout), m, n, k, P(sfa), P(sfb), C.c_float(0.75), 0, capi.stream_ptr())
    torch.cuda.synchronize()
    rel, cos = O.gemm_error_metrics(out.cpu(), rout.cpu())
    assert rel <= 1e-3 and cos >= 0.9999, (rel, cos)


@pytest.mark.parametrize("m,n,k", [(64, 128, 96), (300, 256, 160), (16, 128, 32), (256, 512, 224)])
def test_k_not_a_multiple_of_64(m, n, k):
    """K % 64 != 0: the tensor cores read whole 64-element scale groups, so the scale bytes that pad the last
    group must not hold NaN patterns.  The quantisers of this library write them as zero whatever the buffer
    held before (here: 0x7F, the e4m3 NaN)."""
    g = torch.Generator().manual_seed(5 + k)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    ap, sfa = alloc_fp4(m, k, fill=0x7F)
    bp, sfb = alloc_fp4(n, k, fill=0x7F)
    quantize(x, ap, sfa)
    quantize(w, bp, sfb)
    out = gemm(ap, sfa, bp, sfb, m, n, k)
    assert not torch.isnan(out.float()).any()
    assert_close(out, oracle_out(ap, sfa, bp, sfb, m, n, k))
