"""GPU parity of the HBM-bound kernels, through the C ABI:
bit-exact against the CPU oracle and, where oracle/_ref is built, against the
reference's own CUDA kernels running on the same GPU."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from tests.gpu_common import (DEV, O, alloc_fp4, bits, capi, quantize, randn_bf16, ref_lib, sf_bytes,  # noqa: E402
                              sf_linear)

P = capi.ptr


def st():
    return capi.stream_ptr()


_KEEP = []


@pytest.fixture(autouse=True)
def _release_device_copies():
    yield
    torch.cuda.synchronize()
    _KEEP.clear()


def D(t):
    """device copy that stays alive until the test ends (a temporary would be
    freed, and its memory reused, before the asynchronous kernel reads it)"""
    d = t.to(DEV)
    _KEEP.append(d)
    return d


@pytest.mark.parametrize("rows,dim", [(1, 1024), (2, 4096), (31, 4096), (33, 4096), (127, 2048), (129, 4096),
                                      (16, 12288), (64, 16384), (130, 80), (5, 16)])
def test_sf_layout(rows, dim):
    g = torch.Generator().manual_seed(rows * 7 + dim)
    lin = torch.randint(0, 256, (rows, dim // 16), generator=g, dtype=torch.uint8)
    out = torch.full((sf_bytes(rows, dim),), 0xAB, dtype=torch.uint8, device=DEV)
    capi.check(capi.lib().frt_nvfp4_sf_linear_to_swizzled(P(D(lin)), P(out), rows, dim, st()))
    want = O.sf_linear_to_swizzled(lin.numpy())
    got = out.cpu().numpy()
    offs = O.sf_offsets(rows, dim).reshape(-1)
    np.testing.assert_array_equal(got[offs], want[offs])
    mask = np.ones(got.size, bool)
    mask[offs] = False
    # bytes that complete a real row's last 64-element group are written as zero (the tensor cores read
    # them); bytes of rows beyond `rows` are left alone
    nb, groups = dim // 16, (dim + 63) // 64
    k_pad = np.zeros(got.size, bool)
    r = np.arange(rows)
    for kb in range(nb, 4 * groups):
        k_pad[((r >> 7) * groups + (kb >> 2)) * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (kb & 3)] = True
    assert np.all(got[k_pad] == 0)
    assert np.all(got[mask & ~k_pad] == 0xAB)


@pytest.mark.parametrize("encoder", [0, 1])
@pytest.mark.parametrize("rows,dim,scale,dtype", [
    (1, 5120, 1.5, torch.bfloat16), (8, 5120, 1.5, torch.float16), (128, 512, 1.5, torch.bfloat16),
    (257, 4096, 1.0, torch.bfloat16), (63, 2048, 0.02, torch.bfloat16), (130, 4096, 0.25, torch.float16),
    (4096, 4096, 1.0, torch.bfloat16)])
def test_quantizer_bit_exact(rows, dim, scale, dtype, encoder):
    g = torch.Generator().manual_seed(8100 + rows + dim)
    x = (torch.randn(rows, dim, generator=g) * scale).to(dtype)
    x[0, :16] = 0                      # an all-zero block
    x[0, 16:32] = 2.0 ** -13           # scale rounds to zero
    x[0, 32] = -0.0
    if dim >= 64:
        x[0, 48:64] = -(2.0 ** -13)    # zero scale, negative values: q = -inf
    if rows > 1 and dim >= 48:
        ties = torch.tensor([6, .25, .75, 1.25, 1.75, 2.5, 3.5, 5, -.25, -.75, -1.25, -1.75, -2.5, -3.5, -5, -6])
        x[1, :16] = ties.to(dtype)                                    # scale 1.0: q hits every threshold
        up = ties.to(dtype).view(torch.int16) + 1                      # one ulp further from zero
        x[1, 16:32] = up.view(dtype)
        x[1, 16], x[1, 31] = 6.0, -6.0
        down = ties.to(dtype).view(torch.int16) - 1                    # one ulp nearer to zero
        x[1, 32:48] = down.view(dtype)
        x[1, 32] = 6.0
    prev = capi.lib().frt_set_option(1, encoder)
    try:
        packed, sf = alloc_fp4(rows, dim, fill=0)
        quantize(D(x), packed, sf)
    finally:
        capi.lib().frt_set_option(1, prev)
    want_p, want_s = O.quantize_nvfp4(x.float().numpy())
    np.testing.assert_array_equal(sf.cpu().numpy(), O.sf_linear_to_swizzled(want_s))
    np.testing.assert_array_equal(packed.cpu().numpy(), want_p)
    ref = ref_lib()
    if ref is not None:
        rp, rs = alloc_fp4(rows, dim, fill=0)
        fn = ref.ref_quantize_bf16_vec if dtype == torch.bfloat16 else ref.ref_quantize_fp16
        assert fn(P(D(x)), P(rp), P(rs), rows, dim, st()) == 0
        torch.cuda.synchronize()
        assert torch.equal(rp, packed) and torch.equal(rs, sf)


@pytest.mark.parametrize("encoder", [0, 1])
def test_quantizer_every_scale_byte(encoder):
    """one block per UE4M3 scale value 0x01..0x7E (amax = 6 * value), other elements random
    fractions of it: checks the reciprocal-scale table entry by entry"""
    lut = np.asarray(O.UE4M3_LUT, dtype=np.float32)
    g = torch.Generator().manual_seed(77)
    rows, dim = 126, 64
    x = torch.zeros(rows, dim)
    for b in range(1, 127):
        amax = 6.0 * float(lut[b])
        for blk in range(4):
            v = (torch.rand(16, generator=g) * 2 - 1) * amax
            v[blk] = amax if blk % 2 == 0 else -amax
            x[b - 1, 16 * blk:16 * blk + 16] = v
    x = x.bfloat16()
    prev = capi.lib().frt_set_option(1, encoder)
    try:
        packed, sf = alloc_fp4(rows, dim, fill=0)
        quantize(D(x), packed, sf)
    finally:
        capi.lib().frt_set_option(1, prev)
    want_p, want_s = O.quantize_nvfp4(x.float().numpy())
    assert set(np.unique(want_s)) >= set(range(1, 127))
    np.testing.assert_array_equal(sf.cpu().numpy(), O.sf_linear_to_swizzled(want_s))
    np.testing.assert_array_equal(packed.cpu().numpy(), want_p)


def test_dequantize_exact():
    rows, dim = 130, 1024
    g = torch.Generator().manual_seed(3)
    packed = torch.randint(0, 256, (rows, dim // 2), generator=g, dtype=torch.uint8)
    lin = torch.randint(0, 0x7F, (rows, dim // 16), generator=g, dtype=torch.uint8)
    sf = torch.from_numpy(O.sf_linear_to_swizzled(lin.numpy()))
    out = torch.empty(rows, dim, dtype=torch.float16, device=DEV)
    capi.check(capi.lib().frt_nvfp4_dequantize_fp16(P(D(packed)), P(D(sf)), P(out), rows, dim, st()))
    want = torch.from_numpy(O.dequantize_nvfp4(packed.numpy(), lin.numpy())).to(torch.float16)
    assert torch.equal(out.cpu().view(torch.int16), want.view(torch.int16))      # exact, signed zeros included


CASES = [(1, 1024), (16, 128), (131, 128), (37, 256), (100, 64), (45, 192), (63, 2048), (128, 4096), (257, 4096), (33, 5120), (9, 8192), (5, 12288), (3, 16384)]

# The norm kernels exist in two forms (one CTA per row group; persistent CTAs fed by bulk
# copies); the library picks one by row width.  FRT_OPT_NORM_FORM (key 5) forces each form, so
# every case is checked on both.
FORMS = [1, 2]


@pytest.fixture(params=FORMS, ids=["per_group", "streamed"])
def form(request):
    prev = capi.lib().frt_set_option(5, request.param)
    yield request.param
    capi.lib().frt_set_option(5, prev)


@pytest.mark.parametrize("rows,dim", CASES)
def test_rms_norm_bf16(rows, dim, form):
    x, w = randn_bf16((rows, dim), 23 + rows), randn_bf16((dim,), 24, 0.1, 1.0)
    out = torch.empty(rows, dim, dtype=torch.bfloat16, device=DEV)
    capi.check(capi.lib().frt_rms_norm_bf16(P(D(x)), P(D(w)), P(out), rows, dim, 1e-6, st()))
    np.testing.assert_array_equal(bits(out), O.rms_norm_bf16(bits(x), bits(w), 1e-6))
    ref = ref_lib()
    if ref is not None and dim % 2 == 0:
        ro = torch.empty_like(out)
        ref.ref_rms_norm_bf16(P(D(x)), P(D(w)), P(ro), rows, dim, C.c_float(1e-6), st())
        torch.cuda.synchronize()
        assert (ro.float() - out.float()).abs().max() <= 2.0 ** -6   # reference's own tolerance (p99 2^-6)
        assert (ro != out).float().mean() < 0.01


@pytest.mark.parametrize("rows,dim", CASES)
def test_residual_add_rms_norm_bf16(rows, dim, form):
    x, r, w = randn_bf16((rows, dim), 1 + rows), randn_bf16((rows, dim), 2 + rows), randn_bf16((dim,), 3, 0.1, 1.0)
    res = r.to(DEV).clone()
    out = torch.empty(rows, dim, dtype=torch.bfloat16, device=DEV)
    capi.check(capi.lib().frt_residual_add_rms_norm_bf16(P(res), P(D(x)), P(D(w)), P(out), rows, dim,
                                                         1e-6, st()))
    want_res, want_y = O.residual_add_rms_norm_bf16(bits(r), bits(x), bits(w), 1e-6)
    np.testing.assert_array_equal(bits(res), want_res)
    np.testing.assert_array_equal(bits(out), want_y)
    ref = ref_lib()
    if ref is not None:
        rres, ro = r.to(DEV).clone(), torch.empty_like(out)
        ref.ref_residual_add_rms_norm_bf16(P(rres), P(D(x)), P(D(w)), P(ro), rows, dim, C.c_float(1e-6), st())
        torch.cuda.synchronize()
        assert torch.equal(rres, res)                                   # in-place residual exactly equal
        assert (ro.float() - out.float()).abs().max() <= 2.0 ** -6


@pytest.mark.parametrize("encoder", [0, 1])
@pytest.mark.parametrize("rows,dim", CASES + [(4096, 4096), (1500, 3072), (700, 8192)])
def test_fused_residual_norm_quant(rows, dim, encoder, form):
    """residual_add_rms_norm_quant_nvfp4_swizzled_bf16 semantics, bit-exact
    against the oracle (same summation order) and, end to end, against the
    reference's fused kernel up to its different fp32 summation order."""
    x, r, w = randn_bf16((rows, dim), 11 + rows), randn_bf16((rows, dim), 12 + rows), randn_bf16((dim,), 13, 0.1, 1.0)
    res = r.to(DEV).clone()
    packed, sf = alloc_fp4(rows, dim)
    normed = torch.empty(rows, dim, dtype=torch.bfloat16, device=DEV)
    prev = capi.lib().frt_set_option(1, encoder)
    try:
        capi.check(capi.lib().frt_norm_quant_nvfp4(P(res), P(D(x)), P(D(w)), 1e-6, 1.0, P(normed),
                                                   P(packed), P(sf), rows, dim, 0, st()))
    finally:
        capi.lib().frt_set_option(1, prev)
    want = O.fused_norm_quant(bits(x), bits(w), 1e-6, res_bits=bits(r))
    np.testing.assert_array_equal(bits(res), want["residual"])
    np.testing.assert_array_equal(bits(normed), want["normed"])
    np.testing.assert_array_equal(sf.cpu().numpy(), O.sf_linear_to_swizzled(want["sf_linear"]))
    np.testing.assert_array_equal(packed.cpu().numpy(), want["packed"])
    ref = ref_lib()
    # the reference kernel runs dim/16 threads per row and sums only whole warps: it needs dim >= 512
    if ref is not None and ref.ref_has_cutlass() and 512 <= dim <= 16384:
        rres = r.to(DEV).clone()
        rp, rs = alloc_fp4(rows, dim)
        ref.ref_res_rms_fp4_bf16(P(rres), P(D(x)), P(D(w)), P(rp), P(rs), rows, dim, C.c_float(1e-6), st())
        torch.cuda.synchronize()
        assert torch.equal(rres, res)
        # rstd may differ in the last bit (other summation order): allow a sliver of code flips
        code_mismatch = (O.unpack_codes(rp.cpu().numpy()) != O.unpack_codes(packed.cpu().numpy())).mean()
        sf_mismatch = (rs != sf).float().mean().item()
        assert code_mismatch < 2e-3 and sf_mismatch < 2e-3, (code_mismatch, sf_mismatch)


@pytest.mark.parametrize("rows,dim", [(1, 2048), (63, 2048), (257, 4096)])
def test_rms_norm_quantize_emits_normed(rows, dim):
    """rms_norm_quantize_fp4_sfa_bf16 semantics ((1+w), bf16-rounded, `normed`
    emitted): quantiser(normed) bit-exact, normed within one bf16 step of the
    reference kernel."""
    x, w = randn_bf16((rows, dim), 2026 + rows, 0.2), randn_bf16((dim,), 2027, 0.05)
    packed, sf = alloc_fp4(rows, dim)
    normed = torch.empty(rows, dim, dtype=torch.bfloat16, device=DEV)
    flags = 1 | 2
    capi.check(capi.lib().frt_norm_quant_nvfp4(None, P(D(x)), P(D(w)), 1e-6, 1.0, P(normed), P(packed),
                                               P(sf), rows, dim, flags, st()))
    want = O.fused_norm_quant(bits(x), bits(w), 1e-6, flags=flags)
    np.testing.assert_array_equal(bits(normed), want["normed"])
    np.testing.assert_array_equal(packed.cpu().numpy(), want["packed"])
    np.testing.assert_array_equal(sf_linear(sf, rows, dim), want["sf_linear"])
    qp, qs = quantize(normed)                      # the stand-alone quantiser on our own normed
    assert torch.equal(qp, packed) and torch.equal(qs, sf)
    expected = (x.float() * torch.rsqrt(x.float().square().mean(dim=1, keepdim=True) + 1e-6)
                * (1.0 + w.float())).bfloat16()
    assert (normed.cpu().float() - expected.float()).abs().max() <= 0.015625
    ref = ref_lib()
    if ref is not None and dim <= 8192:
        rn, (rp, rs) = torch.empty_like(normed), alloc_fp4(rows, dim)
        assert ref.ref_rms_norm_quantize_bf16(P(D(x)), P(D(w)), C.c_float(1e-6), P(rn), P(rp), P(rs),
                                              rows, dim, st()) == 0
        torch.cuda.synchronize()
        assert (rn.float() - normed.float()).abs().max() <= 0.015625
        assert (rn != normed).float().mean() < 0.01


def test_rule_b_variant():
    rows, dim = 33, 2048
    x, r, w = randn_bf16((rows, dim), 5), randn_bf16((rows, dim), 6), randn_bf16((dim,), 7, 0.1, 1.0)
    res = r.to(DEV).clone()
    packed, sf = alloc_fp4(rows, dim)
    flags = 2 | 4 | 8
    capi.check(capi.lib().frt_norm_quant_nvfp4(P(res), P(D(x)), P(D(w)), 1e-6, 1.0, None, P(packed), P(sf),
                                               rows, dim, flags, st()))
    want = O.fused_norm_quant(bits(x), bits(w), 1e-6, res_bits=bits(r), flags=flags)
    np.testing.assert_array_equal(bits(res), want["residual"])
    np.testing.assert_array_equal(packed.cpu().numpy(), want["packed"])
    np.testing.assert_array_equal(sf_linear(sf, rows, dim), want["sf_linear"])


def test_two_level_global_scale():
    rows, dim = 17, 4096
    x, r, w = randn_bf16((rows, dim), 8), randn_bf16((rows, dim), 9), randn_bf16((dim,), 10, 0.1, 1.0)
    base = O.fused_norm_quant(bits(x), bits(w), 1e-6, res_bits=bits(r))
    amax = np.abs(O.bf16_bits_to_f32(base["normed"])).max()
    g = np.float32(amax) / np.float32(6 * 448)
    inv_g = float(np.float32(1.0) / g)
    res = r.to(DEV).clone()
    packed, sf = alloc_fp4(rows, dim)
    capi.check(capi.lib().frt_norm_quant_nvfp4(P(res), P(D(x)), P(D(w)), 1e-6, inv_g, None, P(packed),
                                               P(sf), rows, dim, 0, st()))
    want = O.fused_norm_quant(bits(x), bits(w), 1e-6, res_bits=bits(r), inv_global_scale=inv_g)
    np.testing.assert_array_equal(packed.cpu().numpy(), want["packed"])
    np.testing.assert_array_equal(sf_linear(sf, rows, dim), want["sf_linear"])


def test_argument_errors():
    L = capi.lib()
    x = torch.zeros(4, 64, dtype=torch.bfloat16, device=DEV)
    p, s = alloc_fp4(4, 64)
    assert L.frt_nvfp4_quantize(None, 0, P(p), P(s), 4, 64, st()) == -1
    assert L.frt_nvfp4_quantize(P(x), 0, P(p), P(s), 4, 40, st()) == -2          # dim % 16
    assert L.frt_nvfp4_quantize(P(x), 0, P(p), P(s), 0, 64, st()) == -2
    assert L.frt_nvfp4_quantize(C.c_void_p(x.data_ptr() + 2), 0, P(p), P(s), 4, 64, st()) == -3
    assert L.frt_norm_quant_nvfp4(None, P(x), None, 1e-6, 1.0, None, P(p), P(s), 4, 32768, 0, st()) == -4
    assert L.frt_nvfp4_sf_linear_to_swizzled(P(s), P(s), 0, 64, st()) == -2
    assert b"null" in L.frt_error_string(-1)


@pytest.mark.parametrize("rows,dim", CASES)
def test_layer_norm_bf16(rows, dim):
    x, w, b = randn_bf16((rows, dim), 41 + rows, 1.0, 0.3), randn_bf16((dim,), 42, 0.1, 1.0), randn_bf16((dim,), 43, 0.2)
    out = torch.empty(rows, dim, dtype=torch.bfloat16, device=DEV)
    capi.check(capi.lib().frt_layer_norm_bf16(P(D(x)), P(D(w)), P(D(b)), P(out), rows, dim, 1e-5, st()))
    np.testing.assert_array_equal(bits(out), O.layer_norm_bf16(bits(x), bits(w), bits(b), 1e-5))
    want = torch.nn.functional.layer_norm(x.float(), (dim,), w.float(), b.float(), 1e-5)
    assert (out.float().cpu() - want).abs().max() <= 2.0 ** -5        # bf16 rounding of values of a few units
    ref = ref_lib()
    if ref is not None:
        ro = torch.empty_like(out)
        ref.ref_layer_norm_bf16(P(D(x)), P(D(w)), P(D(b)), P(ro), rows, dim, C.c_float(1e-5), st())
        torch.cuda.synchronize()
        assert (ro.float() - out.float()).abs().max() <= 2.0 ** -5
        assert (ro != out).float().mean() < 0.02


@pytest.mark.parametrize("with_residual", [False, True])
@pytest.mark.parametrize("rows,dim", [(1, 1024), (63, 2048), (257, 4096), (9, 8192)])
def test_rms_norm_quant_fp8_static(rows, dim, with_residual):
    x, r, w = randn_bf16((rows, dim), 51 + rows), randn_bf16((rows, dim), 52 + rows), randn_bf16((dim,), 53, 0.1, 1.0)
    scale_v = 0.037
    scale = torch.tensor([scale_v], dtype=torch.float32, device=DEV)
    out = torch.empty(rows, dim, dtype=torch.uint8, device=DEV)
    res = r.to(DEV).clone()
    capi.check(capi.lib().frt_rms_norm_quant_fp8(P(res) if with_residual else None, P(D(x)), P(D(w)), P(scale), P(out),
                                                 rows, dim, 1e-6, st()))
    want_res, want = O.rms_norm_quant_fp8(bits(x), bits(w), scale_v, 1e-6, res_bits=bits(r) if with_residual else None)
    np.testing.assert_array_equal(out.cpu().numpy(), want)
    if with_residual:
        np.testing.assert_array_equal(bits(res), want_res)
    ref = ref_lib()
    if ref is not None:
        ro = torch.empty_like(out)
        rres = r.to(DEV).clone()
        ref.ref_rms_norm_quant_fp8(P(rres) if with_residual else None, P(D(x)), P(D(w)), P(ro), rows, dim,
                                   C.c_float(1e-6), P(scale), st())
        torch.cuda.synchronize()
        if with_residual:
            assert torch.equal(rres, res)
        # other summation order and the approximate rsqrt: a sliver of values lands on the other side of an
        # e4m3 rounding boundary, one code step away
        assert (ro != out).float().mean() < 0.02
        d = (ro.view(torch.float8_e4m3fn).float() - out.view(torch.float8_e4m3fn).float()).abs()
        assert (d <= 0.13 * out.view(torch.float8_e4m3fn).float().abs() + 2.0 ** -9).all()


def test_norm_package_torch_ops():
    import flashrt_residual_norm_quant as pkg
    rows, dim = 33, 1024
    x, r, w, b = (randn_bf16((rows, dim), 61).to(DEV), randn_bf16((rows, dim), 62).to(DEV),
                  randn_bf16((dim,), 63, 0.1, 1.0).to(DEV), randn_bf16((dim,), 64, 0.2).to(DEV))
    scale = torch.tensor([0.05], dtype=torch.float32, device=DEV)
    y = pkg.layer_norm_bf16(x, w, b)
    np.testing.assert_array_equal(bits(y), O.layer_norm_bf16(bits(x), bits(w), bits(b), 1e-5))
    q = pkg.rms_norm_quant_fp8_static_bf16(x, w, scale)
    assert q.dtype == torch.float8_e4m3fn
    np.testing.assert_array_equal(q.view(torch.uint8).cpu().numpy(), O.rms_norm_quant_fp8(bits(x), bits(w), 0.05, 1e-6)[1])
    res = r.clone()
    q2 = pkg.residual_add_rms_norm_quant_fp8_static_bf16(res, x, w, scale)
    want_res, want = O.rms_norm_quant_fp8(bits(x), bits(w), 0.05, 1e-6, res_bits=bits(r))
    np.testing.assert_array_equal(q2.view(torch.uint8).cpu().numpy(), want)
    np.testing.assert_array_equal(bits(res), want_res)
    with pytest.raises(RuntimeError, match="float8_e4m3fn"):
        pkg.rms_norm_quant_fp8_static_bf16(x, w, scale, out=torch.empty_like(x))


@pytest.mark.parametrize("rows,dim", [(1, 1024), (63, 2048), (257, 4096), (9, 8192)])
def test_fp16_residual_norm_quant(rows, dim):
    """residual_add_rms_norm_fp4_sfa_v2_fp16: fp16 activations and residual, unweighted, eps 1e-6"""
    g = torch.Generator().manual_seed(700 + rows)
    x = torch.randn(rows, dim, generator=g).to(torch.float16)
    r = torch.randn(rows, dim, generator=g).to(torch.float16)
    res = r.to(DEV).clone()
    packed, sf = alloc_fp4(rows, dim)
    capi.check(capi.lib().frt_residual_norm_quant_nvfp4_fp16(P(res), P(D(x)), 1e-6, P(packed), P(sf), rows, dim, st()))
    want = O.residual_norm_quant_fp16(r.numpy(), x.numpy(), 1e-6)
    assert torch.equal(res.cpu(), torch.from_numpy(want["residual"]))
    np.testing.assert_array_equal(sf.cpu().numpy(), O.sf_linear_to_swizzled(want["sf_linear"]))
    np.testing.assert_array_equal(packed.cpu().numpy(), want["packed"])
    ref = ref_lib()
    if ref is not None and ref.ref_has_cutlass() and dim >= 512:
        rres = r.to(DEV).clone()
        rp, rs = alloc_fp4(rows, dim)
        ref.ref_res_rms_fp4_v2_fp16(P(rres), P(D(x)), P(rp), P(rs), rows, dim, st())
        torch.cuda.synchronize()
        assert torch.equal(rres, res)
        code_mismatch = (O.unpack_codes(rp.cpu().numpy()) != O.unpack_codes(packed.cpu().numpy())).mean()
        assert code_mismatch < 2e-3 and (rs != sf).float().mean().item() < 2e-3
    import fp4_fused_ops
    res2 = r.to(DEV).clone()
    p2, s2 = fp4_fused_ops.residual_add_rms_norm_fp4_sfa_v2_fp16(res2, x.to(DEV))
    assert torch.equal(p2, packed) and torch.equal(res2, res)


@pytest.mark.parametrize("tokens,heads_a,heads_b,head_dim,extra", [(37, 32, 8, 128, 1024), (5, 4, 0, 64, 0), (130, 3, 2, 256, 48),
                                                                   (9, 2, 2, 512, 512)])
def test_rms_norm_heads_in_place_equals_per_head_norm(tokens, heads_a, heads_b, head_dim, extra):
    """frt_rms_norm_heads_bf16 (the q and k heads of a stacked q/k/v output, in place, one launch) against
    frt_rms_norm_bf16 of each head group's contiguous copy: bit-equal; the columns after the heads stay untouched."""
    width = (heads_a + heads_b) * head_dim + extra
    x = randn_bf16((tokens, width), 5 + tokens).to(DEV)
    wa, wb = randn_bf16((head_dim,), 6, 0.1, 1.0).to(DEV), randn_bf16((head_dim,), 7, 0.1, 1.0).to(DEV)
    L = capi.lib()
    want = x.clone()
    for lo, n, w in ((0, heads_a, wa), (heads_a * head_dim, heads_b, wb)):
        if n == 0:
            continue
        part = x[:, lo:lo + n * head_dim].reshape(tokens * n, head_dim).contiguous()
        out = torch.empty_like(part)
        capi.check(L.frt_rms_norm_bf16(P(part), P(w), P(out), tokens * n, head_dim, 1e-6, st()))
        want[:, lo:lo + n * head_dim] = out.view(tokens, n * head_dim)
    got = x.clone()
    capi.check(L.frt_rms_norm_heads_bf16(P(got), tokens, width, head_dim, heads_a, P(wa), heads_b, P(wb) if heads_b else None,
                                         1e-6, st()))
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    # argument checks
    assert L.frt_rms_norm_heads_bf16(P(got), tokens, width, 48, 1, P(wa), 0, None, 1e-6, st()) == -4
    assert L.frt_rms_norm_heads_bf16(P(got), tokens, head_dim, head_dim, heads_a + 1, P(wa), heads_b, P(wb), 1e-6, st()) == -2
    assert L.frt_rms_norm_heads_bf16(P(got), tokens, width, head_dim, heads_a, P(wa), 1, None, 1e-6, st()) == -1
