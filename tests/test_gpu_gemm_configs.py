"""GPU parity of the NVFP4 GEMM at the full layer shapes of the decode sweep (Qwen3-8B linears at
1 / 4 / 16 / 64 tokens) and of the Llama-3-70B FFN (8192 tokens, whole and column-sharded).

Oracle: dequantise the exact bytes the kernel consumed, fp32 matmul, bf16
(fp4-gemm/tests/test_fp4_gemm.py:593-636).  Tolerance: relative Frobenius error <= 1e-2 and cosine >= 0.999.
Tier structure follows the reference's small-M gate (fp4-gemm/tests/test_fp4_gemm.py:801-1010): multi-row
results equal the per-row GEMV bit for bit, and shapes follow its coverage note
(fp4-gemm/docs/tile-and-shape-coverage.md:83-160).
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from tests.gpu_common import DEV, O, capi, device_status, gemm, quantize, ref_lib, sf_linear  # noqa: E402

REL_FROB, COSINE = 1e-2, 0.999

QWEN3_8B = {"qkv": (6144, 4096), "o": (4096, 4096), "gate_up": (24576, 4096), "down": (4096, 12288)}


def plan(m, n, k):
    cfg, split = C.c_int(0), C.c_int(0)
    capi.check(capi.lib().frt_nvfp4_gemm_plan(m, n, k, C.byref(cfg), C.byref(split)))
    return cfg.value, split.value


def check(got, want):
    rel, cos = O.gemm_error_metrics(got.cpu(), want.cpu() if torch.is_tensor(want) else want)
    assert rel <= REL_FROB and cos >= COSINE, (rel, cos)


@pytest.fixture(scope="module", params=sorted(QWEN3_8B))
def layer(request):
    """One Qwen3-8B linear: N(0, 0.02) bf16 weights packed by the library's quantiser, plus the dequantised
    fp32 weight on the host and on the device (shared by every token count)."""
    n, k = QWEN3_8B[request.param]
    g = torch.Generator().manual_seed(900 + n + k)
    w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16).to(DEV)
    bp, sfb = quantize(w)
    torch.cuda.synchronize()
    wdq = O.dequantize_nvfp4(bp.cpu().numpy(), sf_linear(sfb, n, k))
    return dict(name=request.param, n=n, k=k, bp=bp, sfb=sfb, wdq=wdq, wdq_dev=torch.from_numpy(wdq).to(DEV))


def activations(m, k, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    return quantize(x)


@pytest.mark.parametrize("m", [1, 4, 16, 64])
def test_decode_sweep_full_layer_shapes(layer, m):
    """every output of the M-token GEMM against the CPU oracle (all rows) and against the fp32 GPU matmul"""
    n, k = layer["n"], layer["k"]
    ap, sfa = activations(m, k, 40 + m)
    out = gemm(ap, sfa, layer["bp"], layer["sfb"], m, n, k)
    adq = O.dequantize_nvfp4(ap.cpu().numpy(), sf_linear(sfa, m, k))
    want_cpu = torch.from_numpy(adq @ layer["wdq"].T).to(torch.bfloat16)
    check(out, want_cpu)
    want_gpu = (torch.from_numpy(adq).to(DEV) @ layer["wdq_dev"].T).to(torch.bfloat16)
    check(out, want_gpu)
    assert device_status() == 0


def test_64_token_split_k_path(layer):
    """The 64-token o and down projections (32 weight tiles for 148 SMs, two CTAs per SM) run as clusters of
    eight CTAs that share a tile's K and sum their partials through distributed shared memory, qkv (48 tiles)
    as clusters of four; gate/up runs unsplit.  The split result is checked against the oracle and against the
    same kernel with the split turned off."""
    n, k, m = layer["n"], layer["k"], 64
    cfg, split = plan(m, n, k)
    assert cfg == 13
    assert split == {"o": 8, "down": 8, "qkv": 4, "gate_up": 1}[layer["name"]]
    ap, sfa = activations(m, k, 77)
    out = gemm(ap, sfa, layer["bp"], layer["sfb"], m, n, k)
    adq = O.dequantize_nvfp4(ap.cpu().numpy(), sf_linear(sfa, m, k))
    check(out, torch.from_numpy(adq @ layer["wdq"].T).to(torch.bfloat16))
    prev = capi.lib().frt_set_option(7, 0)              # FRT_OPT_GEMM_SPLIT_K off
    try:
        assert plan(m, n, k) == (13, 1)
        unsplit = gemm(ap, sfa, layer["bp"], layer["sfb"], m, n, k)
    finally:
        capi.lib().frt_set_option(7, prev)
    check(out, unsplit)
    d = (out.float() - unsplit.float()).abs()
    # same products, another fp32 summation order: at most one bf16 step apart
    assert float((d / unsplit.float().abs().clamp_min(2.0 ** -6)).max()) <= 2.0 ** -6
    assert device_status() == 0


@pytest.mark.parametrize("m", [2, 4, 7, 8, 16])
def test_rows_equal_per_row_gemv_bitwise(layer, m):
    """fp4-gemm/tests/test_fp4_gemm.py:909-945: each row of the multi-row result equals the one-row GEMV of
    that row bit for bit (1..16 tokens share one kernel configuration and split, hence one summation order)"""
    n, k = layer["n"], layer["k"]
    assert plan(m, n, k) == plan(1, n, k)
    g = torch.Generator().manual_seed(5 + m)
    x = (torch.randn(m, k, generator=g) * 0.25).to(torch.bfloat16).to(DEV)
    ap, sfa = quantize(x)
    rows = gemm(ap, sfa, layer["bp"], layer["sfb"], m, n, k)
    diffs = 0
    for r in range(m):
        ar, sr = quantize(x[r:r + 1].contiguous())
        one = gemm(ar, sr, layer["bp"], layer["sfb"], 1, n, k)
        diffs += int((rows[r].view(torch.int16) != one[0].view(torch.int16)).sum())
    assert diffs == 0
    assert device_status() == 0


# ---- Llama-3-70B FFN, 8192 tokens: whole layers and the column shards of 2 / 4 / 8 GPUs ------------------
LLAMA70B = [("gate_up", 57344, 8192), ("down", 8192, 28672)]


@pytest.mark.parametrize("name,n,k", LLAMA70B)
def test_llama3_70b_ffn_shapes_and_column_shards(name, n, k):
    m = 8192
    g = torch.Generator().manual_seed(70 + n)
    ap, sfa = quantize(torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV))
    idx = torch.randperm(m, generator=g)[:64]
    la = sf_linear(sfa, m, k)
    a_rows = O.dequantize_nvfp4(ap.cpu().numpy()[idx], la[idx])
    adq_dev = torch.from_numpy(O.dequantize_nvfp4(ap.cpu().numpy(), la)).to(DEV)
    # the weight in column slabs of N/8 rows: a slab is one 8-GPU shard, 2 / 4 slabs the wider shards; packed
    # rows and swizzled scales of a shard are contiguous byte ranges of the whole weight's buffers
    slab = n // 8
    assert slab % 128 == 0
    bp = torch.empty(n, k // 2, dtype=torch.uint8, device=DEV)
    sfb = torch.empty(int(capi.lib().frt_nvfp4_sf_swizzled_bytes(n, k)), dtype=torch.uint8, device=DEV)
    sf_slab = sfb.numel() // 8
    for s in range(8):
        w = (torch.randn(slab, k, generator=g) * 0.02).to(torch.bfloat16).to(DEV)
        quantize(w, bp[s * slab:(s + 1) * slab], sfb[s * sf_slab:(s + 1) * sf_slab])
        del w
    torch.cuda.synchronize()

    sf_per_group = sfb.numel() // (n // 128)             # scale bytes of one 128-row group of the weight

    whole = gemm(ap, sfa, bp, sfb, m, n, k)
    assert plan(m, n, k) == (4, 1)
    samples = []                                         # CPU-oracle outputs of the 64 sampled token rows, per slab
    for s in range(8):                                   # the whole output, one slab of reference at a time
        c0, c1 = s * slab, (s + 1) * slab
        wdq = O.dequantize_nvfp4(bp[c0:c1].cpu().numpy(),
                                 sf_linear(sfb[c0 // 128 * sf_per_group:c1 // 128 * sf_per_group], slab, k))
        full = (adq_dev @ torch.from_numpy(wdq).to(DEV).T).to(torch.bfloat16)
        samples.append(torch.from_numpy(a_rows @ wdq.T).to(torch.bfloat16))
        check(whole[:, c0:c1], full)
        check(whole[idx.to(DEV)][:, c0:c1], samples[-1])
        del full, wdq
    # column shards as separate calls on the shard's byte ranges: N/2, N/4, N/8 wide
    for world in (2, 4, 8):
        width = n // world
        for rank in sorted({0, world - 1}):
            c0 = rank * width
            sf0 = c0 // 128 * sf_per_group
            out = gemm(ap, sfa, bp[c0:c0 + width], sfb[sf0:sf0 + width // 128 * sf_per_group], m, width, k)
            # another tile raster may sum in another order: equal or within a tenth of the tolerance
            assert O.gemm_error_metrics(out.cpu(), whole[:, c0:c0 + width].cpu())[0] <= 1e-3
            check(out[idx.to(DEV)], torch.cat(samples[c0 // slab:(c0 + width) // slab], dim=1))
    assert device_status() == 0


# ---- the reference's own Sm100 CUTLASS kernel on the same bytes ------------------------------------------
@pytest.mark.parametrize("name,m,n,k", [("qkv", 4096, 6144, 4096), ("o", 4096, 4096, 4096),
                                        ("gate_up", 4096, 24576, 4096), ("down", 4096, 4096, 12288)])
def test_against_reference_cutlass_gemm_prefill_shapes(name, m, n, k):
    """fp4-gemm/csrc/gemm/fp4/cutlass_nvfp4_w4a16_gemm_sm100.cu (default and widen tiles) compiled unmodified
    into oracle/_ref.  Where that library exists it must contain the CUTLASS kernels: a build that lost them
    fails here instead of skipping."""
    ref = ref_lib()
    if ref is None:
        pytest.skip("oracle/_ref/libflashrt_ref.so not built (no reference checkout at build time)")
    if not ref.ref_has_cutlass():
        pytest.fail("oracle/_ref was built without the reference's CUTLASS Sm100 GEMM")
    g = torch.Generator().manual_seed(3 + n + k)
    ap, sfa = quantize(torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV))
    bp, sfb = quantize((torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16).to(DEV))
    out = gemm(ap, sfa, bp, sfb, m, n, k, alpha=0.75)
    P = capi.ptr
    for variant in (0, 1):                                # default tile, widen tile
        rout = torch.zeros_like(out)
        rc = ref.ref_gemm_sm100_bf16(P(ap), P(bp), P(rout), m, n, k, P(sfa), P(sfb), C.c_float(0.75), variant,
                                     capi.stream_ptr())
        torch.cuda.synchronize()
        assert rc == 0, (variant, rc)
        rel, cos = O.gemm_error_metrics(out.cpu(), rout.cpu())
        assert rel <= 1e-3 and cos >= 0.9999, (variant, rel, cos)


# ---- bind-time interleaved weight layout of the one-row GEMV ----------------------------------------------
@pytest.mark.parametrize("n,k", [(17408, 5120), (5120, 17408), (1024, 5120), (4096, 4096), (4104, 320)])
def test_interleaved_repack_and_gemv(n, k):
    """fp4-gemm/tests/test_fp4_gemm.py:806-836: the repack equals the host byte permutation
    b.view(N/8, 8, K/64, 32).permute(0, 2, 1, 3), and the GEMV over the repacked weight equals the plain-layout
    GEMV bit for bit (random weight bytes, constant 0x38 scales, as the reference's gate uses)."""
    import fp4_gemm
    g = torch.Generator(device=DEV).manual_seed(20260815 % 1000 + n)
    a = torch.randint(0, 256, (1, k // 2), device=DEV, dtype=torch.uint8, generator=g)
    b = torch.randint(0, 256, (n, k // 2), device=DEV, dtype=torch.uint8, generator=g)
    sfa = torch.full((int(capi.lib().frt_nvfp4_sf_swizzled_bytes(1, k)),), 0x38, device=DEV, dtype=torch.uint8)
    sfb = torch.full((int(capi.lib().frt_nvfp4_sf_swizzled_bytes(n, k)),), 0x38, device=DEV, dtype=torch.uint8)
    b_ilv = fp4_gemm.fp4_repack_b_interleaved_sm120(b)
    host = b.view(n // 8, 8, k // 64, 32).permute(0, 2, 1, 3).contiguous().view_as(b)
    assert torch.equal(b_ilv, host)
    base = fp4_gemm.fp4_w4a4_gemv_warpsplit_bf16(a, b, sfa, sfb, alpha=2.0 ** -6)
    got = fp4_gemm.fp4_w4a4_gemv_warpsplit_interleaved_bf16(a, b_ilv, sfa, sfb, alpha=2.0 ** -6)
    torch.cuda.synchronize()
    assert torch.equal(got, base)
    want = O.gemm_bf16(a.cpu().numpy(), sf_linear(sfa, 1, k), b.cpu().numpy(), sf_linear(sfb, n, k), alpha=2.0 ** -6)
    check(got, want)
    with pytest.raises(RuntimeError, match="M=1 only"):
        fp4_gemm.fp4_w4a4_gemv_warpsplit_interleaved_bf16(torch.cat([a, a]), b_ilv, sfa, sfb,
                                                          out=torch.empty((2, n), device=DEV, dtype=torch.bfloat16))
    assert device_status() == 0


# ---- tuning overrides of the small-M form keep the result --------------------------------------------------
@pytest.mark.parametrize("m,depth,split", [(1, 2, 0), (1, 3, 8), (16, 2, 4), (24, 3, 0), (24, 2, 2), (64, 3, 0), (64, 3, 4), (64, 8, 0), (64, 8, 4)])
def test_small_m_ring_depth_and_split_overrides(m, depth, split):
    """FRT_OPT_SMALLM_STAGES (shallower shared-memory rings, more CTAs per SM) and a forced FRT_OPT_GEMM_SPLIT_K run
    other instantiations of the weight-streaming kernel; every one must give the oracle's result."""
    n, k = 1024, 4096
    g = torch.Generator().manual_seed(m * 7 + depth)
    ap, sfa = quantize((torch.randn(m, k, generator=g) * 0.5).to(torch.bfloat16).to(DEV))
    bp, sfb = quantize((torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16).to(DEV))
    L = capi.lib()
    prev = L.frt_set_option(8, depth), L.frt_set_option(7, split)
    try:
        assert plan(m, n, k)[1] == max(split, 1)         # 0 = never split, >= 2 = that many CTAs per tile
        out = gemm(ap, sfa, bp, sfb, m, n, k)
    finally:
        L.frt_set_option(8, prev[0]); L.frt_set_option(7, prev[1])
    check(out, O.gemm_bf16(ap.cpu().numpy(), sf_linear(sfa, m, k), bp.cpu().numpy(), sf_linear(sfb, n, k)))
    assert device_status() == 0


def test_bounded_wait_runs_out_and_the_context_stays_usable():
    """A device-side wait that nothing satisfies gives up after its clock budget, reports through the status word
    and returns: here the wait for a peer flag of an epoch that no rank ever publishes, with the budget lowered to
    2^20 clocks.  The stream stays usable: the next GEMM on it is correct and the status word is clean again."""
    L, P = capi.lib(), capi.ptr
    flags = torch.zeros(8, dtype=torch.int32, device=DEV)
    prev = L.frt_set_option(9, 20)                       # FRT_OPT_WAIT_LIMIT_LOG2
    try:
        capi.check(L.frt_peer_wait(P(flags), 2, 1, capi.stream_ptr()))
        torch.cuda.synchronize()
    finally:
        L.frt_set_option(9, prev)
    assert device_status() == 0x400
    assert device_status() == 0                          # reading the word clears it
    flags[:2] = 5                                        # published epochs: the same wait now returns at once
    capi.check(L.frt_peer_wait(P(flags), 2, 5, capi.stream_ptr()))
    m, n, k = 64, 256, 512
    g = torch.Generator().manual_seed(3)
    ap, sfa = quantize((torch.randn(m, k, generator=g) * 0.5).to(torch.bfloat16).to(DEV))
    bp, sfb = quantize((torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16).to(DEV))
    out = gemm(ap, sfa, bp, sfb, m, n, k)
    check(out, O.gemm_bf16(ap.cpu().numpy(), sf_linear(sfa, m, k), bp.cpu().numpy(), sf_linear(sfb, n, k)))
    assert device_status() == 0


@pytest.mark.parametrize("m,n,k", [(1, 4096, 4096), (3, 6144, 4096), (16, 4096, 12288), (64, 4096, 12288)])
def test_split_k_results_are_bit_stable_over_repeated_launches(m, n, k):
    """The cluster split-K forms (partials pushed to the owning CTA up to 16 token columns, pulled between two
    cluster barriers above) add their partials in rank order: 100 back-to-back launches into a poisoned output give
    the same bytes every time (a race in the exchange would not)."""
    assert plan(m, n, k)[1] > 1
    g = torch.Generator().manual_seed(m + n + k)
    ap = torch.randint(0, 256, (m, k // 2), generator=g, dtype=torch.uint8).to(DEV)
    bp = torch.randint(0, 256, (n, k // 2), generator=g, dtype=torch.uint8).to(DEV)
    L = capi.lib()
    sfa = torch.randint(32, 80, (int(L.frt_nvfp4_sf_swizzled_bytes(m, k)),), generator=g, dtype=torch.uint8).to(DEV)
    sfb = torch.randint(32, 80, (int(L.frt_nvfp4_sf_swizzled_bytes(n, k)),), generator=g, dtype=torch.uint8).to(DEV)
    ref = gemm(ap, sfa, bp, sfb, m, n, k).clone()
    out = torch.empty_like(ref)
    for it in range(100):
        out.fill_(7.0)
        gemm(ap, sfa, bp, sfb, m, n, k, out=out)
        if it % 25 == 24:
            torch.cuda.synchronize()
            assert torch.equal(out, ref)
    assert device_status() == 0
