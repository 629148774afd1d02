"""GPU parity of the grouped (MoE) NVFP4 GEMM, through the C ABI and the torch
op layer.  Inputs and tolerances follow grouped-moe-gemm/tests/test_grouped_moe_gemm.py:
random packed bytes (all 16 codes, -0 included), random scale bytes in [32,80),
alpha ~ U(0.5,1.5); pass: cosine >= 0.999, rel-L2 <= 0.0025, max_rel <= 0.01."""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from tests.gpu_common import DEV, O, capi, device_status, sf_bytes  # noqa: E402

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "flashrt-hf-kernels_b200" / "torch-ext"))


@pytest.fixture(autouse=True, params=[1, 2], ids=["weight_major", "token_major"])
def grouped_form(request):
    """every case runs on both forms of the grouped kernel (FRT_OPT_GROUPED_FORM, key 10): expert weights on the
    256-row axis with a transposed output tile, and token rows on the 256-row axis"""
    prev = capi.lib().frt_set_option(10, request.param)
    yield request.param
    capi.lib().frt_set_option(10, prev)


def make_inputs(rows, n, k, experts, seed):
    g = torch.Generator().manual_seed(seed)
    ap = torch.randint(0, 256, (rows, k // 2), generator=g, dtype=torch.uint8)
    wp = torch.randint(0, 256, (experts, n, k // 2), generator=g, dtype=torch.uint8)
    al = torch.randint(32, 80, (rows, k // 16), generator=g, dtype=torch.uint8)
    wl = torch.randint(32, 80, (experts, n, k // 16), generator=g, dtype=torch.uint8)
    alpha = torch.rand(experts, generator=g) + 0.5
    asw = torch.from_numpy(O.sf_linear_to_swizzled(al.numpy()))
    wsw = torch.stack([torch.from_numpy(O.sf_linear_to_swizzled(wl[e].numpy())) for e in range(experts)])
    return ap, wp, al, wl, alpha, asw, wsw


def run_capi(ap, wp, asw, wsw, alpha, out, offsets=None, tile_expert=None, tile_rows=0):
    L, P = capi.lib(), capi.ptr
    rows, k = ap.shape[0], ap.shape[1] * 2
    experts, n = wp.shape[0], wp.shape[1]
    work = torch.empty(int(L.frt_nvfp4_grouped_gemm_workspace_bytes(rows, experts)), dtype=torch.uint8, device=DEV)
    capi.check(L.frt_nvfp4_grouped_gemm_bf16(P(ap), P(asw), P(wp), P(wsw), P(alpha), P(offsets), P(tile_expert),
                                             tile_rows, P(out), rows, n, k, experts, n * (k // 2), wsw.shape[1],
                                             P(work), capi.stream_ptr()), "grouped")
    torch.cuda.synchronize()
    return out


def check(got, want, mask=None):
    g, w = got.cpu().float(), want.float()
    if mask is not None:
        g, w = g[mask], w[mask]
    d = (g - w).abs().flatten()
    cos = torch.nn.functional.cosine_similarity(g.flatten(), w.flatten(), dim=0).item()
    rel_l2 = (d.norm() / w.norm().clamp_min(1e-12)).item()
    max_rel = (d.max() / w.abs().max().clamp_min(1e-12)).item()
    assert cos >= 0.999 and rel_l2 <= 0.0025 and max_rel <= 0.01, (cos, rel_l2, max_rel)
    assert device_status() == 0


REFERENCE_CASES = [(16, 8, 64, 3, 4), (16, 72, 128, 3, 4), (16, 1024, 2048, 2, 3), (64, 16, 64, 2, 3),
                   (64, 80, 256, 2, 3), (64, 64, 64, 2, 3), (64, 128, 256, 2, 3), (64, 1024, 2048, 1, 2),
                   (64, 1024, 2048, 2, 4), (64, 2048, 512, 2, 4), (16, 256, 512, 11, 3), (64, 384, 1024, 9, 4)]


@pytest.mark.parametrize("tr,n,k,tiles,experts", REFERENCE_CASES)
def test_tile_expert_signature(tr, n, k, tiles, experts):
    rows = tr * tiles
    ap, wp, al, wl, alpha, asw, wsw = make_inputs(rows, n, k, experts, 19 + n + k)
    te = (torch.arange(tiles, dtype=torch.int32) % experts)
    out = torch.zeros(rows, n, dtype=torch.bfloat16, device=DEV)
    run_capi(ap.to(DEV), wp.to(DEV), asw.to(DEV), wsw.to(DEV), alpha.to(DEV), out, tile_expert=te.to(DEV), tile_rows=tr)
    want = O.grouped_gemm_bf16(ap.numpy(), al.numpy(), wp.numpy(), wl.numpy(), alpha.numpy(),
                               np.repeat(te.numpy(), tr))
    check(out, want)


def test_skipped_tiles_and_runs_leave_output_untouched():
    tr, n, k, experts = 16, 136, 256, 5
    te = torch.tensor([2, 2, -1, 0, 0, 0, -1, -1, 4, 1, 1, 3, 3, 3, 3, 3, 3, 3, 3, 3, 3, 3, 3, 3, 3, 3, 3, 2],
                      dtype=torch.int32)
    rows = tr * te.numel()
    ap, wp, al, wl, alpha, asw, wsw = make_inputs(rows, n, k, experts, 5)
    out = torch.full((rows, n), 7.0, dtype=torch.bfloat16, device=DEV)
    run_capi(ap.to(DEV), wp.to(DEV), asw.to(DEV), wsw.to(DEV), alpha.to(DEV), out, tile_expert=te.to(DEV), tile_rows=tr)
    row_e = np.repeat(te.numpy(), tr)
    want = O.grouped_gemm_bf16(ap.numpy(), al.numpy(), wp.numpy(), wl.numpy(), alpha.numpy(), row_e)
    live = torch.from_numpy(row_e >= 0)
    check(out, want, live)
    assert torch.all(out.cpu()[~live] == 7.0)


@pytest.mark.parametrize("with_skips", [False, True])
def test_many_short_runs_fit_the_work_list(with_skips):
    """16-row tiles of alternating experts make every tile its own window: 64 tiles give 64 work items
    (grouped-moe-gemm/tests/test_grouped_moe_gemm.py:53-66 uses this `arange(tiles) % experts` pattern).
    The documented workspace holds them, nothing is dropped (status word 0), skipped tiles stay untouched."""
    tr, n, k, experts, tiles = 16, 264, 256, 3, 64
    te = torch.arange(tiles, dtype=torch.int32) % experts
    if with_skips:
        te[1::5] = -1
    rows = tr * tiles
    ap, wp, al, wl, alpha, asw, wsw = make_inputs(rows, n, k, experts, 77)
    out = torch.full((rows, n), 7.0, dtype=torch.bfloat16, device=DEV)
    run_capi(ap.to(DEV), wp.to(DEV), asw.to(DEV), wsw.to(DEV), alpha.to(DEV), out, tile_expert=te.to(DEV), tile_rows=tr)
    row_e = np.repeat(te.numpy(), tr)
    want = O.grouped_gemm_bf16(ap.numpy(), al.numpy(), wp.numpy(), wl.numpy(), alpha.numpy(), row_e)
    live = torch.from_numpy(row_e >= 0)
    check(out, want, live)
    assert torch.all(out.cpu()[~live] == 7.0)


def test_overlapping_offsets_are_cut_short_not_overrun():
    """Offsets that go back and forth describe more rows than exist: here 64 of 128 experts each claim all
    4096 rows, 1024 row windows for a work list that holds 4096/16 + 2*128 + 8 = 520.  The windows that do not
    fit are dropped (bit 0x200 of the status word), bytes beyond the workspace stay untouched, and the next,
    well-formed call is clean."""
    n, k, experts, rows = 128, 128, 128, 4096
    ap, wp, al, wl, alpha, asw, wsw = make_inputs(rows, n, k, experts, 9)
    offs = torch.zeros(experts + 1, dtype=torch.int32)
    offs[1::2] = rows
    L, P = capi.lib(), capi.ptr
    need = int(L.frt_nvfp4_grouped_gemm_workspace_bytes(rows, experts))
    assert need == 16 + 32 * 520
    work = torch.full((need + 4096,), 0xAB, dtype=torch.uint8, device=DEV)
    out = torch.zeros(rows, n, dtype=torch.bfloat16, device=DEV)
    dev = [t.to(DEV) for t in (ap, asw, wp, wsw, alpha, offs)]
    capi.check(L.frt_nvfp4_grouped_gemm_bf16(P(dev[0]), P(dev[1]), P(dev[2]), P(dev[3]), P(dev[4]), P(dev[5]), None, 0,
                                             P(out), rows, n, k, experts, n * (k // 2), wsw.shape[1], P(work),
                                             capi.stream_ptr()))
    torch.cuda.synchronize()
    assert device_status() & 0x200
    assert torch.all(work[need:] == 0xAB)
    assert torch.isfinite(out.float()).all()
    # a sorted description on the same buffers afterwards
    good = torch.arange(experts + 1, dtype=torch.int32) * (rows // experts)
    out.zero_()
    run_capi(dev[0], dev[2], dev[1], dev[3], dev[4], out, offsets=good.to(DEV))
    row_e = np.repeat(np.arange(experts), rows // experts)
    check(out, O.grouped_gemm_bf16(ap.numpy(), al.numpy(), wp.numpy(), wl.numpy(), alpha.numpy(), row_e))


def test_golden_fixture_from_reference_helpers(golden_dir):
    g = np.load(golden_dir / "grouped_moe.npz")
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    rows, n = g["a_packed"].shape[0], g["w_packed"].shape[1]
    out = torch.zeros(rows, n, dtype=torch.bfloat16, device=DEV)
    run_capi(t(g["a_packed"]), t(g["w_packed"]), t(g["a_sf_swz"]), t(g["w_sf_swz"]), t(g["alpha"]), out,
             tile_expert=t(g["tile_expert"]), tile_rows=64)
    check(out, O.bits_to_torch_bf16(g["out_bf16"]))


@pytest.mark.parametrize("sizes", [[5, 0, 300, 1, 31, 33, 64, 0, 257, 100], [1000], [0, 0, 17], [32, 32, 32, 32],
                                   [255, 257, 256, 1, 1, 1, 511],
                                   # windows of 257..320 rows (one pass over the weights, two MMAs) at every start
                                   # offset, next to windows just past 320 and short ones
                                   [7, 300, 13, 320, 20, 289, 45, 321, 3, 260, 60, 600, 31, 288, 288, 288]])
def test_offsets_signature_ragged(sizes):
    n, k = 264, 512
    experts = len(sizes)
    offs = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int32)
    rows = int(offs[-1]) + 9                       # trailing rows owned by nobody stay untouched
    ap, wp, al, wl, alpha, asw, wsw = make_inputs(rows, n, k, experts, 77 + len(sizes))
    out = torch.full((rows, n), -3.0, dtype=torch.bfloat16, device=DEV)
    run_capi(ap.to(DEV), wp.to(DEV), asw.to(DEV), wsw.to(DEV), alpha.to(DEV), out,
             offsets=torch.from_numpy(offs).to(DEV))
    row_e = np.full(rows, -1)
    for e in range(experts):
        row_e[offs[e]:offs[e + 1]] = e
    want = O.grouped_gemm_bf16(ap.numpy(), al.numpy(), wp.numpy(), wl.numpy(), alpha.numpy(), row_e)
    live = torch.from_numpy(row_e >= 0)
    check(out, want, live)
    assert torch.all(out.cpu()[~live] == -3.0)


@pytest.mark.parametrize("name,n,k", [("gate_up", 1536, 2048), ("down", 2048, 768)])
def test_qwen3_30b_a3b_shape(name, n, k):
    """128 experts, top-8 of softmax over seeded N(0,1) logits, 4096 tokens ->
    32768 routed rows; whole output against per-expert fp32 GPU matmuls of the
    exactly dequantised bytes."""
    experts, tokens, top_k = 128, 4096, 8
    rng = np.random.default_rng(3)
    _, offs = O.route_topk(rng.standard_normal((tokens, experts)).astype(np.float32), top_k)
    rows = int(offs[-1])
    assert rows == tokens * top_k
    g = torch.Generator(device=DEV).manual_seed(11)
    ap = torch.randint(0, 256, (rows, k // 2), generator=g, dtype=torch.uint8, device=DEV)
    wp = torch.randint(0, 256, (experts, n, k // 2), generator=g, dtype=torch.uint8, device=DEV)
    asw = torch.randint(32, 80, (sf_bytes(rows, k),), generator=g, dtype=torch.uint8, device=DEV)
    wsw = torch.randint(32, 80, (experts, sf_bytes(n, k)), generator=g, dtype=torch.uint8, device=DEV)
    alpha = (torch.rand(experts, generator=g, device=DEV) + 0.5)
    out = torch.zeros(rows, n, dtype=torch.bfloat16, device=DEV)
    run_capi(ap, wp, asw, wsw, alpha, out, offsets=torch.from_numpy(offs).to(DEV))
    L, P = capi.lib(), capi.ptr
    a_deq = torch.empty(rows, k, dtype=torch.float16, device=DEV)
    capi.check(L.frt_nvfp4_dequantize_fp16(P(ap), P(asw), P(a_deq), rows, k, capi.stream_ptr()))
    want = torch.empty(rows, n, dtype=torch.bfloat16, device=DEV)
    w_deq = torch.empty(n, k, dtype=torch.float16, device=DEV)
    for e in range(experts):
        capi.check(L.frt_nvfp4_dequantize_fp16(P(wp[e]), P(wsw[e]), P(w_deq), n, k, capi.stream_ptr()))
        lo, hi = int(offs[e]), int(offs[e + 1])
        want[lo:hi] = ((a_deq[lo:hi].float() @ w_deq.float().T) * alpha[e]).to(torch.bfloat16)
    torch.cuda.synchronize()
    check(out, want.cpu())


def test_torch_ops_both_signatures_compile_and_graph():
    import grouped_moe_gemm as pkg
    tr, n, k, tiles, experts = 64, 128, 256, 6, 3
    rows = tr * tiles
    ap, wp, al, wl, alpha, asw, wsw = [t.to(DEV) if isinstance(t, torch.Tensor) else t
                                       for t in make_inputs(rows, n, k, experts, 19)]
    te = (torch.arange(tiles, dtype=torch.int32) % experts).to(DEV)
    got = pkg.grouped_nvfp4_gemm_bf16(ap, wp, asw, wsw, alpha, te, tile_rows=tr)
    want = O.grouped_gemm_bf16(ap.cpu().numpy(), al.cpu().numpy(), wp.cpu().numpy(), wl.cpu().numpy(),
                               alpha.cpu().numpy(), np.repeat(te.cpu().numpy(), tr))
    check(got, want)
    compiled = torch.compile(lambda aa: pkg.grouped_nvfp4_gemm_bf16(aa, wp, asw, wsw, alpha, te, tile_rows=tr),
                             fullgraph=True)
    assert torch.equal(compiled(ap), got)
    # offsets form: the same rows described as sorted runs
    order = torch.argsort(torch.repeat_interleave(te, tr), stable=True)
    offs = torch.zeros(experts + 1, dtype=torch.int32)
    offs[1:] = torch.cumsum(torch.bincount(te.cpu().long(), minlength=experts) * tr, 0)
    a_sorted = ap[order].contiguous()
    al_sorted = al[order.cpu()] if not al.is_cuda else al[order]
    asw_sorted = torch.from_numpy(O.sf_linear_to_swizzled(al_sorted.cpu().numpy())).to(DEV)
    out2 = pkg.grouped_nvfp4_gemm_bf16_offsets(a_sorted, wp, asw_sorted, wsw, alpha, offs.to(DEV))
    assert torch.equal(out2, got[order])
    gout = torch.empty_like(got)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        work = pkg.grouped_workspace(rows, experts, DEV)
        pkg.grouped_nvfp4_gemm_bf16_offsets(a_sorted, wp, asw_sorted, wsw, alpha, offs.to(DEV), workspace=work, out=gout)
        graph = torch.cuda.CUDAGraph()
        offs_d = offs.to(DEV)
        with torch.cuda.graph(graph, stream=s):
            pkg.grouped_nvfp4_gemm_bf16_offsets(a_sorted, wp, asw_sorted, wsw, alpha, offs_d, workspace=work, out=gout)
    gout.zero_(); graph.replay(); torch.cuda.synchronize()
    assert torch.equal(gout, out2)


def test_grouped_rejections():
    L, P = capi.lib(), capi.ptr
    ap, wp, al, wl, alpha, asw, wsw = [t.to(DEV) for t in make_inputs(64, 64, 64, 2, 1)]
    out = torch.zeros(64, 64, dtype=torch.bfloat16, device=DEV)
    te = torch.zeros(1, dtype=torch.int32, device=DEV)
    work = torch.empty(4096, dtype=torch.uint8, device=DEV)
    args = lambda **kw: (P(ap), P(asw), P(wp), P(wsw), P(alpha), kw.get("off"), kw.get("te", P(te)), kw.get("tr", 64),
                         P(out), 64, 64, kw.get("k", 64), 2, 64 * 32, int(wsw.shape[1]), P(work), capi.stream_ptr())
    assert L.frt_nvfp4_grouped_gemm_bf16(*args(tr=32)) == -2
    assert L.frt_nvfp4_grouped_gemm_bf16(*args(k=96)) == -2
    assert L.frt_nvfp4_grouped_gemm_bf16(*args(off=P(te))) == -1          # both descriptions given
    assert L.frt_nvfp4_grouped_gemm_bf16(*args(te=None)) == -1            # none given
