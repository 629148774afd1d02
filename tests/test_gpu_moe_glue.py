"""GPU parity of the MoE routing glue (router top-k, routing plan, NVFP4 gather, weighted
un-permute) through the C ABI, against the CPU oracle and the reference's own kernels, and the
whole routed expert layer end to end."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from tests.gpu_common import (DEV, O, alloc_fp4, bits, capi, quantize, randn_bf16, ref_lib, sf_linear)  # noqa: E402

P = capi.ptr


def st():
    return capi.stream_ptr()


def topk(logits, k):
    tokens, n = logits.shape
    idx = torch.empty(tokens, k, dtype=torch.int32, device=DEV)
    val = torch.empty(tokens, k, dtype=torch.float32, device=DEV)
    capi.check(capi.lib().frt_router_topk_bf16(P(logits), P(idx), P(val), tokens, n, k, st()))
    return idx, val


@pytest.mark.parametrize("tokens,n,k", [(1, 256, 8), (5, 128, 8), (4096, 128, 8), (33, 60, 4), (7, 1000, 32),
                                        (3, 4, 8)])
def test_router_topk(tokens, n, k):
    logits = randn_bf16((tokens, n), 70 + tokens + n).to(DEV)          # bf16: plenty of exact ties
    idx, val = topk(logits, k)
    want_idx, want_val = O.router_topk(bits(logits), k)
    np.testing.assert_array_equal(idx.cpu().numpy(), want_idx)
    np.testing.assert_array_equal(val.cpu().numpy(), want_val)
    ref = ref_lib()
    if ref is not None and k <= n and n <= 256:
        for t in range(min(tokens, 4)):
            ri = torch.empty(k, dtype=torch.int32, device=DEV)
            rv = torch.empty(k, dtype=torch.float32, device=DEV)
            assert ref.ref_router_topk_bf16(P(logits[t]), P(ri), P(rv), n, k, st()) == 0
            torch.cuda.synchronize()
            assert torch.equal(ri, idx[t]) and torch.equal(rv, val[t])


def test_router_topk_reference_known_answer():
    # transformer-fused-ops/tests/test_transformer_fused_ops.py:736-740
    router = torch.linspace(-1.0, 1.0, 256, device=DEV).to(torch.bfloat16)
    idx, val = topk(router[None, :], 8)
    ref_val, _ = torch.topk(router.float(), 8)
    assert torch.equal(val[0], ref_val)


@pytest.mark.parametrize("tokens,k,n_experts", [(1, 8, 128), (64, 4, 16), (4096, 8, 128), (777, 8, 256), (300, 2, 2048)])
def test_route_plan(tokens, k, n_experts):
    g = torch.Generator().manual_seed(tokens + k)
    scores = torch.rand(tokens, n_experts, generator=g)
    top = torch.topk(scores, k, dim=1).indices.to(torch.int32)
    if tokens > 2:
        top[1, 0] = -1                   # pairs with an index outside the expert range are dropped
        top[2, k - 1] = n_experts
    d_top = top.to(DEV)
    off = torch.empty(n_experts + 1, dtype=torch.int32, device=DEV)
    rop = torch.full((tokens, k), -7, dtype=torch.int32, device=DEV)
    tor = torch.full((tokens * k,), -7, dtype=torch.int32, device=DEV)
    capi.check(capi.lib().frt_moe_route_plan(P(d_top), tokens, k, n_experts, P(off), P(rop), P(tor), st()))
    w_off, w_rop, w_tor = O.route_plan(top.numpy(), n_experts)
    np.testing.assert_array_equal(off.cpu().numpy(), w_off)
    np.testing.assert_array_equal(rop.cpu().numpy(), w_rop)
    np.testing.assert_array_equal(tor.cpu().numpy()[: w_tor.size], w_tor)


@pytest.mark.parametrize("tokens,K,k", [(5, 64, 2), (130, 2048, 8), (257, 768, 4)])
def test_gather_nvfp4(tokens, K, k):
    x = randn_bf16((tokens, K), 90 + tokens).to(DEV)
    packed, sf = quantize(x)
    g = torch.Generator().manual_seed(1)
    tor = torch.randint(0, tokens, (tokens * k,), generator=g, dtype=torch.int32)
    rows = tokens * k
    op, osf = alloc_fp4(rows, K)
    capi.check(capi.lib().frt_moe_gather_nvfp4(P(packed), P(sf), P(tor.to(DEV)), P(op), P(osf), rows, tokens, K, st()))
    torch.cuda.synchronize()
    assert torch.equal(op.cpu(), packed.cpu()[tor.long()])
    np.testing.assert_array_equal(sf_linear(osf, rows, K), sf_linear(sf, tokens, K)[tor.numpy()])


@pytest.mark.parametrize("tokens,k,hidden,stride", [(1, 1, 128, 128), (3, 4, 320, 384), (17, 8, 2048, 2112),
                                                    (9, 8, 100, 101), (4096, 8, 2048, 2048)])
def test_weighted_sum(tokens, k, hidden, stride):
    g = torch.Generator().manual_seed(tokens * 31 + k)
    n_rows = tokens * k + 5
    y = torch.randn(n_rows, stride, generator=g).bfloat16()
    rows = torch.randint(0, n_rows, (tokens, k), generator=g, dtype=torch.int32)
    w = torch.softmax(torch.randn(tokens, k, generator=g), dim=-1)
    dy, dr, dw = y.to(DEV), rows.to(DEV), w.to(DEV)
    out = torch.empty(tokens, hidden, dtype=torch.float32, device=DEV)
    capi.check(capi.lib().frt_moe_weighted_sum_bf16(P(dy), P(dr), P(dw), P(out), tokens, k, hidden, stride, st()))
    want = O.weighted_sum(bits(y), rows.numpy(), w.numpy(), hidden)
    np.testing.assert_array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))
    ref = ref_lib()
    if ref is not None:
        ro = torch.empty_like(out)
        assert ref.ref_moe_weighted_sum_bf16(P(dy), P(dr), P(dw), P(ro), tokens, k, hidden, stride, st()) == 0
        torch.cuda.synchronize()
        assert torch.equal(ro, out)
    if tokens > 1:                       # negative rows are skipped
        rows[0, 0] = -1
        capi.check(capi.lib().frt_moe_weighted_sum_bf16(P(dy), P(rows.to(DEV)), P(dw), P(out), tokens, k, hidden,
                                                        stride, st()))
        want = O.weighted_sum(bits(y), rows.numpy(), w.numpy(), hidden)
        np.testing.assert_array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))


def test_routed_expert_layer_end_to_end():
    """router -> plan -> gather -> grouped gate/up -> SwiGLU -> NVFP4 -> grouped down -> weighted sum,
    every stage a kernel of this library (torch operator API), against the same chain in the oracle."""
    import fp4_fused_ops
    import fp4_gemm
    import grouped_moe_gemm
    import transformer_fused_ops
    tokens, hid, inter, E, k = 96, 256, 128, 8, 2
    x = randn_bf16((tokens, hid), 500).to(DEV)
    logits = randn_bf16((tokens, E), 501).to(DEV)
    w1 = randn_bf16((E, 2 * inter, hid), 502, 0.05).to(DEV)
    w2 = randn_bf16((E, hid, inter), 503, 0.05).to(DEV)
    w1p, w1s = zip(*[fp4_gemm.quantize_fp4_sfa_bf16(w1[e]) for e in range(E)])
    w2p, w2s = zip(*[fp4_gemm.quantize_fp4_sfa_bf16(w2[e]) for e in range(E)])
    w1p, w1s, w2p, w2s = (torch.stack(t).contiguous() for t in (w1p, w1s, w2p, w2s))
    alpha = torch.ones(E, dtype=torch.float32, device=DEV)

    idx, val = transformer_fused_ops.router_topk_bf16(logits, k)
    weights = torch.softmax(val, dim=-1)
    offsets, row_of_pair, token_of_row = grouped_moe_gemm.moe_route_plan(idx, E)
    xp, xs = fp4_gemm.quantize_fp4_sfa_bf16(x)
    gp, gs = grouped_moe_gemm.moe_gather_nvfp4(xp, xs, token_of_row)
    h = grouped_moe_gemm.grouped_nvfp4_gemm_bf16_offsets(gp, w1p, gs, w1s, alpha, offsets)
    hp, hs = fp4_fused_ops.silu_mul_quantize_fp4_sfa_bf16(h)
    y = grouped_moe_gemm.grouped_nvfp4_gemm_bf16_offsets(hp, w2p, hs, w2s, alpha, offsets)
    out = transformer_fused_ops.moe_weighted_sum_bf16_to_fp32(y, row_of_pair, weights)
    torch.cuda.synchronize()

    # oracle chain on the CPU
    o_idx, o_val = O.router_topk(bits(logits), k)
    np.testing.assert_array_equal(idx.cpu().numpy(), o_idx)
    o_off, o_rop, o_tor = O.route_plan(o_idx, E)
    rows = tokens * k
    xq, xsl = O.quantize_nvfp4(x.float().cpu().numpy())
    a_p, a_s = xq[o_tor], xsl[o_tor]
    w1q = [O.quantize_nvfp4(w1[e].float().cpu().numpy()) for e in range(E)]
    w2q = [O.quantize_nvfp4(w2[e].float().cpu().numpy()) for e in range(E)]
    hh = np.zeros((rows, 2 * inter), dtype=np.uint16)
    for e in range(E):
        lo, hi = o_off[e], o_off[e + 1]
        if hi > lo:
            hh[lo:hi] = bits(O.gemm_bf16(a_p[lo:hi], a_s[lo:hi], w1q[e][0], w1q[e][1]))
    sq = O.silu_mul_quantize(hh)
    yy = np.zeros((rows, hid), dtype=np.uint16)
    for e in range(E):
        lo, hi = o_off[e], o_off[e + 1]
        if hi > lo:
            yy[lo:hi] = bits(O.gemm_bf16(sq["packed"][lo:hi], sq["sf_linear"][lo:hi], w2q[e][0], w2q[e][1]))
    o_w = torch.softmax(torch.from_numpy(o_val), dim=-1).numpy()
    want = O.weighted_sum(yy, o_rop, o_w, hid)
    rel, cos = O.gemm_error_metrics(out.cpu(), torch.from_numpy(want))
    assert rel <= 2e-2 and cos >= 0.999, (rel, cos)      # two chained NVFP4 GEMMs: twice the GEMM tolerance


def test_glue_argument_errors():
    L = capi.lib()
    t = torch.zeros(8, dtype=torch.int32, device=DEV)
    lg = randn_bf16((2, 2048), 1).to(DEV)
    f = torch.zeros(8, dtype=torch.float32, device=DEV)
    assert L.frt_router_topk_bf16(P(lg), P(t), P(f), 2, 2048, 4, st()) < 0        # more than 1024 experts
    assert L.frt_router_topk_bf16(None, P(t), P(f), 2, 16, 4, st()) == -1
    assert L.frt_moe_route_plan(P(t), 0, 4, 8, P(t), P(t), P(t), st()) < 0
    assert L.frt_moe_gather_nvfp4(P(t), P(t), P(t), P(t), P(t), 4, 4, 48, st()) < 0
    assert L.frt_moe_weighted_sum_bf16(P(lg), P(t), P(f), P(f), 1, 2, 64, 32, st()) < 0  # stride < hidden


def test_router_softmax_and_quantize_scatter():
    """the fused forms equal the separate stages: softmax of the selected logits; quantise + gather"""
    import grouped_moe_gemm
    import fp4_gemm
    import transformer_fused_ops
    tokens, E, k, K = 300, 64, 4, 320
    logits = randn_bf16((tokens, E), 801).to(DEV)
    idx, val, weight = transformer_fused_ops.router_topk_softmax_bf16(logits, k)
    idx2, val2 = transformer_fused_ops.router_topk_bf16(logits, k)
    assert torch.equal(idx, idx2) and torch.equal(val, val2)
    torch.testing.assert_close(weight, torch.softmax(val, dim=-1), rtol=1e-6, atol=1e-7)
    idx[3, 1] = -1                                       # an unrouted pair is skipped
    offsets, row_of_pair, token_of_row = grouped_moe_gemm.moe_route_plan(idx, E)
    rows = int(offsets[-1].item())
    x = randn_bf16((tokens, K), 802).to(DEV)
    xp, xs = fp4_gemm.quantize_fp4_sfa_bf16(x)
    gp, gs = grouped_moe_gemm.moe_gather_nvfp4(xp, xs, token_of_row[:rows].contiguous())
    sp, ss = alloc_fp4(tokens * k, K, fill=0x7F)
    grouped_moe_gemm.moe_quantize_scatter_nvfp4(x, row_of_pair, out_packed=sp, out_sfa=ss)
    torch.cuda.synchronize()
    assert torch.equal(sp[:rows], gp)
    np.testing.assert_array_equal(sf_linear(ss, tokens * k, K)[:rows], sf_linear(gs, rows, K))
