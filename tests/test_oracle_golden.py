"""The CPU oracle against the golden vectors produced by the reference's own
Python helpers (tests/golden/make_golden.py) and its known-answer tests."""
import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O


def load(golden_dir, name):
    return np.load(golden_dir / name)


@pytest.mark.parametrize("rows,dim", [(1, 1024), (33, 4096), (129, 4096), (16, 12288), (130, 80)])
def test_layout_matches_reference_loop(golden_dir, rows, dim):
    g = load(golden_dir, "sf_layout.npz")
    lin, swz = g[f"lin_{rows}_{dim}"], g[f"swz_{rows}_{dim}"]
    assert O.sf_swizzled_bytes(rows, dim) == swz.size
    np.testing.assert_array_equal(O.sf_linear_to_swizzled(lin), swz)
    np.testing.assert_array_equal(O.sf_swizzled_to_linear(swz, rows, dim), lin)


@pytest.mark.parametrize("rows,dim,expect", [(129, 4096, 65536), (1, 1024, 8192), (128, 4096, 32768),
                                             (64, 16384, 131072), (16, 12288, 98304)])
def test_swizzled_size_formula(rows, dim, expect):
    # flashrt-nvfp4/tests/test_nvfp4_sf_reshape.py:30-48, VALIDATION.md:70-84
    assert O.sf_swizzled_bytes(rows, dim) == expect


def test_ue4m3_encode_matches_torch_float8():
    # torch's float8_e4m3fn cast is RNE; it agrees with the CUDA conversion
    # below the saturation point (above 448 CUDA saturates, torch gives NaN).
    rng = np.random.default_rng(0)
    x = np.concatenate([
        np.exp(rng.uniform(np.log(1e-13), np.log(448.0), 200000)).astype(np.float32),
        O.UE4M3_LUT[:0x7F],                                     # exact values
        (O.UE4M3_LUT[:0x7E] + O.UE4M3_LUT[1:0x7F]) / 2,         # exact midpoints (ties)
        np.array([0.0, 1e-12, 2.0 ** -10, 2.0 ** -9, 448.0], dtype=np.float32)])
    x = x.astype(np.float32)
    want = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    np.testing.assert_array_equal(O.ue4m3_encode(x), want)
    assert O.ue4m3_encode(np.array([449.0, 464.0, 1000.0, 2784.0, 1e6], np.float32)).tolist() == [0x7E] * 5
    # decode LUT equals torch's
    lut = torch.arange(0, 0x7F, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    np.testing.assert_array_equal(O.UE4M3_LUT[:0x7F], lut)


@pytest.mark.parametrize("tag", ["unit", "small", "wide"])
def test_quantizer_vs_reference_torch_helper(golden_dir, tag):
    """SF bytes identical; codes identical except where the reference's
    division form and the CUDA kernels' reciprocal-multiply form land on
    opposite sides of a rule-A threshold (adjacent codes, < 0.5 % of elements)."""
    g = load(golden_dir, "quant_torch_reference.npz")
    x = O.bf16_bits_to_f32(g[f"{tag}_x"])
    rows, dim = x.shape
    packed, sf = O.quantize_nvfp4(x)
    np.testing.assert_array_equal(O.sf_linear_to_swizzled(sf), g[f"{tag}_sfa"])
    mine, ref = O.unpack_codes(packed).astype(int), O.unpack_codes(g[f"{tag}_packed"]).astype(int)
    diff = mine != ref
    assert diff.mean() < 0.005
    assert np.all(np.abs(mine[diff] - ref[diff]) == 1)
    # every disagreement is an exact tie of one of the two forms
    s = np.repeat(O.UE4M3_LUT[sf], 16, axis=1)
    q_div = np.abs(x / s)[diff]
    q_mul = np.abs(x * (np.float32(1) / s))[diff]
    at_tie = np.isin(q_div, O.RULE_A_THRESHOLDS) | np.isin(q_mul, O.RULE_A_THRESHOLDS)
    assert at_tie.all()


def test_zero_and_tiny_blocks():
    x = np.zeros((1, 48), dtype=np.float32)
    x[0, 16:32] = 2.0 ** -13      # scale rounds to zero -> inf -> code 7
    x[0, 32] = 3.0                # amax 3 -> scale .5 -> code of 3/.5 = 6 -> 7
    packed, sf = O.quantize_nvfp4(x)
    assert sf.tolist() == [[0, 0, 0x30]]
    assert packed[0, :8].tolist() == [0x77] * 8      # NaN falls through the <= chain
    assert packed[0, 8:16].tolist() == [0x77] * 8    # +inf
    assert packed[0, 16] == 0x07
    deq = O.dequantize_nvfp4(packed, sf)
    assert np.all(deq[0, :32] == 0) and deq[0, 32] == 3.0


def test_sweep_helpers(golden_dir):
    g = load(golden_dir, "sweep_helpers.npz")
    np.testing.assert_array_equal(O.UE4M3_LUT[:0x7F], g["ue4m3_lut"][:0x7F])
    np.testing.assert_array_equal(O.E2M1_CODEBOOK[O.unpack_codes(g["b_packed"])], g["b_unpacked"])
    np.testing.assert_array_equal(O.sf_linear_to_swizzled(g["sfb_lin"]), g["sfb_swz"])
    np.testing.assert_array_equal(O.sf_swizzled_to_linear(g["sfb_swz"], 48, 512), g["sfb_deswz"])
    out = O.gemm_bf16(g["a_packed"][None, :], g["sfa_lin"], g["b_packed"], g["sfb_lin"], float(g["alpha"]))
    want = O.bits_to_torch_bf16(g["out_bf16"])
    rel, cos = O.gemm_error_metrics(out.flatten(), want)
    assert rel <= 1e-2 and cos >= 0.999


def test_grouped_moe_reference(golden_dir):
    g = load(golden_dir, "grouped_moe.npz")
    np.testing.assert_array_equal(O.sf_linear_to_swizzled(g["a_sf_lin"]), g["a_sf_swz"])
    np.testing.assert_array_equal(O.dequantize_nvfp4(g["a_packed"], g["a_sf_lin"]), g["a_deq"])
    row_expert = np.repeat(g["tile_expert"], 64)
    out = O.grouped_gemm_bf16(g["a_packed"], g["a_sf_lin"], g["w_packed"], g["w_sf_lin"], g["alpha"], row_expert)
    rel, cos = O.gemm_error_metrics(out, O.bits_to_torch_bf16(g["out_bf16"]))
    assert rel <= 0.0025 and cos >= 0.999


def test_constant_gemv_known_answer():
    # flashrt-smallm-gemm/tests/test_nvfp4_w4a4_decode_matvec.py:32-52
    for K in (4096, 12288):
        a = np.full((1, K // 2), 0x11, np.uint8)
        b = np.full((16, K // 2), 0x11, np.uint8)
        out = O.gemm_bf16(a, np.full((1, K // 16), 0x38, np.uint8), b, np.full((16, K // 16), 0x38, np.uint8), 0.5)
        assert torch.all(out.float() == K * 0.25 * 0.5)


def test_rms_norm_reference(golden_dir):
    g = load(golden_dir, "rms_norm.npz")
    eps = float(g["eps"])
    y = O.rms_norm_bf16(g["x"], g["w"], eps)
    d = np.abs(O.bf16_bits_to_f32(y) - O.bf16_bits_to_f32(g["y"]))
    assert d.max() <= 2.0 ** -6 and (y != g["y"]).mean() < 0.01
    res_out, y_res = O.residual_add_rms_norm_bf16(g["res"], g["x"], g["w"], eps)
    np.testing.assert_array_equal(res_out, g["res_out"])          # exact in-place residual
    d = np.abs(O.bf16_bits_to_f32(y_res) - O.bf16_bits_to_f32(g["y_res"]))
    assert d.max() <= 2.0 ** -6 and (y_res != g["y_res"]).mean() < 0.01


def test_bf16_roundtrip_matches_torch():
    x = torch.randn(4096) * 3
    np.testing.assert_array_equal(O.f32_to_bf16_bits(x.numpy()), O.torch_bf16_to_bits(x.bfloat16()))


def test_rne_rule_against_table():
    q = np.array([0.0, 0.25, 0.26, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 5.01, 7.0, -0.75, -2.5], np.float32)
    # ties to even mantissa: .25->0, .75->1.0(code2), 1.25->1.0(2), 1.75->2.0(4), 2.5->2(4), 3.5->4(6), 5->4(6)
    assert O.e2m1_rne_codes(q).tolist() == [0, 0, 1, 2, 2, 4, 4, 6, 6, 7, 7, 8 | 2, 8 | 4]


def test_fused_default_is_quantizer_of_its_own_norm():
    rng = np.random.default_rng(5)
    rows, dim = 9, 1024
    x = O.f32_to_bf16_bits(rng.standard_normal((rows, dim)).astype(np.float32))
    r = O.f32_to_bf16_bits(rng.standard_normal((rows, dim)).astype(np.float32))
    w = O.f32_to_bf16_bits((1 + 0.1 * rng.standard_normal(dim)).astype(np.float32))
    out = O.fused_norm_quant(x, w, 1e-6, res_bits=r)
    a = O.bf16_bits_to_f32(r) + O.bf16_bits_to_f32(x)
    np.testing.assert_array_equal(out["residual"], O.f32_to_bf16_bits(a))
    v = (a * out["rstd"][:, None]).astype(np.float32) * O.bf16_bits_to_f32(w)[None, :]
    p, s = O.quantize_nvfp4(v.astype(np.float32))
    np.testing.assert_array_equal(out["packed"], p)
    np.testing.assert_array_equal(out["sf_linear"], s)
    # rstd agrees with a float64 evaluation to fp32 rounding noise
    want = 1 / np.sqrt((a.astype(np.float64) ** 2).mean(axis=1) + 1e-6)
    assert np.max(np.abs(out["rstd"] / want - 1)) < 1e-6


@pytest.mark.parametrize("rows", [1, 7, 257])
def test_swiglu_stage_matches_reference_chain(golden_dir, rows):
    # the staged value of the reference's production-chain check
    # (fp4-fused-ops/tests/test_fp4_fused_ops.py:483-495)
    g = load(golden_dir, "swiglu.npz")
    merged, staged = g[f"merged_{rows}"], g[f"staged_{rows}"]
    out = O.silu_mul_quantize(merged)
    np.testing.assert_array_equal(out["staged"], staged)
    # and the quantiser stage is the rule-A quantiser of those values
    packed, sf = O.quantize_nvfp4(O.bf16_bits_to_f32(staged))
    np.testing.assert_array_equal(out["packed"], packed)
    np.testing.assert_array_equal(out["sf_linear"], sf)
    # an explicit fp32 evaluation of g / (1 + exp(-g)) * u agrees up to the exponential's last place
    gate = O.bf16_bits_to_f32(merged[:, : merged.shape[1] // 2])
    up = O.bf16_bits_to_f32(merged[:, merged.shape[1] // 2:])
    direct = O.f32_to_bf16_bits((gate / (np.float32(1) + np.exp(-gate, dtype=np.float32))) * up)
    assert (direct != staged).mean() < 2e-3


def test_router_topk_and_plan_oracle():
    # the reference's own check of its router: linspace logits against torch.topk
    # (transformer-fused-ops/tests/test_transformer_fused_ops.py:736-740)
    router = torch.linspace(-1.0, 1.0, 256).to(torch.bfloat16)
    idx, val = O.router_topk(O.torch_bf16_to_bits(router)[None, :], 8)
    ref_val, ref_idx = torch.topk(router.float(), 8)
    # bf16 linspace holds ties; both orders must agree on the values, and on indices where unique
    np.testing.assert_array_equal(val[0], ref_val.numpy())
    assert set(idx[0].tolist()) <= set(range(256)) and (np.diff(val[0]) <= 0).all()
    # ties: bit-reversed index order (2 = 0b10 reverses below 1 = 0b01), as the reference's fold gives
    idx2, val2 = O.router_topk(O.torch_bf16_to_bits(torch.tensor([[1.0, 3.0, 3.0, 2.0]]).bfloat16()), 3)
    assert idx2.tolist() == [[2, 1, 3]] and val2.tolist() == [[3.0, 3.0, 2.0]]
    # the plan is the stable sort by expert, consistent with the sort the grouped tests use
    rng = np.random.default_rng(5)
    logits = rng.standard_normal((64, 16)).astype(np.float32)
    top = np.argsort(-logits, axis=1, kind="stable")[:, :4].astype(np.int32)
    offsets, row_of_pair, token_of_row = O.route_plan(top, 16)
    sorted_token, offsets2 = O.route_topk(logits, 4)
    np.testing.assert_array_equal(offsets, offsets2)
    np.testing.assert_array_equal(token_of_row, sorted_token)
    for t in range(64):
        for j in range(4):
            r = row_of_pair[t, j]
            assert token_of_row[r] == t and offsets[top[t, j]] <= r < offsets[top[t, j] + 1]


def test_weighted_sum_oracle_matches_reference_definition():
    # transformer-fused-ops/tests/test_transformer_fused_ops.py:748-760 (tolerance 1e-5 there)
    g = torch.Generator().manual_seed(3)
    y = torch.randn(37, 384, generator=g).bfloat16()
    rows = torch.randint(0, 37, (3, 4), generator=g, dtype=torch.int32)
    w = torch.softmax(torch.randn(3, 4, generator=g), dim=-1)
    got = O.weighted_sum(O.torch_bf16_to_bits(y), rows.numpy(), w.numpy(), 320)
    ref = (y[rows.long(), :320].float() * w[..., None]).sum(dim=1)
    np.testing.assert_allclose(got, ref.numpy(), rtol=1e-5, atol=1e-5)
