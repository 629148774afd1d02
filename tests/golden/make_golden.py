#!/usr/bin/env python3
"""Generate tests/golden/*.npz by RUNNING the reference's own Python helpers.

Run once in a container that has the reference checkout (it is not present on
the GPU box, so the outputs are committed):

    python tests/golden/make_golden.py --reference /path/to/FlashRT-HF-kernels

The reference's test modules import CUDA-only packages at module scope, so the
helper functions are lifted out of the files by name with `ast` and executed
unmodified on CPU tensors.  Nothing from the reference is copied into this
repository: only seeded inputs and the outputs its functions produced.
"""
from __future__ import annotations

import argparse
import ast
import math
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def lift(path: Path, names, extra_globals=None):
    """exec the named top-level functions / assignments of `path`."""
    tree = ast.parse(path.read_text())
    keep = []
    for node in tree.body:
        if isinstance(node, (ast.FunctionDef,)) and node.name in names:
            node.decorator_list = []
            keep.append(node)
        elif isinstance(node, ast.Assign) and any(
                isinstance(t, ast.Name) and t.id in names for t in node.targets):
            keep.append(node)
    mod = ast.Module(body=keep, type_ignores=[])
    ns = {"torch": torch, "math": math, "__builtins__": __builtins__}
    ns.update(extra_globals or {})
    exec(compile(mod, str(path), "exec"), ns)
    missing = [n for n in names if n not in ns]
    if missing:
        raise RuntimeError(f"{path}: could not lift {missing}")
    return ns


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    args = ap.parse_args()
    ref = Path(args.reference)

    # ---- 1. scale-factor layout: the python double loop of the reference test
    ns = lift(ref / "flashrt-nvfp4/tests/test_nvfp4_sf_reshape.py", ["_reference_swizzle"])
    swz = ns["_reference_swizzle"]
    g = torch.Generator().manual_seed(0)
    layout = {}
    for rows, dim in [(1, 1024), (33, 4096), (129, 4096), (16, 12288), (130, 80)]:
        lin = torch.randint(0, 256, (rows, dim // 16), generator=g, dtype=torch.uint8)
        layout[f"lin_{rows}_{dim}"] = lin.numpy()
        layout[f"swz_{rows}_{dim}"] = swz(lin).numpy()
    np.savez_compressed(HERE / "sf_layout.npz", **layout)

    # ---- 2. the reference's pure-torch rule-A quantiser (division form)
    ns = lift(ref / "fp4-fused-ops/tests/test_fp4_fused_ops.py", ["_reference_nvfp4_sfa"])
    refq = ns["_reference_nvfp4_sfa"]
    quant = {}
    for tag, rows, dim, scale, seed in [("unit", 37, 512, 1.0, 23), ("small", 130, 256, 0.02, 24),
                                        ("wide", 5, 4096, 1.5, 25)]:
        g = torch.Generator().manual_seed(seed)
        x = (torch.randn(rows, dim, generator=g) * scale).to(torch.bfloat16)
        nbytes = ((rows + 127) // 128) * ((dim // 16 + 3) // 4) * 512
        packed, sfa = refq(x, nbytes)
        quant[f"{tag}_x"] = bf16_bits(x)
        quant[f"{tag}_packed"] = packed.numpy()
        quant[f"{tag}_sfa"] = sfa.numpy()
    np.savez_compressed(HERE / "quant_torch_reference.npz", **quant)

    # ---- 3. dequant helpers + small-M reference of the repo-wide sweep
    ns = lift(ref / "scripts/accuracy_sweep.py",
              ["_torch", "_ue4m3_to_float", "_fp4_codebook_tensor", "_ue4m3_lut_tensor", "_unpack_fp4",
               "_deswizzle_scales", "_reference_smallm", "_reference_swizzle", "_swizzled_bytes"])
    ns["_torch"] = lambda: torch
    g = torch.Generator().manual_seed(7)
    K, N = 512, 48
    a_packed = torch.randint(0, 256, (K // 2,), generator=g, dtype=torch.uint8)
    b_packed = torch.randint(0, 256, (N, K // 2), generator=g, dtype=torch.uint8)
    sfa_lin = torch.randint(24, 72, (1, K // 16), generator=g, dtype=torch.uint8)
    sfb_lin = torch.randint(24, 72, (N, K // 16), generator=g, dtype=torch.uint8)
    out = ns["_reference_smallm"](a_packed, b_packed, sfa_lin, sfb_lin, K, 0.75, 16)
    sweep = dict(
        a_packed=a_packed.numpy(), b_packed=b_packed.numpy(), sfa_lin=sfa_lin.numpy(),
        sfb_lin=sfb_lin.numpy(), alpha=np.float32(0.75), out_bf16=bf16_bits(out),
        ue4m3_lut=ns["_ue4m3_lut_tensor"]().numpy(),
        b_unpacked=ns["_unpack_fp4"](b_packed).numpy(),
        sfb_swz=ns["_reference_swizzle"](sfb_lin).numpy(),
        sfb_deswz=ns["_deswizzle_scales"](ns["_reference_swizzle"](sfb_lin), N, K).numpy(),
    )
    np.savez_compressed(HERE / "sweep_helpers.npz", **sweep)

    # ---- 4. grouped-MoE test's dequantiser (codebook with -0.0) and SF maker
    ns = lift(ref / "grouped-moe-gemm/tests/test_grouped_moe_gemm.py",
              ["CODEBOOK", "ue", "sf_bytes", "make_sf", "deq"])
    torch.manual_seed(19)
    rows, n, k, experts = 128, 32, 128, 3
    ap_ = torch.randint(0, 256, (rows, k // 2), dtype=torch.uint8)
    wp = torch.randint(0, 256, (experts, n, k // 2), dtype=torch.uint8)
    asw, al = ns["make_sf"](rows, k, "cpu")
    wsw, wl = zip(*[ns["make_sf"](n, k, "cpu") for _ in range(experts)])
    alpha = torch.rand(experts) + 0.5
    te = torch.arange(rows // 64, dtype=torch.int32) % experts
    adeq = ns["deq"](ap_, al)
    refout = torch.empty(rows, n)
    for t in range(rows // 64):
        e = int(te[t])
        refout[t * 64:(t + 1) * 64] = adeq[t * 64:(t + 1) * 64] @ ns["deq"](wp[e], wl[e], alpha[e]).T
    moe = dict(a_packed=ap_.numpy(), w_packed=wp.numpy(), a_sf_swz=asw.numpy(), a_sf_lin=al.numpy(),
               w_sf_swz=torch.stack(wsw).numpy(), w_sf_lin=torch.stack(wl).numpy(),
               alpha=alpha.numpy(), tile_expert=te.numpy(), a_deq=adeq.numpy(),
               out_bf16=bf16_bits(refout.bfloat16()))
    np.savez_compressed(HERE / "grouped_moe.npz", **moe)

    # ---- 5. RMSNorm references of the norm package's test
    ns = lift(ref / "flashrt-residual-norm-quant/tests/test_residual_norm_quant.py",
              ["ref_rms_norm", "ref_rms_norm_bf16"])
    torch.manual_seed(23)
    rows, dim, eps = 16, 512, 1e-6
    x = torch.randn(rows, dim).to(torch.bfloat16)
    res = torch.randn(rows, dim).to(torch.bfloat16)
    w = (1.0 + 0.1 * torch.randn(dim)).to(torch.bfloat16)
    y = ns["ref_rms_norm_bf16"](x, w, eps)
    # residual form, following ref_residual_add_rms_norm_quant of the same file
    # (test_residual_norm_quant.py:145-151) without the fp8 cast
    added = res.float() + x.float()
    res_out = added.to(torch.bfloat16)
    rms = torch.rsqrt(torch.mean(added * added, dim=1, keepdim=True) + eps)
    y_res = (res_out.float() * rms * w.float()).to(torch.bfloat16)
    norm = dict(x=bf16_bits(x), res=bf16_bits(res), w=bf16_bits(w), eps=np.float32(eps),
                y=bf16_bits(y), res_out=bf16_bits(res_out), y_res=bf16_bits(y_res))
    np.savez_compressed(HERE / "rms_norm.npz", **norm)
    # ---- 6. SwiGLU -> NVFP4 producer: the staged value of the reference's production-chain
    # check (test_fp4_fused_ops.py:483-495: silu(gate.float()) * up.float() -> bf16), on CPU
    # tensors drawn as the test draws them (randn * 0.2 -> bf16); the quantiser that follows
    # it in that check is pinned by section 2.
    swiglu = {}
    for rows, hidden, seed in [(1, 1024, 2026081701), (7, 1024, 2026081707), (257, 1024, 2026081957)]:
        g = torch.Generator().manual_seed(seed)
        merged = (torch.randn(rows, 2 * hidden, generator=g) * 0.2).to(torch.bfloat16)
        staged = (torch.nn.functional.silu(merged[:, :hidden].float()) * merged[:, hidden:].float()).bfloat16()
        swiglu[f"merged_{rows}"] = bf16_bits(merged)
        swiglu[f"staged_{rows}"] = bf16_bits(staged)
    np.savez_compressed(HERE / "swiglu.npz", **swiglu)
    print("wrote", sorted(p.name for p in HERE.glob("*.npz")))


if __name__ == "__main__":
    main()
