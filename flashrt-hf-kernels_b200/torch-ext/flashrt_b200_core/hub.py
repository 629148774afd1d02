"""Local stand-ins for the kernels-hub entry points the reference's users call:

    get_kernel("flashrt/fp4-gemm", version=1, trust_remote_code=True) -> module
    kernelize(model)                                                  -> model

With the `kernels` package installed, `kernelize` registers the RMSNorm layer
through its LocalLayerRepository mapping exactly as the reference demo does
(demos/space/transformers-qwen3/flashrt_kernelize.py:19-40); without it the
same layer's forward is bound to every module whose class name ends in
"RMSNorm" and that has `weight` and `variance_epsilon`."""
from __future__ import annotations

import importlib
import sys
import types
from pathlib import Path

_TORCH_EXT = Path(__file__).resolve().parent.parent
if str(_TORCH_EXT) not in sys.path:
    sys.path.insert(0, str(_TORCH_EXT))

_REPOS = {
    "flashrt/fp4-gemm": "fp4_gemm",
    "flashrt/fp4-fused-ops": "fp4_fused_ops",
    "flashrt/flashrt-nvfp4": "flashrt_nvfp4",
    "flashrt/flashrt-residual-norm-quant": "flashrt_residual_norm_quant",
    "flashrt/grouped-moe-gemm": "grouped_moe_gemm",
    "flashrt/transformer-fused-ops": "transformer_fused_ops",
    "flashrt/flashrt-smallm-gemm": "flashrt_smallm_gemm",
}


def get_kernel(repo_id: str, version=None, trust_remote_code: bool = False) -> types.ModuleType:
    key = repo_id.lower()
    if key not in _REPOS:
        raise ValueError(f"unknown kernel repository {repo_id!r}; available: {sorted(_REPOS)}")
    return importlib.import_module(_REPOS[key])


def kernelize(model, *, device: str = "cuda"):
    from flashrt_layers import RMSNorm
    try:
        from kernels import LocalLayerRepository, Mode, kernelize as hub_kernelize, register_kernel_mapping
    except ImportError:
        for module in model.modules():
            if type(module).__name__.endswith("RMSNorm") and hasattr(module, "weight") and hasattr(
                    module, "variance_epsilon"):
                module.forward = types.MethodType(RMSNorm.forward, module)
        return model
    register_kernel_mapping({"RMSNorm": {device: {Mode.INFERENCE: LocalLayerRepository(
        repo_path=_TORCH_EXT, package_name="flashrt_layers", layer_name="RMSNorm")}}})
    return hub_kernelize(model, mode=Mode.INFERENCE, device=device)
