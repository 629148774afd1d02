from .layers import RMSNorm, FlashRTQuantLinear, FusedNormLinear, FusedSwiGLUFFN

__all__ = ["RMSNorm", "FlashRTQuantLinear", "FusedNormLinear", "FusedSwiGLUFFN"]
