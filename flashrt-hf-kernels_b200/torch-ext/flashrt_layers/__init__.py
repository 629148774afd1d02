from .layers import RMSNorm, FlashRTQuantLinear, FusedNormLinear

__all__ = ["RMSNorm", "FlashRTQuantLinear", "FusedNormLinear"]
