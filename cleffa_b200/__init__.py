"""B200-native Clef-Omni mixture-of-experts block (router, permutation, grouped expert
products, combine) behind the C-ABI of include/clef_cuda_omni.h."""
from .omni import DEVICE, HOST, OmniBackend, OmniError, load_library  # noqa: F401

__all__ = ["OmniBackend", "OmniError", "load_library", "HOST", "DEVICE"]
