"""ironmlx_b200: a B200-native (sm_100a) implementation of the mixture-of-experts
block of ironmlx's Qwen3.5-MoE path behind the reference's own layer and op
names.  The product is libironmlx_b200.so (C ABI, include/ironmlx_b200.h);
this package is the thin host layer above it.  Nothing here falls back to
PyTorch or the CPU: a missing library raises.
"""
from ._lib import IronMLXError, LIB_PATH, lib  # noqa: F401

__all__ = ["IronMLXError", "LIB_PATH", "lib"]
