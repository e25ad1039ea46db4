"""The C-ABI library loads here (no GPU) and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "ironmlx_b200.h")
TESTING_HEADER = os.path.join(ROOT, "include", "ironmlx_b200_testing.h")


def declared_symbols():
    """Every entry point of the boundary header, plus the test hooks of the testing header."""
    src = open(HEADER).read()
    names = set(re.findall(r"IMX_API\s+[\w\s\*]+?\b(imx_\w+)\s*\(", src))
    names |= set(re.findall(r"\b(imx_testing_\w+)\s*\(", open(TESTING_HEADER).read()))
    return sorted(names)


def test_header_declares_the_surface():
    names = declared_symbols()
    for must in ["imx_moe_forward", "imx_moe_forward_host", "imx_moe_workspace_bytes", "imx_moe_route",
                 "imx_moe_sort", "imx_moe_experts", "imx_moe_combine", "imx_dequantize",
                 "imx_quantized_matmul", "imx_quantize", "imx_gather_qmm", "imx_last_error"]:
        assert must in names


def test_library_exports_every_declared_symbol():
    from ironmlx_b200 import _lib, build
    build.build()
    handle = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(handle, name), f"{name} declared in the header but not exported"
    assert set(_lib.SIGNATURES) == set(declared_symbols())
    assert _lib.lib().imx_version().startswith(b"ironmlx_b200")


def test_argument_validation_without_gpu():
    """Pure host-side checks: bad arguments come back as error codes with a message."""
    import ctypes as C
    from ironmlx_b200 import _lib
    lib = _lib.lib()
    out = C.c_size_t(0)
    good = _lib.MoEConfig(2048, 256, 8, 512, 512, 1, 0, 4, 64, 0)
    assert lib.imx_moe_workspace_bytes(C.byref(good), 64, C.byref(out)) == 0 and out.value > 0
    small = out.value
    assert lib.imx_moe_workspace_bytes(C.byref(good), 8192, C.byref(out)) == 0 and out.value > small
    for field, value, needle in [("bits", 7, b"bits"), ("group_size", 48, b"group"), ("top_k", 0, b"top_k"),
                                 ("hidden", 100, b"hidden"), ("mode", 9, b"mode"), ("num_experts", 0, b"num_experts")]:
        bad = _lib.MoEConfig(2048, 256, 8, 512, 512, 1, 0, 4, 64, 0)
        setattr(bad, field, value)
        assert lib.imx_moe_workspace_bytes(C.byref(bad), 64, C.byref(out)) == _lib.ERR_INVALID
        assert needle in lib.imx_last_error()
    bad = _lib.MoEConfig(2048, 256, 8, 512, 512, 1, 1, 4, 32, 0)      # mxfp8 needs 8 bits
    assert lib.imx_moe_workspace_bytes(C.byref(bad), 64, C.byref(out)) == _lib.ERR_INVALID
    # forward with a NULL workspace is refused before any CUDA call
    w = _lib.MoEWeights()
    w.router_w = 256
    w.shared_expert_gate_w = 256
    assert lib.imx_moe_forward(C.byref(good), C.byref(w), 256, 4, 256, None, 0, None, None) == _lib.ERR_WORKSPACE
    with pytest.raises(_lib.IronMLXError):
        _lib.check(_lib.ERR_WORKSPACE)
