"""ctypes binding of libironmlx_b200.so (the C ABI of include/ironmlx_b200.h).

Loading fails loudly: there is no CPU or PyTorch fallback for any op of this
package, so a missing library is an error, not a degraded mode.
"""
from __future__ import annotations

import ctypes as C
import os

# IRONMLX_B200_LIB selects another build of the same library (e.g. one with different compile-time options)
LIB_PATH = os.environ.get("IRONMLX_B200_LIB") or os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                                             "libironmlx_b200.so")

OK, ERR_INVALID, ERR_CUDA, ERR_WORKSPACE, ERR_DEVICE = 0, 1, 2, 3, 4
MODE = {"affine": 0, "mxfp8": 1, "nvfp4": 2}
PATH = {"auto": 0, "decode": 1, "prefill": 2, "generic": 3,
        # cross-check kernels (include/ironmlx_b200_testing.h)
        "decode_regs": 4, "prefill_plain": 5, "prefill_smem": 6}
MODE_DEFAULTS = {"affine": (64, 4), "mxfp8": (32, 8), "nvfp4": (16, 4)}


class QTensor(C.Structure):
    _fields_ = [("w", C.c_void_p), ("scales", C.c_void_p), ("biases", C.c_void_p),
                ("global_scale", C.c_float)]


class MoEConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in (
        "hidden", "num_experts", "top_k", "intermediate", "shared_intermediate", "norm_topk_prob",
        "mode", "bits", "group_size", "path")]


class MoEWeights(C.Structure):
    _fields_ = [("router_w", C.c_void_p), ("router_logit_bias", C.c_void_p),
                ("gate_up", QTensor), ("down", QTensor),
                ("shared_gate_proj", QTensor), ("shared_up_proj", QTensor), ("shared_down_proj", QTensor),
                ("shared_expert_gate_w", C.c_void_p)]


class EpInfo(C.Structure):
    _fields_ = [("want_timing", C.c_int), ("schedule", C.c_int), ("rows_received", C.c_longlong),
                ("bytes_sent", C.c_ulonglong), ("bytes_received", C.c_ulonglong), ("phase_ms", C.c_float * 5)]


EP_SCHEDULE = {"auto": 0, "gathered": 1, "a2a": 2}


class MoETrace(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "topk_idx", "topk_w", "counts", "offsets", "perm", "inv_perm", "shared_gate")]


# name -> (restype, argtypes); every symbol include/ironmlx_b200.h declares
_vp, _i, _f, _sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t
SIGNATURES = {
    "imx_last_error": (C.c_char_p, []),
    "imx_version": (C.c_char_p, []),
    "imx_launch_count": (C.c_ulonglong, []),
    "imx_moe_workspace_bytes": (_i, [C.POINTER(MoEConfig), _i, C.POINTER(_sz)]),
    "imx_moe_forward": (_i, [C.POINTER(MoEConfig), C.POINTER(MoEWeights), _vp, _i, _vp, _vp, _sz, _vp,
                             C.POINTER(MoETrace)]),
    "imx_moe_forward_residual": (_i, [C.POINTER(MoEConfig), C.POINTER(MoEWeights), _vp, _vp, _f, _i, _vp, _vp, _sz, _vp,
                                      C.POINTER(MoETrace)]),
    "imx_rms_norm": (_i, [_vp, _i, _i, _vp, _f, _vp, _vp]),
    "imx_moe_forward_timed": (_i, [C.POINTER(MoEConfig), C.POINTER(MoEWeights), _vp, _i, _vp, _vp, _sz, _vp,
                                   C.POINTER(C.c_float)]),
    "imx_moe_forward_host": (_i, [C.POINTER(MoEConfig), C.POINTER(MoEWeights), _vp, _i, _vp, _vp, _sz, _vp]),
    "imx_moe_status": (_i, [_vp, _vp]),
    "imx_testing_decode_handoff": (None, [_i, _i]),
    "imx_moe_saturations": (_i, [_vp, _vp, C.POINTER(C.c_longlong)]),
    "imx_moe_route": (_i, [_vp, _i, _i, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "imx_moe_route_scratch_bytes": (_i, [_i, _i, _i, C.POINTER(_sz)]),
    "imx_moe_route_ws": (_i, [_vp, _i, _i, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "imx_moe_sort_scratch_bytes": (_i, [_i, _i, C.POINTER(_sz)]),
    "imx_moe_sort": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "imx_moe_sort_static": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "imx_moe_experts_scratch_bytes": (_i, [C.POINTER(MoEConfig), _i, C.POINTER(_sz)]),
    "imx_moe_experts": (_i, [C.POINTER(MoEConfig), C.POINTER(QTensor), C.POINTER(QTensor), _i, _vp, _vp, _vp,
                             _i, _i, _vp, _vp, _vp, _sz, _vp]),
    "imx_moe_combine": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp]),
    "imx_moe_combine_scaled": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp]),
    "imx_moe_combine_partial": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _vp]),
    "imx_gather_rows": (_i, [_vp, _vp, _i, _sz, _vp, _vp]),
    "imx_ep_unique_id": (_i, [_vp]),
    "imx_ep_create": (_i, [C.POINTER(MoEConfig), _vp, _i, _i, C.POINTER(_vp)]),
    "imx_ep_create_from_comm": (_i, [C.POINTER(MoEConfig), _vp, _i, _i, C.POINTER(_vp)]),
    "imx_ep_destroy": (_i, [_vp]),
    "imx_ep_comm": (_vp, [_vp]),
    "imx_ep_workspace_bytes": (_i, [_vp, _i, _i, C.POINTER(_sz)]),
    "imx_ep_forward": (_i, [_vp, C.POINTER(MoEWeights), _vp, _i, _vp, _vp, _sz, _vp, _i, C.POINTER(EpInfo),
                            C.POINTER(MoETrace)]),
    "imx_dequantize": (_i, [C.POINTER(QTensor), _i, _i, _i, _i, _i, _i, _vp, _vp]),
    "imx_quantized_matmul": (_i, [_vp, _i, C.POINTER(QTensor), _i, _i, _i, _i, _i, _i, _vp, _vp]),
    "imx_quantized_matmul_scratch_bytes": (_i, [_i, _i, _i, _i, _i, _i, C.POINTER(_sz)]),
    "imx_quantized_matmul_ws": (_i, [_vp, _i, C.POINTER(QTensor), _i, _i, _i, _i, _i, _vp, _vp, _sz, _vp]),
    "imx_expert_scratch_bytes": (_i, [C.POINTER(MoEConfig), _i, C.POINTER(_sz)]),
    "imx_expert_forward": (_i, [C.POINTER(MoEConfig), C.POINTER(QTensor), C.POINTER(QTensor), _vp, _i, _vp, _vp, _sz, _vp]),
    "imx_linear": (_i, [_vp, _i, _i, _vp, _i, _vp, _vp, _vp]),
    "imx_quantize": (_i, [_vp, _i, _i, _i, _i, _i, _f, _vp, _vp, _vp, _vp]),
    "imx_gather_qmm": (_i, [_vp, _vp, C.POINTER(QTensor), _vp, _i, _i, _i, _i, _i, _i, _vp, _vp]),
}

_lib = None


class IronMLXError(RuntimeError):
    """A call into libironmlx_b200.so returned a non-zero status
    (the analogue of the reference's `Error::Mlx`, mlx/src/error.rs:17-54)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[{code}] {message}")
        self.code = code


def lib() -> C.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m ironmlx_b200.build` "
                "(this package has no fallback path)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status: int) -> None:
    if status != OK:
        raise IronMLXError(status, lib().imx_last_error().decode())


def resolve_format(group_size, bits, mode):
    if mode not in MODE:
        raise IronMLXError(ERR_INVALID, f"unknown quantization mode {mode!r}")
    dg, db = MODE_DEFAULTS[mode]
    return (dg if group_size is None else int(group_size), db if bits is None else int(bits), MODE[mode])
