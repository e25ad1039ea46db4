"""ctypes wrapper of oracle/moe_ref.c (test infrastructure only): the C/OpenMP
restatement of the reference's MoE block, used as a second checker and as the
timed CPU baseline."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

from . import moe as O

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "_build", "libmoe_ref.so")
_MODE = {"affine": 0, "mxfp8": 1, "nvfp4": 2}


class RefQ(C.Structure):
    _fields_ = [("w", C.c_void_p), ("scales", C.c_void_p), ("biases", C.c_void_p), ("global_scale", C.c_float)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        src = os.path.join(HERE, "moe_ref.c")
        if not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
            subprocess.run(["make", "-C", HERE], check=True, capture_output=True)
        _lib = C.CDLL(LIB)
        _lib.moe_ref_threads.restype = C.c_int
        _lib.moe_ref_forward.restype = C.c_int
    return _lib


def threads() -> int:
    return int(lib().moe_ref_threads())


def _q(q, keep):
    if q is None:
        return RefQ(None, None, None, 1.0)
    arrs = [np.ascontiguousarray(q.w), np.ascontiguousarray(q.scales),
            None if q.biases is None else np.ascontiguousarray(q.biases)]
    keep.extend(arrs)
    return RefQ(arrs[0].ctypes.data, arrs[1].ctypes.data, None if arrs[2] is None else arrs[2].ctypes.data,
                1.0 if q.global_scale is None else float(q.global_scale))


def prepare(x, p: O.MoEParams):
    """Marshals the arguments once; returns a zero-argument callable running one
    forward pass and the dict of output arrays it fills."""
    from . import formats as F
    keep = []
    n, h = x.shape
    e, k = p.num_experts, p.num_experts_per_tok
    gu = p.gate_up
    i = gu.w.shape[1] // 2
    i_s = 0 if p.shared_gate_proj is None else p.shared_gate_proj.w.shape[0]
    xb = np.ascontiguousarray(np.asarray(x, dtype=np.float32).astype(F.bf16))
    rw = np.ascontiguousarray(np.asarray(p.router_w).astype(F.bf16))
    bias = None if p.router_logit_bias is None else np.ascontiguousarray(p.router_logit_bias, dtype=np.float32)
    sg = None if p.shared_expert_gate_w is None else np.ascontiguousarray(np.asarray(p.shared_expert_gate_w).astype(F.bf16))
    out = {"y": np.empty((n, h), np.float32), "top_idx": np.empty((n, k), np.int32),
           "top_w": np.empty((n, k), np.float32), "perm": np.empty(n * k, np.int32), "counts": np.empty(e, np.int32)}
    args = [C.c_int(v) for v in (n, h, e, k, i, i_s, int(p.norm_topk_prob), _MODE[gu.mode], gu.bits, gu.group_size)]
    args += [C.c_void_p(xb.ctypes.data), C.c_void_p(rw.ctypes.data),
             C.c_void_p(None if bias is None else bias.ctypes.data),
             _q(p.gate_up, keep), _q(p.down, keep), _q(p.shared_gate_proj, keep), _q(p.shared_up_proj, keep),
             _q(p.shared_down_proj, keep), C.c_void_p(None if sg is None else sg.ctypes.data)]
    args += [C.c_void_p(out[name].ctypes.data) for name in ("y", "top_idx", "top_w", "perm", "counts")]
    keep.extend([xb, rw, bias, sg])
    fn = lib().moe_ref_forward

    def run():
        rc = fn(*args)
        assert rc == 0
        return out

    run._keep = keep
    return run, out


def set_bf16_logits(on: bool) -> None:
    """Router in the reference's dtypes (see oracle.moe.route(bf16_logits=True)); process-wide, off by default."""
    lib().moe_ref_set_bf16_logits(C.c_int(1 if on else 0))


def moe_forward(x, p: O.MoEParams):
    run, out = prepare(x, p)
    return run()
