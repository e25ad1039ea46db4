"""Host-side mirror of the reference's quantized-op wrappers
(mlx/src/ops.rs:630-727): same names, argument order and meaning, errors
raised as `IronMLXError` the way the reference returns `Error::Mlx`.

Tensors are torch CUDA tensors used as plain device buffers; every op is one
call into the C ABI on the given stream.  There is no fallback path.

Packed weights are int32 (the bits of MLX's uint32 words), affine
scales/biases bf16, mxfp8/nvfp4 scales uint8.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from ._lib import IronMLXError, QTensor, check, lib, resolve_format

_OUT_DTYPES = {torch.bfloat16: 0, torch.float32: 1, torch.float16: 2}


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream_ptr(stream=None) -> int:
    """cudaStream_t of a torch stream (default: the current stream)."""
    s = torch.cuda.current_stream() if stream is None else stream
    return s.cuda_stream


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise IronMLXError(_lib.ERR_INVALID, "tensors must be contiguous CUDA tensors")


def qtensor(w, scales, biases=None, global_scale: Optional[float] = None) -> QTensor:
    return QTensor(_ptr(w), _ptr(scales), _ptr(biases), 1.0 if global_scale is None else float(global_scale))


def _packed_cols(in_dim: int, bits: int) -> int:
    return in_dim * bits // 32


def dequantize(w, scales, biases=None, group_size=None, bits=None, mode: str = "affine",
               stream=None, dtype=torch.bfloat16, global_scale=None) -> torch.Tensor:
    """`ops::dequantize` (mlx/src/ops.rs:653-686): packed [.., out, in*bits/32] -> [.., out, in]."""
    g, b, m = resolve_format(group_size, bits, mode)
    _require_cuda(w, scales, biases)
    in_dim = w.shape[-1] * 32 // b
    rows = w.numel() // w.shape[-1]
    out = torch.empty(*w.shape[:-1], in_dim, dtype=dtype, device=w.device)
    qt = qtensor(w, scales, biases, global_scale)
    check(lib().imx_dequantize(C.byref(qt), rows, in_dim, g, b, m, _OUT_DTYPES[dtype], out.data_ptr(),
                               stream_ptr(stream)))
    return out


def quantized_matmul(x, w, scales, biases=None, transpose: bool = True, group_size=None, bits=None,
                     mode: str = "affine", stream=None, global_scale=None) -> torch.Tensor:
    """`ops::quantized_matmul` (mlx/src/ops.rs:695-727): `x @ dequantize(w)^T`
    (transpose=True, how every layer of the path calls it) or `x @ dequantize(w)`."""
    g, b, m = resolve_format(group_size, bits, mode)
    _require_cuda(x, w, scales, biases)
    if x.dtype != torch.bfloat16:
        raise IronMLXError(_lib.ERR_INVALID, "quantized_matmul: x must be bfloat16")
    if w.dim() != 2:
        raise IronMLXError(_lib.ERR_INVALID, "quantized_matmul: w must be 2-D [out, in*bits/32]")
    n_out, in_dim = w.shape[0], w.shape[1] * 32 // b
    inner = in_dim if transpose else n_out
    if x.shape[-1] != inner:
        raise IronMLXError(_lib.ERR_INVALID,
                           f"quantized_matmul: last dimension of x ({x.shape[-1]}) does not match {inner}")
    m_rows = x.numel() // inner
    x = x.contiguous()
    y = torch.empty(*x.shape[:-1], n_out if transpose else in_dim, dtype=torch.bfloat16, device=x.device)
    qt = qtensor(w, scales, biases, global_scale)
    if transpose:
        # the layers' form: on the expert kernels where they take the shape (scratch cached per device and size)
        nb = C.c_size_t(0)
        check(lib().imx_quantized_matmul_scratch_bytes(m_rows, n_out, in_dim, g, b, m, C.byref(nb)))
        ws = scratch(x.device, nb.value)
        check(lib().imx_quantized_matmul_ws(x.data_ptr(), m_rows, C.byref(qt), n_out, in_dim, g, b, m, y.data_ptr(),
                                            ws.data_ptr(), ws.numel(), stream_ptr(stream)))
        return y
    check(lib().imx_quantized_matmul(x.data_ptr(), m_rows, C.byref(qt), n_out, in_dim, 0,
                                     g, b, m, y.data_ptr(), stream_ptr(stream)))
    return y


_SCRATCH = {}


def scratch(device, nbytes: int) -> torch.Tensor:
    """A zero-filled device buffer of at least nbytes, kept per device (the layer calls' scratch; one stream of
    calls at a time per device)."""
    key = (device.type, device.index)
    buf = _SCRATCH.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _SCRATCH[key] = buf
    return buf


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """Dense `x @ W^T (+ b)` (mlx/src/nn/linear.rs:170-177), bf16 in and out, fp32 accumulation."""
    _require_cuda(x, weight, bias)
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or weight.dim() != 2 or x.shape[-1] != weight.shape[1]:
        raise IronMLXError(_lib.ERR_INVALID, "linear: x [.., in] and weight [out, in] must be bfloat16")
    x = x.contiguous()
    n_out, in_dim = weight.shape
    y = torch.empty(*x.shape[:-1], n_out, dtype=torch.bfloat16, device=x.device)
    check(lib().imx_linear(x.data_ptr(), x.numel() // in_dim, in_dim, weight.data_ptr(), n_out, _ptr(bias), y.data_ptr(),
                           stream_ptr(stream)))
    return y


def expert_forward(x: torch.Tensor, gate_up_w, gate_up_s, gate_up_b, down_w, down_s, down_b, group_size=None, bits=None,
                   mode: str = "affine", stream=None, gate_up_scale=None, down_scale=None) -> torch.Tensor:
    """`down(silu(gate(x)) * up(x))` for one expert over all rows of x (mlx/src/nn/moe.rs:26-32,
    mlx/src/nn/mlp.rs:27-33).  gate_up_*: [2I, .] with the gate rows first; down_*: [H, .]."""
    g, b, m = resolve_format(group_size, bits, mode)
    _require_cuda(x, gate_up_w, gate_up_s, gate_up_b, down_w, down_s, down_b)
    hidden = x.shape[-1]
    inter = gate_up_w.shape[-2] // 2
    if x.dtype != torch.bfloat16 or down_w.shape[-2] != hidden:
        raise IronMLXError(_lib.ERR_INVALID, "expert_forward: x must be bfloat16 [.., hidden] matching down [hidden, .]")
    x = x.contiguous()
    rows = x.numel() // hidden
    y = torch.empty_like(x)
    cfg = _lib.MoEConfig(hidden, 1, 1, inter, 0, 1, m, b, g, 0)
    nb = C.c_size_t(0)
    check(lib().imx_expert_scratch_bytes(C.byref(cfg), rows, C.byref(nb)))
    ws = scratch(x.device, nb.value)
    gu, dn = qtensor(gate_up_w, gate_up_s, gate_up_b, gate_up_scale), qtensor(down_w, down_s, down_b, down_scale)
    check(lib().imx_expert_forward(C.byref(cfg), C.byref(gu), C.byref(dn), x.data_ptr(), rows, y.data_ptr(), ws.data_ptr(),
                                   ws.numel(), stream_ptr(stream)))
    return y


def quantize(w, group_size=None, bits=None, mode: str = "affine", stream=None, global_scale=None):
    """Quantize float weights [.., out, in] -> (packed int32, scales, biases-or-None).
    For nvfp4 the fp32 tensor scale is taken from `global_scale`, or derived
    from the tensor's absolute maximum, and returned as a fourth element."""
    g, b, m = resolve_format(group_size, bits, mode)
    w = w.to(torch.float32).contiguous()
    _require_cuda(w)
    in_dim = w.shape[-1]
    rows = w.numel() // in_dim
    if in_dim % g or (in_dim * b) % 32:
        raise IronMLXError(_lib.ERR_INVALID, f"quantize: last dimension {in_dim} does not fit group {g} / {b} bits")
    packed = torch.empty(*w.shape[:-1], _packed_cols(in_dim, b), dtype=torch.int32, device=w.device)
    sdtype = torch.bfloat16 if mode == "affine" else torch.uint8
    scales = torch.empty(*w.shape[:-1], in_dim // g, dtype=sdtype, device=w.device)
    biases = torch.empty_like(scales) if mode == "affine" else None
    gs = 1.0
    if mode == "nvfp4":
        gs = float(global_scale) if global_scale is not None else max(float(w.abs().max()), 1e-30) / (6.0 * 448.0)
    check(lib().imx_quantize(w.data_ptr(), rows, in_dim, g, b, m, gs, packed.data_ptr(), scales.data_ptr(),
                             _ptr(biases), stream_ptr(stream)))
    if mode == "nvfp4":
        return packed, scales, None, gs
    return packed, scales, biases


def gather_qmm(x, w, scales, biases, lhs_indices, rhs_indices, group_size=None, bits=None,
               mode: str = "affine", stream=None, global_scale=None) -> torch.Tensor:
    """y[j] = x[lhs_indices[j]] @ dequantize(w[rhs_indices[j]])^T: the per-row
    form of the reference's take_axis + quantized_matmul per expert
    (mlx/src/nn/moe.rs:124-130).  w: [E, out, in*bits/32]."""
    g, b, m = resolve_format(group_size, bits, mode)
    _require_cuda(x, w, scales, biases, lhs_indices, rhs_indices)
    if x.dtype != torch.bfloat16 or w.dim() != 3:
        raise IronMLXError(_lib.ERR_INVALID, "gather_qmm: x must be bfloat16 and w 3-D [E, out, in*bits/32]")
    n_out, in_dim = w.shape[1], w.shape[2] * 32 // b
    n_rows = rhs_indices.numel()
    y = torch.empty(n_rows, n_out, dtype=torch.bfloat16, device=x.device)
    qt = qtensor(w, scales, biases, global_scale)
    lhs = None if lhs_indices is None else lhs_indices.to(torch.int32)
    check(lib().imx_gather_qmm(x.data_ptr(), _ptr(lhs), C.byref(qt), rhs_indices.to(torch.int32).data_ptr(),
                               n_rows, n_out, in_dim, g, b, m, y.data_ptr(), stream_ptr(stream)))
    return y


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float, stream=None) -> torch.Tensor:
    """`fast::rms_norm` (mlx/src/fast.rs:37-49): x * rsqrt(mean(x^2) + eps) * weight over the last
    axis; bf16 in and out."""
    _require_cuda(x, weight)
    if x.dtype != torch.bfloat16 or (weight is not None and weight.dtype != torch.bfloat16):
        raise IronMLXError(_lib.ERR_INVALID, "rms_norm: x and weight must be bfloat16")
    h = x.shape[-1]
    if weight is not None and weight.numel() != h:
        raise IronMLXError(_lib.ERR_INVALID, f"rms_norm: weight has {weight.numel()} elements, rows have {h}")
    x = x.contiguous()
    y = torch.empty_like(x)
    check(lib().imx_rms_norm(x.data_ptr(), x.numel() // h, h, None if weight is None else weight.data_ptr(),
                             float(eps), y.data_ptr(), stream_ptr(stream)))
    return y
