"""MLX quantized weight formats, restated in numpy (test infrastructure only).

The reference never spells these formats out in code: it passes packed
tensors straight to `mlx_dequantize` / `mlx_quantized_matmul`
(mlx/src/ops.rs:653-727) and documents them only in comments
(mlx/src/ops.rs:646-652 "packed uint32 ... per-group scale factors ...
per-group biases", ops.rs:688-693 "`x @ dequantize(w, scales, biases)^T` ...
Supported modes: affine (2/3/4/6/8 bit), mxfp8, nvfp4") and in the shapes the
expert builder slices (mlx/src/model/qwen35.rs:581-590,653-687).  The bit
layouts below follow MLX's public documentation of `mx.quantize`:

affine  w ~= scale * q + bias, q an unsigned `bits`-wide integer.  A row of
        `in` values is a little-endian bit stream (value i occupies bits
        [i*bits, (i+1)*bits)), stored as uint32 words, so the packed shape is
        [out, in*bits/32].  For 2/4/8 bits this is "element i%(32/bits) of
        word i/(32/bits), low bits first"; 3/5/6-bit values straddle bytes.
        scales/biases: [out, in/group_size] in the activation float type
        (bf16 here).
mxfp8   q is float8 e4m3 (fn variant), four per uint32 in byte order; one
        ue8m0 scale (a biased power of two, 2**(s-127)) per 32 values; no
        biases.
nvfp4   q is float4 e2m1, eight per uint32 low nibble first; one float8 e4m3
        scale per 16 values; optionally one fp32 scale for the whole tensor.

Parity between the CUDA path and this oracle is defined on the packed
tensors, so the rounding policy of the quantizers below cannot cause a
mismatch; it matters only for how well the synthetic weights resemble real
checkpoints.
"""
from __future__ import annotations

import math

import ml_dtypes
import numpy as np

bf16 = ml_dtypes.bfloat16
AFFINE_BITS = (2, 3, 4, 5, 6, 8)


def to_bf16(a) -> np.ndarray:
    """Round to bfloat16 (nearest even) and return the values as float32."""
    return np.asarray(a, dtype=np.float32).astype(bf16).astype(np.float32)


# ── bit packing ──────────────────────────────────────────────────────────────

def pack_bits(q: np.ndarray, bits: int) -> np.ndarray:
    """Pack unsigned `bits`-wide integers along the last axis into uint32 words.

    Little-endian bit stream per row: value i sits at bits [i*bits, (i+1)*bits).
    """
    q = np.ascontiguousarray(q)
    n = q.shape[-1]
    if (n * bits) % 32:
        raise ValueError(f"row of {n} {bits}-bit values does not fill whole uint32 words")
    lead = q.shape[:-1]
    per = math.lcm(bits, 8) // bits          # values per whole-byte unit
    nbytes = per * bits // 8                 # bytes per unit
    q64 = q.reshape(-1, n // per, per).astype(np.uint64)
    acc = np.zeros(q64.shape[:2], dtype=np.uint64)
    for i in range(per):
        acc |= q64[:, :, i] << np.uint64(i * bits)
    out = np.empty(acc.shape + (nbytes,), dtype=np.uint8)
    for b in range(nbytes):
        out[:, :, b] = ((acc >> np.uint64(8 * b)) & np.uint64(0xFF)).astype(np.uint8)
    out = out.reshape(-1, n * bits // 8)
    return out.view("<u4").reshape(lead + (n * bits // 32,))


def unpack_bits(w: np.ndarray, bits: int) -> np.ndarray:
    """Inverse of `pack_bits`: uint32 words -> uint8 values along the last axis."""
    w = np.ascontiguousarray(w).astype("<u4", copy=False)
    lead = w.shape[:-1]
    n = w.shape[-1] * 32 // bits
    per = math.lcm(bits, 8) // bits
    nbytes = per * bits // 8
    by = w.view(np.uint8).reshape(-1, n // per, nbytes).astype(np.uint64)
    acc = np.zeros(by.shape[:2], dtype=np.uint64)
    for b in range(nbytes):
        acc |= by[:, :, b] << np.uint64(8 * b)
    out = np.empty(acc.shape + (per,), dtype=np.uint8)
    mask = np.uint64((1 << bits) - 1)
    for i in range(per):
        out[:, :, i] = ((acc >> np.uint64(i * bits)) & mask).astype(np.uint8)
    return out.reshape(lead + (n,))


# ── affine ───────────────────────────────────────────────────────────────────

def affine_quantize(w, group_size: int = 64, bits: int = 4):
    """Quantize [.., out, in] float weights to (packed uint32, scales, biases).

    Per group of `group_size` values along the last axis, following the
    algorithm MLX documents for `mx.quantize(mode="affine")`: the grid is
    anchored on whichever of min/max has the larger magnitude so that that
    edge is represented exactly, scale = (max-min)/(2**bits-1) (sign chosen by
    the anchored side), q = clip(round((w-bias)/scale), 0, 2**bits-1).
    scales/biases are returned in bfloat16, the activation type of the path.
    """
    if bits not in AFFINE_BITS:
        raise ValueError(f"affine bits must be one of {AFFINE_BITS}")
    w = np.asarray(w, dtype=np.float32)
    n = w.shape[-1]
    if n % group_size:
        raise ValueError("last dimension must be a multiple of group_size")
    g = w.reshape(w.shape[:-1] + (n // group_size, group_size))
    n_bins = np.float32((1 << bits) - 1)
    eps = np.float32(1e-7)
    w_max = g.max(-1)
    w_min = g.min(-1)
    side = np.abs(w_min) > np.abs(w_max)
    scale = np.maximum((w_max - w_min) / n_bins, eps).astype(np.float32)
    scale = np.where(side, scale, -scale).astype(np.float32)
    edge = np.where(side, w_min, w_max).astype(np.float32)
    q0 = np.rint(edge / scale)
    nz = q0 != 0
    scale = np.where(nz, edge / np.where(nz, q0, 1), scale).astype(np.float32)
    bias = np.where(nz, edge, np.float32(0)).astype(np.float32)
    q = np.rint((g - bias[..., None]) / scale[..., None])
    q = np.clip(q, 0, n_bins).astype(np.uint8).reshape(w.shape)
    return pack_bits(q, bits), scale.astype(bf16), bias.astype(bf16)


def affine_dequantize(w, scales, biases, group_size: int = 64, bits: int = 4) -> np.ndarray:
    """packed -> float32 [.., out, in]: scale*q + bias evaluated in fp32."""
    q = unpack_bits(w, bits).astype(np.float32)
    s = np.asarray(scales).astype(np.float32)
    b = np.asarray(biases).astype(np.float32)
    n = q.shape[-1]
    qg = q.reshape(q.shape[:-1] + (n // group_size, group_size))
    return (qg * s[..., None] + b[..., None]).reshape(q.shape).astype(np.float32)


# ── mxfp8: e4m3 values, ue8m0 scale per 32 ───────────────────────────────────

E4M3_MAX = 448.0
E2M1_MAX = 6.0


def mxfp8_quantize(w, group_size: int = 32):
    """-> (packed uint32 [.., out, in/4], scales uint8 ue8m0 [.., out, in/32])."""
    w = np.asarray(w, dtype=np.float32)
    n = w.shape[-1]
    g = w.reshape(w.shape[:-1] + (n // group_size, group_size))
    amax = np.abs(g).max(-1)
    # smallest power of two 2**e with amax / 2**e <= 448, from the exponent bits
    mant, ex = np.frexp((amax / np.float32(E4M3_MAX)).astype(np.float32))
    e = np.where(mant == 0.5, ex - 1, ex)
    e = np.clip(e, -127, 127).astype(np.int32)
    e = np.where(amax == 0, -127, e)
    scale = np.exp2(e.astype(np.float32))
    v = np.clip(g / scale[..., None], -E4M3_MAX, E4M3_MAX).astype(np.float32)
    q = v.astype(ml_dtypes.float8_e4m3fn).view(np.uint8).reshape(w.shape)
    packed = np.ascontiguousarray(q).view("<u4")
    return packed, (e + 127).astype(np.uint8)


def e4m3_to_f32(u8: np.ndarray) -> np.ndarray:
    return np.asarray(u8, dtype=np.uint8).view(ml_dtypes.float8_e4m3fn).astype(np.float32)


def e2m1_to_f32(nib: np.ndarray) -> np.ndarray:
    lut = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6], dtype=np.float32)
    return lut[np.asarray(nib, dtype=np.uint8) & 0xF]


def mxfp8_dequantize(w, scales, group_size: int = 32) -> np.ndarray:
    q = np.ascontiguousarray(w).astype("<u4", copy=False).view(np.uint8)
    v = e4m3_to_f32(q)
    s = np.exp2(np.asarray(scales).astype(np.float32) - 127.0).astype(np.float32)
    n = v.shape[-1]
    vg = v.reshape(v.shape[:-1] + (n // group_size, group_size))
    return (vg * s[..., None]).reshape(v.shape).astype(np.float32)


# ── nvfp4: e2m1 values, e4m3 scale per 16, optional fp32 tensor scale ────────

def nvfp4_quantize(w, group_size: int = 16, with_global_scale: bool = True):
    """-> (packed uint32 [.., out, in/8], scales uint8 e4m3 [.., out, in/16], fp32 tensor scale)."""
    w = np.asarray(w, dtype=np.float32)
    n = w.shape[-1]
    g = w.reshape(w.shape[:-1] + (n // group_size, group_size))
    amax = np.abs(g).max(-1)
    if with_global_scale:
        t = np.float32(max(float(amax.max()), 1e-30) / (E2M1_MAX * E4M3_MAX))
    else:
        t = np.float32(1.0)
    s = np.clip(amax / E2M1_MAX / t, 0, E4M3_MAX).astype(np.float32)
    s8 = s.astype(ml_dtypes.float8_e4m3fn)
    sf = s8.astype(np.float32) * t
    sf_safe = np.where(sf == 0, np.float32(1), sf)
    v = np.clip(g / sf_safe[..., None], -E2M1_MAX, E2M1_MAX).astype(np.float32)
    nib = v.astype(ml_dtypes.float4_e2m1fn).view(np.uint8).reshape(w.shape) & 0xF
    return pack_bits(nib, 4), s8.view(np.uint8), t


def nvfp4_dequantize(w, scales, group_size: int = 16, global_scale=1.0) -> np.ndarray:
    nib = unpack_bits(w, 4)
    v = e2m1_to_f32(nib)
    s = e4m3_to_f32(scales)
    n = v.shape[-1]
    vg = v.reshape(v.shape[:-1] + (n // group_size, group_size))
    # value x block scale is exact in fp32 (2 + 4 significant bits); one rounding with the tensor scale
    return ((vg * s[..., None]) * np.float32(global_scale)).reshape(v.shape).astype(np.float32)


# ── the reference's two quantized ops (mlx/src/ops.rs:653-727) ──────────────

MODE_DEFAULTS = {"affine": (64, 4), "mxfp8": (32, 8), "nvfp4": (16, 4)}


def resolve(group_size, bits, mode):
    """Fill `None` group_size/bits the way the reference's optionals default."""
    if mode not in MODE_DEFAULTS:
        raise ValueError(f"unknown quantization mode {mode!r}")
    dg, db = MODE_DEFAULTS[mode]
    group_size = dg if group_size is None else group_size
    bits = db if bits is None else bits
    if mode == "mxfp8" and (group_size, bits) != (32, 8):
        raise ValueError("mxfp8 requires group_size=32, bits=8")
    if mode == "nvfp4" and (group_size, bits) != (16, 4):
        raise ValueError("nvfp4 requires group_size=16, bits=4")
    if mode == "affine" and (bits not in AFFINE_BITS or group_size not in (32, 64, 128)):
        raise ValueError("affine requires bits in 2/3/4/5/6/8 and group_size in 32/64/128")
    return group_size, bits


def quantize(w, group_size=None, bits=None, mode="affine"):
    """-> (packed, scales, biases-or-None, global_scale-or-None)."""
    group_size, bits = resolve(group_size, bits, mode)
    if mode == "affine":
        p, s, b = affine_quantize(w, group_size, bits)
        return p, s, b, None
    if mode == "mxfp8":
        p, s = mxfp8_quantize(w, group_size)
        return p, s, None, None
    p, s, t = nvfp4_quantize(w, group_size)
    return p, s, None, t


def dequantize(w, scales, biases=None, group_size=None, bits=None, mode="affine", global_scale=None):
    """`ops::dequantize` (mlx/src/ops.rs:653-686): packed -> float32 matrix."""
    group_size, bits = resolve(group_size, bits, mode)
    if mode == "affine":
        if biases is None:
            raise ValueError("affine mode needs biases")
        return affine_dequantize(w, scales, biases, group_size, bits)
    if mode == "mxfp8":
        return mxfp8_dequantize(w, scales, group_size)
    return nvfp4_dequantize(w, scales, group_size, 1.0 if global_scale is None else global_scale)


def quantized_matmul(x, w, scales, biases=None, transpose=True, group_size=None, bits=None,
                     mode="affine", global_scale=None):
    """`ops::quantized_matmul` (mlx/src/ops.rs:695-727), fp32 with float64 accumulation.

    transpose=True: x[.., in] @ dequantize(w)[out, in]^T  (how every layer on
    the path calls it, mlx/src/nn/linear.rs:51-63); transpose=False:
    x[.., out] @ dequantize(w)[out, in].
    """
    wd = dequantize(w, scales, biases, group_size, bits, mode, global_scale).astype(np.float64)
    x = np.asarray(x, dtype=np.float64)
    y = x @ (wd.T if transpose else wd)
    return y.astype(np.float32)


def bytes_per_weight(mode: str, bits: int, group_size: int) -> float:
    """Stored bytes per weight element (payload + per-group metadata)."""
    if mode == "affine":
        return bits / 8 + 4 / group_size
    if mode == "mxfp8":
        return 1 + 1 / 32
    if mode == "nvfp4":
        return 0.5 + 1 / 16
    raise ValueError(mode)
