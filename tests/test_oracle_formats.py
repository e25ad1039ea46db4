"""The CPU checker's format code against hand-computed vectors and round trips."""
import numpy as np
import pytest

from oracle import formats as F


@pytest.mark.parametrize("bits", F.AFFINE_BITS)
def test_pack_unpack_round_trip(bits):
    rng = np.random.default_rng(bits)
    q = rng.integers(0, 1 << bits, size=(3, 5, 64), dtype=np.uint8)
    w = F.pack_bits(q, bits)
    assert w.dtype == np.uint32 and w.shape == (3, 5, 64 * bits // 32)
    assert np.array_equal(F.unpack_bits(w, bits), q)


def test_pack_known_words():
    # 4-bit: value i in nibble i, low nibble first
    q = np.arange(8, dtype=np.uint8)[None]
    assert F.pack_bits(q, 4)[0, 0] == 0x76543210
    # 8-bit: byte order
    q = np.array([[0x11, 0x22, 0x33, 0x44]], dtype=np.uint8)
    assert F.pack_bits(q, 8)[0, 0] == 0x44332211
    # 2-bit: 16 values per word, value i at bits [2i, 2i+2)
    q = (np.arange(16, dtype=np.uint8) % 4)[None]
    assert F.pack_bits(q, 2)[0, 0] == sum((i % 4) << (2 * i) for i in range(16))
    # 3-bit: contiguous little-endian bit stream, 32 values -> 3 words
    q = (np.arange(32, dtype=np.uint8) % 8)[None]
    stream = sum(int(v) << (3 * i) for i, v in enumerate(q[0]))
    words = F.pack_bits(q, 3)[0]
    assert [int(w) for w in words] == [(stream >> (32 * j)) & 0xFFFFFFFF for j in range(3)]
    # 6-bit: 16 values -> 3 words
    q = (np.arange(16, dtype=np.uint8) * 4 + 1)[None]
    stream = sum(int(v) << (6 * i) for i, v in enumerate(q[0]))
    assert [int(w) for w in F.pack_bits(q, 6)[0]] == [(stream >> (32 * j)) & 0xFFFFFFFF for j in range(3)]


def test_affine_dequantize_known():
    # one group of 64 4-bit codes 0..15 repeated, scale 0.5, bias -2
    q = (np.arange(64) % 16).astype(np.uint8)[None]
    w = F.pack_bits(q, 4)
    s = np.array([[0.5]], dtype=F.bf16)
    b = np.array([[-2.0]], dtype=F.bf16)
    d = F.affine_dequantize(w, s, b, 64, 4)
    assert np.array_equal(d[0], (np.arange(64) % 16) * 0.5 - 2.0)


@pytest.mark.parametrize("bits", F.AFFINE_BITS)
@pytest.mark.parametrize("group", [32, 64, 128])
def test_affine_quantize_error_bound(bits, group):
    rng = np.random.default_rng(100 + bits)
    w = (rng.standard_normal((16, 256)) * 0.02).astype(np.float32)
    p, s, b = F.affine_quantize(w, group, bits)
    assert p.shape == (16, 256 * bits // 32) and s.shape == b.shape == (16, 256 // group)
    d = F.affine_dequantize(p, s, b, group, bits)
    # anchoring the grid on one edge can push the far edge one step outside the
    # code range; bf16 rounding of scale/bias adds up to (2^bits-1)*step/256 + |bias|/256
    step = np.abs(s.astype(np.float32)).repeat(group, -1)
    bias = np.abs(b.astype(np.float32)).repeat(group, -1)
    bound = (1.01 + ((1 << bits) - 1) / 256) * step + bias / 256
    assert np.all(np.abs(d - w) <= bound)
    # the anchored edge of every group is one of the extreme codes
    codes = F.unpack_bits(p, bits).reshape(16, -1, group)
    assert np.all((codes.min(-1) == 0) | (codes.max(-1) == (1 << bits) - 1))


def test_affine_quantize_known_group():
    # group spanning [-1.5, 0]: |min| > |max| -> anchored on the min, positive scale
    w = np.linspace(-1.5, 0.0, 64, dtype=np.float32)[None]
    p, s, b = F.affine_quantize(w, 64, 4)
    assert float(b[0, 0]) == -1.5 and abs(float(s[0, 0]) - 0.1) < 1e-3
    codes = F.unpack_bits(p, 4)[0]
    assert codes[0] == 0 and codes[-1] == 15 and np.all(np.diff(codes.astype(int)) >= 0)


def test_fp_element_decoders():
    assert np.array_equal(F.e2m1_to_f32(np.arange(16)),
                          np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6], np.float32))
    # e4m3: 0x38 = 1.0, 0x7e = 448, 0x01 = 2^-9, 0xc0 = -2.0
    assert np.array_equal(F.e4m3_to_f32(np.array([0x38, 0x7E, 0x01, 0xC0], np.uint8)),
                          np.array([1.0, 448.0, 2.0 ** -9, -2.0], np.float32))


def test_mxfp8_known_and_bound():
    w = np.zeros((1, 32), np.float32)
    w[0, 0] = 448.0      # amax/448 = 1 -> e = 0 -> scale byte 127, code 0x7e
    w[0, 1] = 1.0
    p, s = F.mxfp8_quantize(w)
    assert s[0, 0] == 127
    by = p.view(np.uint8)
    assert by[0, 0] == 0x7E and by[0, 1] == 0x38
    rng = np.random.default_rng(5)
    w = (rng.standard_normal((8, 128)) * 0.02).astype(np.float32)
    p, s = F.mxfp8_quantize(w)
    d = F.mxfp8_dequantize(p, s)
    amax = np.abs(w.reshape(8, 4, 32)).max(-1).repeat(32, -1)
    assert np.all(np.abs(d - w) <= np.maximum(np.abs(w) * 2 ** -4, amax * 2 ** -9))


def test_nvfp4_known_and_bound():
    rng = np.random.default_rng(6)
    w = (rng.standard_normal((8, 128)) * 0.02).astype(np.float32)
    p, s, t = F.nvfp4_quantize(w)
    assert p.shape == (8, 16) and s.shape == (8, 8) and t > 0
    d = F.nvfp4_dequantize(p, s, 16, t)
    amax = np.abs(w.reshape(8, 8, 16)).max(-1).repeat(16, -1)
    # e2m1 grid spacing is at most amax/3 between 4 and 6; scale rounding adds 2^-4
    assert np.all(np.abs(d - w) <= amax * (1 / 6 + 2 ** -3))
    # exact case: values on the grid with scale 1 and tensor scale 1
    grid = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0.5, -1, -1.5, -2, -3, -4, -6, 6], np.float32)[None]
    p, s, t = F.nvfp4_quantize(grid, with_global_scale=False)
    assert np.array_equal(F.nvfp4_dequantize(p, s, 16, t), grid)


def test_resolve_and_errors():
    assert F.resolve(None, None, "affine") == (64, 4)
    assert F.resolve(None, None, "mxfp8") == (32, 8)
    assert F.resolve(None, None, "nvfp4") == (16, 4)
    for bad in [(64, 7, "affine"), (48, 4, "affine"), (64, 8, "mxfp8"), (32, 4, "nvfp4"), (64, 4, "int4")]:
        with pytest.raises(ValueError):
            F.resolve(*bad)


@pytest.mark.parametrize("mode,bits,group", [("affine", 4, 64), ("affine", 3, 32), ("affine", 8, 128),
                                             ("mxfp8", 8, 32), ("nvfp4", 4, 16)])
def test_quantized_matmul_matches_dense(mode, bits, group):
    rng = np.random.default_rng(9)
    w = (rng.standard_normal((24, 128)) * 0.02).astype(np.float32)
    x = F.to_bf16(rng.standard_normal((5, 128)))
    p, s, b, t = F.quantize(w, group, bits, mode)
    wd = F.dequantize(p, s, b, group, bits, mode, t)
    y = F.quantized_matmul(x, p, s, b, True, group, bits, mode, t)
    assert np.allclose(y, x @ wd.T, rtol=1e-5, atol=1e-6)
    x2 = F.to_bf16(rng.standard_normal((5, 24)))
    y2 = F.quantized_matmul(x2, p, s, b, False, group, bits, mode, t)
    assert np.allclose(y2, x2 @ wd, rtol=1e-5, atol=1e-6)
