// Decoding of MLX's packed weight formats on the device (any format, eight
// consecutive values at a time).  Layouts: see include/ironmlx_b200.h.
//   affine  little-endian bit stream of `bits`-wide unsigned q per row;
//           w = scale*q + bias, scale/bias bf16 per `group` values
//   mxfp8   e4m3 bytes; w = q * 2^(s-127), s uint8 per 32 values
//   nvfp4   e2m1 nibbles (low nibble first); w = q * e4m3 scale per 16 values
//           (* one fp32 tensor scale, applied by the caller)
#pragma once
#include "common.cuh"

namespace imx {

// Row r of a [rows, in] quantized matrix.
struct QRow {
    const uint8_t* w;
    const uint8_t* s;
    const uint8_t* b;
};

__device__ __forceinline__ QRow qrow(const QMat& m, size_t row, int in, const QFormat& f) {
    QRow r;
    r.w = m.w + row * packed_row_bytes(in, f.bits);
    r.s = m.scales + row * scale_row_bytes(in, f);
    r.b = m.biases ? m.biases + row * scale_row_bytes(in, f) : nullptr;
    return r;
}

// Raw codes of the eight values k0..k0+7 (k0 a multiple of 8) of a row.
__device__ __forceinline__ uint64_t load_codes8(const uint8_t* roww, int k0, int bits) {
    const uint8_t* p = roww + (size_t)(k0 >> 3) * bits;   // 8 values = `bits` bytes
    if (bits == 4) return *reinterpret_cast<const uint32_t*>(p);
    if (bits == 8) return *reinterpret_cast<const uint64_t*>(p);
    if (bits == 2) return *reinterpret_cast<const uint16_t*>(p);
    uint64_t v = 0;
    for (int i = 0; i < bits; ++i) v |= (uint64_t)p[i] << (8 * i);
    return v;
}

// w[k0..k0+8) as fp32 (nvfp4: without the tensor scale).
__device__ __forceinline__ void dequant8(const QRow& r, int k0, const QFormat& f, float out[8]) {
    const uint64_t c = load_codes8(r.w, k0, f.bits);
    const int g = k0 / f.group;
    if (f.mode == IMX_MODE_AFFINE) {
        const float s = bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(r.s)[g]);
        const float b = bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(r.b)[g]);
        const uint32_t mask = (1u << f.bits) - 1u;
#pragma unroll
        for (int i = 0; i < 8; ++i)   // product and sum rounded separately (no fma), as numpy does
            out[i] = __fadd_rn(__fmul_rn((float)((uint32_t)(c >> (i * f.bits)) & mask), s), b);
    } else if (f.mode == IMX_MODE_MXFP8) {
        const float s = ue8m0_to_f32(r.s[g]);
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] = e4m3_to_f32((uint32_t)(c >> (8 * i)) & 0xffu) * s;
    } else {
        const float s = e4m3_to_f32(r.s[g]);
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] = e2m1_to_f32((uint32_t)(c >> (4 * i)) & 0xfu) * s;
    }
}

}  // namespace imx
