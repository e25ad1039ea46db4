// Shared device/host helpers for the MoE-block kernels (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <string>

#include "../../include/ironmlx_b200.h"

namespace imx {

// ── error plumbing (return codes + thread-local message, never abort) ───────
void set_error(const char* fmt, ...);
const char* last_error();

#define IMX_CHECK_CUDA(expr)                                                        \
    do {                                                                            \
        cudaError_t _e = (expr);                                                    \
        if (_e != cudaSuccess) {                                                    \
            ::imx::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                             __FILE__, __LINE__);                                   \
            return IMX_ERR_CUDA;                                                    \
        }                                                                           \
    } while (0)

#define IMX_REQUIRE(cond, ...)                 \
    do {                                       \
        if (!(cond)) {                         \
            ::imx::set_error(__VA_ARGS__);     \
            return IMX_ERR_INVALID;            \
        }                                      \
    } while (0)

#define IMX_TRY(expr)                   \
    do {                                \
        int _s = (expr);                \
        if (_s != IMX_OK) return _s;    \
    } while (0)

// Every kernel launch of the library is counted (a process-wide counter read through imx_launch_count):
// callers that replay a captured graph multiply the launches recorded during capture by their replays.
void count_launch();
#define IMX_LAUNCHED() ::imx::count_launch()

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ── format description shared by all kernels ────────────────────────────────
struct QFormat {
    int mode;        // IMX_MODE_*
    int bits;        // stored bits per value
    int group;       // values per scale
};

// Bytes of one packed row of `in` values.
__host__ __device__ inline size_t packed_row_bytes(int in, int bits) { return (size_t)in * bits / 8; }
// Bytes of one row of scales (and of biases, when the mode has them).
__host__ __device__ inline size_t scale_row_bytes(int in, const QFormat& f) {
    return (size_t)(in / f.group) * (f.mode == IMX_MODE_AFFINE ? 2 : 1);
}

// One quantized matrix [rows, in] (or a stack of them) on the device.
struct QMat {
    const uint8_t* w;        // packed values
    const uint8_t* scales;   // bf16 (affine) or uint8 (mxfp8: ue8m0, nvfp4: e4m3)
    const uint8_t* biases;   // bf16 (affine) or nullptr
    float global_scale;      // nvfp4 tensor scale, 1 otherwise
};

#ifdef __CUDACC__
// ── small device helpers ─────────────────────────────────────────────────────
__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) { return __uint_as_float(((uint32_t)b) << 16); }

__device__ __forceinline__ float e4m3_to_f32(uint32_t v) {
    // fp8 e4m3 (fn): sign 1, exponent 4 (bias 7), mantissa 3.  Placing the
    // seven low bits four positions below an fp16's exponent field gives the
    // same value scaled by 2^-8 for normals and subnormals alike.
    uint16_t h = (uint16_t)(((v & 0x80u) << 8) | ((v & 0x7fu) << 7));
    return __half2float(__ushort_as_half(h)) * 256.0f;
}

__device__ __forceinline__ float e2m1_to_f32(uint32_t v) {
    // fp4 e2m1: sign 1, exponent 2 (bias 1), mantissa 1 -> same trick, 2^-14.
    uint16_t h = (uint16_t)(((v & 0x8u) << 12) | ((v & 0x7u) << 9));
    return __half2float(__ushort_as_half(h)) * 16384.0f;
}

__device__ __forceinline__ float ue8m0_to_f32(uint32_t s) {
    // 2^(s-127); s = 0 is 2^-127 (an fp32 subnormal), s = 255 is NaN in the format.
    return s == 0 ? __uint_as_float(0x00400000u) : __uint_as_float(s << 23);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// One element of RMSNorm as the reference's kernels compute it: the normalised value is rounded to bf16,
// then multiplied by the (bf16) weight and rounded again.
__device__ __forceinline__ __nv_bfloat16 rms_norm_apply(__nv_bfloat16 x, float inv, __nv_bfloat16 w, bool has_w) {
    const __nv_bfloat16 t = __float2bfloat16_rn(__bfloat162float(x) * inv);
    return has_w ? __float2bfloat16_rn(__bfloat162float(w) * __bfloat162float(t)) : t;
}
__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + __expf(-g)); }

// Saturating fp32 -> fp16 (the activations are carried in fp16 between the
// products; values beyond the fp16 range clamp instead of becoming inf).
__device__ __forceinline__ __half f32_to_f16_sat(float v) {
    v = fminf(fmaxf(v, -65504.0f), 65504.0f);
    return __float2half_rn(v);
}
// The same, counting the values that had to be clamped (word 4 of a workspace's status block, read and cleared
// by imx_moe_saturations): a clamp changes the result and must not pass unnoticed.
constexpr int kStatusSaturations = 4;
__device__ __forceinline__ __half f32_to_f16_sat(float v, int32_t* status) {
    if (status != nullptr && fabsf(v) > 65504.0f) atomicAdd(status + kStatusSaturations, 1);
    return f32_to_f16_sat(v);
}
#endif

}  // namespace imx
