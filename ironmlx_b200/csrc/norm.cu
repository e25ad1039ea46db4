// RMSNorm (mlx/src/nn/norm.rs:21-24 -> fast::rms_norm, mlx/src/fast.rs:37-49):
//   inv = rsqrt(mean(x^2) + eps)                 fp32
//   y   = w * T(x * inv)                          the normalised value is rounded to the
//                                                 array type T (bf16) before the weight
//                                                 multiplies it, and the product is
//                                                 rounded again
// One warp per row.  Also serves the decoder-layer tail: with `inv_out` the
// per-row factor is left for the router, which normalises its tiles as it
// loads them (y may then be null).
#include "internal.h"

namespace imx {

namespace {

__global__ void __launch_bounds__(256)
rms_norm_kernel(const __nv_bfloat16* __restrict__ x, int n, int H, const __nv_bfloat16* __restrict__ w, float eps,
                __nv_bfloat16* __restrict__ y, float* __restrict__ inv_out) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= n) return;
    const __nv_bfloat16* xr = x + (size_t)row * H;
    float ss = 0.f;
    for (int c = lane * 8; c < H; c += 256) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(xr + c));
        const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(b[i]);
            ss = fmaf(f.x, f.x, ss);
            ss = fmaf(f.y, f.y, ss);
        }
    }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)H + eps);
    if (inv_out != nullptr && lane == 0) inv_out[row] = inv;
    if (y == nullptr) return;
    __nv_bfloat16* yr = y + (size_t)row * H;
    for (int c = lane * 8; c < H; c += 256) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(xr + c));
        uint4 wv = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);        // ones
        if (w != nullptr) wv = __ldg(reinterpret_cast<const uint4*>(w + c));
        const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(&v);
        const __nv_bfloat16* wb = reinterpret_cast<const __nv_bfloat16*>(&wv);
        __nv_bfloat16 o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rms_norm_apply(xb[i], inv, wb[i], w != nullptr);
        *reinterpret_cast<uint4*>(yr + c) = *reinterpret_cast<const uint4*>(o);
    }
}

}  // namespace

int launch_rms_norm(const void* x, int n, int H, const void* w, float eps, void* y, float* inv_out, cudaStream_t stream) {
    IMX_REQUIRE(n >= 0 && H > 0 && H % 8 == 0, "rms_norm: the row length (%d) must be a positive multiple of 8", H);
    IMX_REQUIRE(x != nullptr && (y != nullptr || inv_out != nullptr), "rms_norm: x and an output are required");
    IMX_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)y % 16) == 0 && ((uintptr_t)w % 16) == 0,
                "rms_norm: arrays must be 16-byte aligned");
    if (n == 0) return IMX_OK;
    rms_norm_kernel<<<ceil_div(n, 8), 256, 0, stream>>>((const __nv_bfloat16*)x, n, H, (const __nv_bfloat16*)w, eps,
                                                        (__nv_bfloat16*)y, inv_out); IMX_LAUNCHED();
    IMX_CHECK_CUDA(cudaGetLastError());
    return IMX_OK;
}

}  // namespace imx
