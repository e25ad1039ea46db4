// The reference's quantized-op surface (mlx/src/ops.rs:630-727) as standalone
// kernels: dequantize, quantized_matmul (both transposes), plus quantize and
// the per-row gather form.  These are the generic, any-format versions; the
// MoE block's hot kernels live in decode_tmap.cu / prefill_tc.cu.
#include <cuda_fp8.h>

#include "internal.h"
#include "qformat.cuh"

namespace imx {

int validate_format(int mode, int bits, int group, QFormat* out) {
    if (mode == IMX_MODE_AFFINE) {
        IMX_REQUIRE(bits == 2 || bits == 3 || bits == 4 || bits == 5 || bits == 6 || bits == 8,
                    "affine quantization supports 2/3/4/5/6/8 bits, got %d", bits);
        IMX_REQUIRE(group == 32 || group == 64 || group == 128,
                    "affine quantization supports group sizes 32/64/128, got %d", group);
    } else if (mode == IMX_MODE_MXFP8) {
        IMX_REQUIRE(bits == 8 && group == 32, "mxfp8 requires bits=8, group_size=32 (got %d, %d)", bits, group);
    } else if (mode == IMX_MODE_NVFP4) {
        IMX_REQUIRE(bits == 4 && group == 16, "nvfp4 requires bits=4, group_size=16 (got %d, %d)", bits, group);
    } else {
        IMX_REQUIRE(false, "unknown quantization mode %d", mode);
    }
    out->mode = mode;
    out->bits = bits;
    out->group = group;
    return IMX_OK;
}

namespace {

template <typename T>
__device__ __forceinline__ T cast_out(float v);
template <>
__device__ __forceinline__ float cast_out<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 cast_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half cast_out<__half>(float v) { return __float2half_rn(v); }

template <typename T>
__global__ void dequantize_kernel(QMat m, int rows, int in, QFormat f, T* __restrict__ out) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;   // one thread per 8 values
    const long per_row = in / 8;
    if (i >= (long)rows * per_row) return;
    const long row = i / per_row;
    const int k0 = (int)(i - row * per_row) * 8;
    float v[8];
    dequant8(qrow(m, (size_t)row, in, f), k0, f, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) out[(size_t)row * in + k0 + j] = cast_out<T>(v[j] * m.global_scale);
}

// ── quantize ────────────────────────────────────────────────────────────────
__device__ __forceinline__ uint32_t f32_to_e2m1(float v) {
    // nearest, ties to the even code, saturating at 6
    const uint32_t sign = v < 0.f ? 8u : 0u;
    const float a = fabsf(v);
    uint32_t c;
    if (a <= 0.25f) c = 0;
    else if (a < 0.75f) c = 1;
    else if (a <= 1.25f) c = 2;
    else if (a < 1.75f) c = 3;
    else if (a <= 2.5f) c = 4;
    else if (a < 3.5f) c = 5;
    else if (a <= 5.0f) c = 6;
    else c = 7;
    return sign | c;
}

// One thread per group.
__global__ void quantize_kernel(const float* __restrict__ w, int rows, int in, QFormat f, float gscale,
                                uint8_t* __restrict__ wp, uint8_t* __restrict__ scales,
                                uint8_t* __restrict__ biases) {
    const long gi = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const int gpr = in / f.group;
    if (gi >= (long)rows * gpr) return;
    const long row = gi / gpr;
    const int g = (int)(gi - row * gpr);
    const float* src = w + (size_t)row * in + (size_t)g * f.group;
    uint8_t* dst = wp + (size_t)row * packed_row_bytes(in, f.bits) + (size_t)g * f.group * f.bits / 8;
    float mx = -INFINITY, mn = INFINITY, amax = 0.f;
    for (int i = 0; i < f.group; ++i) {
        const float v = src[i];
        mx = fmaxf(mx, v);
        mn = fminf(mn, v);
        amax = fmaxf(amax, fabsf(v));
    }
    if (f.mode == IMX_MODE_AFFINE) {
        const float n_bins = (float)((1 << f.bits) - 1);
        const bool side = fabsf(mn) > fabsf(mx);
        float scale = fmaxf(__fdiv_rn(__fsub_rn(mx, mn), n_bins), 1e-7f);
        scale = side ? scale : -scale;
        const float edge = side ? mn : mx;
        const float q0 = rintf(__fdiv_rn(edge, scale));
        float bias = 0.f;
        if (q0 != 0.f) {
            scale = __fdiv_rn(edge, q0);
            bias = edge;
        }
        reinterpret_cast<__nv_bfloat16*>(scales)[(size_t)row * gpr + g] = __float2bfloat16_rn(scale);
        reinterpret_cast<__nv_bfloat16*>(biases)[(size_t)row * gpr + g] = __float2bfloat16_rn(bias);
        uint64_t buf = 0;
        int nb = 0;
        uint32_t* out32 = reinterpret_cast<uint32_t*>(dst);
        for (int i = 0; i < f.group; ++i) {
            float q = rintf(__fdiv_rn(__fsub_rn(src[i], bias), scale));
            q = fminf(fmaxf(q, 0.f), n_bins);
            buf |= (uint64_t)(uint32_t)q << nb;
            nb += f.bits;
            if (nb >= 32) {
                *out32++ = (uint32_t)buf;
                buf >>= 32;
                nb -= 32;
            }
        }
    } else if (f.mode == IMX_MODE_MXFP8) {
        // smallest power of two 2^e with amax / 2^e <= 448
        int e = -127;
        if (amax > 0.f) {
            int ex;
            const float mant = frexpf(__fdiv_rn(amax, 448.f), &ex);
            e = (mant == 0.5f) ? ex - 1 : ex;
            e = max(-127, min(127, e));
        }
        scales[(size_t)row * gpr + g] = (uint8_t)(e + 127);
        const float sc = ue8m0_to_f32((uint32_t)(e + 127));
        for (int i = 0; i < f.group; ++i) {
            float v = __fdiv_rn(src[i], sc);
            v = fminf(fmaxf(v, -448.f), 448.f);
            dst[i] = (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
        }
    } else {
        float s = __fdiv_rn(__fdiv_rn(amax, 6.f), gscale);
        s = fminf(fmaxf(s, 0.f), 448.f);
        const uint8_t s8 = (uint8_t)__nv_cvt_float_to_fp8(s, __NV_SATFINITE, __NV_E4M3);
        scales[(size_t)row * gpr + g] = s8;
        float sf = __fmul_rn(e4m3_to_f32(s8), gscale);
        if (sf == 0.f) sf = 1.f;
        for (int i = 0; i < f.group; i += 2) {
            float v0 = fminf(fmaxf(__fdiv_rn(src[i], sf), -6.f), 6.f);
            float v1 = fminf(fmaxf(__fdiv_rn(src[i + 1], sf), -6.f), 6.f);
            dst[i / 2] = (uint8_t)(f32_to_e2m1(v0) | (f32_to_e2m1(v1) << 4));
        }
    }
}

// ── quantized_matmul, transpose = true (and the gather form) ───────────────
// y[j, n] = x[lhs(j), :] . dequant(W[rhs(j)])[n, :]
constexpr int kQThreads = 256;
constexpr int kQRows = 8;          // x rows per CTA
constexpr int kQOut = 64;          // output rows per CTA (8 warps x 8)

__global__ void __launch_bounds__(kQThreads)
qmm_t_kernel(const __nv_bfloat16* __restrict__ x, int m, QMat w, int n_out, int in, QFormat f,
             __nv_bfloat16* __restrict__ y, const int32_t* __restrict__ lhs_index,
             const int32_t* __restrict__ rhs_index, size_t w_stride, size_t s_stride, int rows_per_cta) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* s_x = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [kQRows][in]
    const int j0 = blockIdx.x * rows_per_cta;
    const int nrows = min(rows_per_cta, m - j0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int r = 0; r < kQRows; ++r) {
        const __nv_bfloat16* src = nullptr;
        if (r < nrows) src = x + (size_t)(lhs_index ? lhs_index[j0 + r] : j0 + r) * in;
        for (int c = tid * 8; c < in; c += kQThreads * 8) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (src) v = *reinterpret_cast<const uint4*>(src + c);
            *reinterpret_cast<uint4*>(s_x + (size_t)r * in + c) = v;
        }
    }
    __syncthreads();
    QMat mat = w;
    if (rhs_index != nullptr) {
        const size_t e = (size_t)rhs_index[j0];
        mat.w += e * w_stride;
        mat.scales += e * s_stride;
        if (mat.biases) mat.biases += e * s_stride;
    }
    for (int jr = 0; jr < kQOut / 8; ++jr) {
        const int n = blockIdx.y * kQOut + warp * (kQOut / 8) + jr;
        if (n >= n_out) break;
        const QRow row = qrow(mat, (size_t)n, in, f);
        float acc[kQRows];
#pragma unroll
        for (int r = 0; r < kQRows; ++r) acc[r] = 0.f;
        for (int k0 = lane * 8; k0 < in; k0 += 256) {
            float wv[8];
            dequant8(row, k0, f, wv);
#pragma unroll
            for (int r = 0; r < kQRows; ++r) {
                uint4 xv = *reinterpret_cast<const uint4*>(s_x + (size_t)r * in + k0);
                const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float2 xf = __bfloat1622float2(xb[i]);
                    acc[r] = fmaf(wv[2 * i], xf.x, acc[r]);
                    acc[r] = fmaf(wv[2 * i + 1], xf.y, acc[r]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < kQRows; ++r) acc[r] = warp_sum(acc[r]) * mat.global_scale;
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < kQRows; ++r)
                if (r < nrows) y[(size_t)(j0 + r) * n_out + n] = __float2bfloat16_rn(acc[r]);
        }
    }
}

// ── quantized_matmul, transpose = false: y[m, in] = x[m, n_out] @ dequant(W[n_out, in]) ──
__global__ void __launch_bounds__(kQThreads)
qmm_n_kernel(const __nv_bfloat16* __restrict__ x, int m, QMat w, int n_out, int in, QFormat f,
             __nv_bfloat16* __restrict__ y) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* s_x = reinterpret_cast<float*>(smem_raw);                     // [kQRows][n_out]
    const int j0 = blockIdx.x * kQRows;
    const int nrows = min(kQRows, m - j0);
    const int tid = threadIdx.x;
    for (int i = tid; i < kQRows * n_out; i += kQThreads) {
        const int r = i / n_out, c = i - r * n_out;
        s_x[i] = r < nrows ? __bfloat162float(x[(size_t)(j0 + r) * n_out + c]) : 0.f;
    }
    __syncthreads();
    const int k0 = (blockIdx.y * kQThreads + tid) * 8;
    if (k0 >= in) return;
    float acc[kQRows][8];
#pragma unroll
    for (int r = 0; r < kQRows; ++r)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[r][i] = 0.f;
    for (int n = 0; n < n_out; ++n) {
        float wv[8];
        dequant8(qrow(w, (size_t)n, in, f), k0, f, wv);
#pragma unroll
        for (int r = 0; r < kQRows; ++r) {
            const float xv = s_x[r * n_out + n];
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[r][i] = fmaf(xv, wv[i], acc[r][i]);
        }
    }
    for (int r = 0; r < nrows; ++r)
#pragma unroll
        for (int i = 0; i < 8; ++i)
            y[(size_t)(j0 + r) * in + k0 + i] = __float2bfloat16_rn(acc[r][i] * w.global_scale);
}

}  // namespace

int launch_dequantize(const QMat& w, int rows, int in, QFormat f, int out_dtype, void* out,
                      cudaStream_t stream) {
    IMX_REQUIRE(in % f.group == 0 && in % 8 == 0 && ((long)in * f.bits) % 32 == 0,
                "dequantize: input dimension %d does not fit group size %d / %d bits", in, f.group, f.bits);
    const long n = (long)rows * (in / 8);
    if (n == 0) return IMX_OK;
    const int blocks = (int)((n + 255) / 256);
    if (out_dtype == 0) dequantize_kernel<<<blocks, 256, 0, stream>>>(w, rows, in, f, (__nv_bfloat16*)out);
    else if (out_dtype == 1) dequantize_kernel<<<blocks, 256, 0, stream>>>(w, rows, in, f, (float*)out);
    else if (out_dtype == 2) dequantize_kernel<<<blocks, 256, 0, stream>>>(w, rows, in, f, (__half*)out);
    else IMX_REQUIRE(false, "dequantize: out_dtype must be 0 (bf16), 1 (fp32) or 2 (fp16)");
    IMX_LAUNCHED();
    IMX_CHECK_CUDA(cudaGetLastError());
    return IMX_OK;
}

int launch_quantize(const float* w, int rows, int in, QFormat f, float gscale, void* wp, void* scales,
                    void* biases, cudaStream_t stream) {
    IMX_REQUIRE(in % f.group == 0 && ((long)f.group * f.bits) % 32 == 0,
                "quantize: input dimension %d does not fit group size %d / %d bits", in, f.group, f.bits);
    IMX_REQUIRE(f.mode != IMX_MODE_AFFINE || biases != nullptr, "quantize: affine mode needs a biases output");
    IMX_REQUIRE(f.mode != IMX_MODE_NVFP4 || gscale > 0.f, "quantize: nvfp4 needs a positive tensor scale");
    const long n = (long)rows * (in / f.group);
    if (n == 0) return IMX_OK;
    quantize_kernel<<<(int)((n + 127) / 128), 128, 0, stream>>>(w, rows, in, f, gscale, (uint8_t*)wp,
                                                                (uint8_t*)scales, (uint8_t*)biases); IMX_LAUNCHED();
    IMX_CHECK_CUDA(cudaGetLastError());
    return IMX_OK;
}

int launch_qmm(const void* x, int m, const QMat& w, int n_out, int in, int transpose, QFormat f, void* y,
               const int32_t* lhs_index, const int32_t* rhs_index, size_t w_stride, size_t s_stride,
               cudaStream_t stream) {
    IMX_REQUIRE(in % f.group == 0 && in % 8 == 0 && ((long)in * f.bits) % 32 == 0,
                "quantized_matmul: input dimension %d does not fit group size %d / %d bits", in, f.group, f.bits);
    if (m == 0 || n_out == 0) return IMX_OK;
    if (transpose) {
        const int rows_per_cta = rhs_index ? 1 : kQRows;
        const size_t smem = (size_t)kQRows * in * sizeof(__nv_bfloat16);
        IMX_REQUIRE(smem <= 200 * 1024, "quantized_matmul: input dimension %d too large", in);
        IMX_CHECK_CUDA(cudaFuncSetAttribute(qmm_t_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        dim3 grid(ceil_div(m, rows_per_cta), ceil_div(n_out, kQOut));
        qmm_t_kernel<<<grid, kQThreads, smem, stream>>>((const __nv_bfloat16*)x, m, w, n_out, in, f,
                                                        (__nv_bfloat16*)y, lhs_index, rhs_index, w_stride,
                                                        s_stride, rows_per_cta); IMX_LAUNCHED();
    } else {
        IMX_REQUIRE(lhs_index == nullptr && rhs_index == nullptr, "gather form requires transpose");
        const size_t smem = (size_t)kQRows * n_out * sizeof(float);
        IMX_REQUIRE(smem <= 200 * 1024, "quantized_matmul: output dimension %d too large", n_out);
        IMX_CHECK_CUDA(cudaFuncSetAttribute(qmm_n_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        dim3 grid(ceil_div(m, kQRows), ceil_div(in, kQThreads * 8));
        qmm_n_kernel<<<grid, kQThreads, smem, stream>>>((const __nv_bfloat16*)x, m, w, n_out, in, f,
                                                        (__nv_bfloat16*)y); IMX_LAUNCHED();
    }
    IMX_CHECK_CUDA(cudaGetLastError());
    return IMX_OK;
}

}  // namespace imx
