// Combine stage (mlx/src/nn/moe.rs:147-181): per token, the fp32 sum of its k
// weighted expert rows plus the gated shared-expert row, rounded once to bf16.
//
// The reference appends a token's rows while looping over experts in
// ascending order (moe.rs:117-144) and sums them in that order
// (moe.rs:154-163); the sorted slot index grows with the expert id, so the
// kernel sorts the token's k slots and adds in ascending slot order, which
// also makes the result independent of launch geometry.
#include "internal.h"

namespace imx {

namespace {

constexpr int kCThreads = 128;
constexpr int kCCols = kCThreads * 4;      // columns per CTA
constexpr int kMaxK = 64;

template <bool F32_OUT>
__global__ void __launch_bounds__(kCThreads)
combine_kernel(const float* __restrict__ rows, const float* __restrict__ row_scale,
               const int32_t* __restrict__ inv_perm, int k, int H, const float* __restrict__ shared_rows,
               void* __restrict__ y_out, const __nv_bfloat16* __restrict__ residual) {
    __shared__ int s_raw[kMaxK];
    __shared__ int s_slot[kMaxK];
    const int t = blockIdx.x;
    const int tid = threadIdx.x;
    // the token's k slots in ascending order: one load per thread, then a rank sort (k is tiny)
    if (tid < k) s_raw[tid] = inv_perm[(size_t)t * k + tid];
    __syncthreads();
    if (tid < k) {
        const int v = s_raw[tid];
        int rank = 0;
        for (int j = 0; j < k; ++j) {
            const int o = s_raw[j];
            rank += (o < v) || (o == v && j < tid);
        }
        s_slot[rank] = v;
    }
    __syncthreads();
    const int c = blockIdx.y * kCCols + tid * 4;
    if (c >= H) return;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < k; s0 += 8) {          // eight independent row loads in flight, added in order
        float4 v[8];
        float w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int slot = (s0 + j < k) ? s_slot[s0 + j] : -1;
            v[j] = slot >= 0 ? __ldg(reinterpret_cast<const float4*>(rows + (size_t)slot * H + c))
                             : make_float4(0.f, 0.f, 0.f, 0.f);      // dropped assignment (moe.rs:100)
            w[j] = (slot >= 0 && row_scale != nullptr) ? __ldg(row_scale + slot) : 1.f;
        }
        if (row_scale != nullptr) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {      // rows arrive unweighted: scale (one rounding), then add
                acc.x += v[j].x * w[j]; acc.y += v[j].y * w[j]; acc.z += v[j].z * w[j]; acc.w += v[j].w * w[j];
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                acc.x += v[j].x; acc.y += v[j].y; acc.z += v[j].z; acc.w += v[j].w;
            }
        }
    }
    if (shared_rows != nullptr) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(shared_rows + (size_t)t * H + c));
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (residual != nullptr) {       // the layer's residual stream (qwen35.rs:276), added before the one rounding
        const uint2 rv = __ldg(reinterpret_cast<const uint2*>(residual + (size_t)t * H + c));
        const float2 r0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&rv.x));
        const float2 r1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&rv.y));
        acc.x += r0.x; acc.y += r0.y; acc.z += r1.x; acc.w += r1.y;
    }
    if (F32_OUT) {           // partial sums of expert parallelism: summed across ranks before the rounding
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(y_out) + (size_t)t * H + c) = acc;
        return;
    }
    __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(y_out);
    __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y);
    __nv_bfloat162 hi = __floats2bfloat162_rn(acc.z, acc.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&lo);
    o.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(y + (size_t)t * H + c) = o;
}

// dst[j, :] = src[index[j], :] for rows of `row_bytes` bytes (a multiple of 4)
__global__ void gather_rows_kernel(const uint32_t* __restrict__ src, const int32_t* __restrict__ index, int words,
                                   uint32_t* __restrict__ dst) {
    const int j = blockIdx.x;
    const uint32_t* s = src + (size_t)index[j] * words;
    uint32_t* d = dst + (size_t)j * words;
    if ((words & 3) == 0) {
        for (int i = threadIdx.x; i < words / 4; i += blockDim.x)
            reinterpret_cast<uint4*>(d)[i] = __ldg(reinterpret_cast<const uint4*>(s) + i);
    } else {
        for (int i = threadIdx.x; i < words; i += blockDim.x) d[i] = __ldg(s + i);
    }
}

}  // namespace

int launch_gather_rows(const void* src, const int32_t* index, int n_rows, size_t row_bytes, void* dst,
                       cudaStream_t stream) {
    IMX_REQUIRE(row_bytes % 4 == 0 && row_bytes > 0, "gather_rows: row size (%zu) must be a positive multiple of 4", row_bytes);
    IMX_REQUIRE(row_bytes % 16 != 0 || (((uintptr_t)src | (uintptr_t)dst) % 16) == 0,
                "gather_rows: 16-byte rows need 16-byte aligned buffers");
    if (n_rows == 0) return IMX_OK;
    const int words = (int)(row_bytes / 4);
    const int threads = words >= 1024 ? 256 : (words >= 128 ? 128 : 32);
    gather_rows_kernel<<<n_rows, threads, 0, stream>>>((const uint32_t*)src, index, words, (uint32_t*)dst);
    IMX_CHECK_CUDA(cudaGetLastError());
    return IMX_OK;
}

int launch_combine(const float* rows, const float* row_scale, const int32_t* inv_perm, int n, int k, int H,
                   const float* shared_rows, void* y, cudaStream_t stream, bool f32_out, const void* residual) {
    IMX_REQUIRE(k >= 1 && k <= kMaxK, "combine: top_k (%d) must be in 1..%d", k, kMaxK);
    IMX_REQUIRE(H % 4 == 0, "combine: hidden (%d) must be a multiple of 4", H);
    if (n == 0) return IMX_OK;
    dim3 grid(n, ceil_div(H, kCCols));
    const __nv_bfloat16* res = (const __nv_bfloat16*)residual;
    if (f32_out) combine_kernel<true><<<grid, kCThreads, 0, stream>>>(rows, row_scale, inv_perm, k, H, shared_rows, y, res);
    else combine_kernel<false><<<grid, kCThreads, 0, stream>>>(rows, row_scale, inv_perm, k, H, shared_rows, y, res);
    IMX_CHECK_CUDA(cudaGetLastError());
    return IMX_OK;
}

}  // namespace imx
