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

// V consecutive values of a row of expert output: 4 of an fp32 row or 8 of an fp16 row (16 bytes either way)
template <bool F16>
__device__ __forceinline__ void load_row(const void* rows, size_t idx, float* v) {
    if (F16) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(rows) + idx));
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
            v[2 * e] = f.x;
            v[2 * e + 1] = f.y;
        }
    } else {
        const float4 q = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(rows) + idx));
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    }
}

template <bool F32_OUT, bool F16_ROWS>
__global__ void __launch_bounds__(kCThreads)
combine_kernel(const void* __restrict__ rows, const float* __restrict__ row_scale,
               const int32_t* __restrict__ inv_perm, int k, int H, const void* __restrict__ shared_rows,
               void* __restrict__ y_out, const __nv_bfloat16* __restrict__ residual,
               const float* __restrict__ shared_scale) {
    constexpr int V = F16_ROWS ? 8 : 4;          // columns per thread
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
    const int c = (blockIdx.y * kCThreads + tid) * V;
    if (c >= H) return;
    float acc[V];
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = 0.f;
    // Eight independent 16-byte row loads in flight per thread, kept as they arrive (four registers each) and
    // unpacked when they are added, in slot order.
    constexpr int kBatch = 8;
    for (int s0 = 0; s0 < k; s0 += kBatch) {
        uint4 raw[kBatch];
        float w[kBatch];
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
            const int slot = (s0 + j < k) ? s_slot[s0 + j] : -1;
            raw[j] = make_uint4(0u, 0u, 0u, 0u);      // dropped assignment (moe.rs:100) or past the last slot: zeros
            if (slot >= 0) {
                const size_t idx = (size_t)slot * H + c;
                raw[j] = F16_ROWS ? __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(rows) + idx))
                                  : __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(rows) + idx));
            }
            w[j] = (slot >= 0 && row_scale != nullptr) ? __ldg(row_scale + slot) : 1.f;
        }
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
            float v[V];
            if (F16_ROWS) {
                const uint32_t q[4] = {raw[j].x, raw[j].y, raw[j].z, raw[j].w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&q[e]));
                    v[2 * e] = f.x;
                    v[2 * e + 1] = f.y;
                }
            } else {
                v[0] = __uint_as_float(raw[j].x); v[1] = __uint_as_float(raw[j].y);
                v[2] = __uint_as_float(raw[j].z); v[3] = __uint_as_float(raw[j].w);
            }
            if (row_scale != nullptr) {               // rows arrive unweighted: scale (one rounding), then add
#pragma unroll
                for (int i = 0; i < V; ++i) acc[i] += v[i] * w[j];
            } else {
#pragma unroll
                for (int i = 0; i < V; ++i) acc[i] += v[i];
            }
        }
    }
    if (shared_rows != nullptr) {
        float v[V];
        load_row<F16_ROWS>(shared_rows, (size_t)t * H + c, v);
        const float sw = shared_scale != nullptr ? __ldg(shared_scale + t) : 1.f;   // the shared-expert gate, when the row is ungated
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] += v[i] * sw;
    }
    if (residual != nullptr) {       // the layer's residual stream (qwen35.rs:276), added before the one rounding
#pragma unroll
        for (int i = 0; i < V; i += 2) {
            const float2 r = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(residual + (size_t)t * H + c + i));
            acc[i] += r.x;
            acc[i + 1] += r.y;
        }
    }
    if (F32_OUT) {           // partial sums of expert parallelism: summed across ranks before the rounding
        float* yf = reinterpret_cast<float*>(y_out) + (size_t)t * H + c;
#pragma unroll
        for (int i = 0; i < V; i += 4) *reinterpret_cast<float4*>(yf + i) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
        return;
    }
    __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(y_out) + (size_t)t * H + c;
#pragma unroll
    for (int i = 0; i < V; i += 4) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(acc[i], acc[i + 1]);
        __nv_bfloat162 hi = __floats2bfloat162_rn(acc[i + 2], acc[i + 3]);
        uint2 o;
        o.x = *reinterpret_cast<uint32_t*>(&lo);
        o.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(y + i) = o;
    }
}

// dst[j, :] = src[index[j], :] for rows of `row_bytes` bytes (a multiple of 4)
__global__ void gather_rows_kernel(const uint32_t* __restrict__ src, const int32_t* __restrict__ index, int words,
                                   uint32_t* __restrict__ dst) {
    const int j = blockIdx.x;
    const uint32_t* s = src + (size_t)index[j] * words;
    uint32_t* d = dst + (size_t)j * words;
    for (int i = threadIdx.x; i < words; i += blockDim.x) d[i] = __ldg(s + i);
}

// The same for rows that are multiples of 16 bytes: a warp per row at a time, eight 16-byte pieces per lane
// in flight before the first is stored (one small CTA per row spends its time being launched).
constexpr int kGatherWarps = 8;
__global__ void __launch_bounds__(kGatherWarps * 32)
gather_rows16_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ index, int n_rows, int pieces,
                     uint4* __restrict__ dst, const int32_t* __restrict__ skip_from_dev, int skip_to) {
    const int lane = threadIdx.x & 31;
    const int stride = gridDim.x * kGatherWarps;
    const int skip_from = skip_from_dev != nullptr ? __ldg(skip_from_dev) : n_rows;   // rows [skip_from, skip_to) are nobody's
    for (int j = blockIdx.x * kGatherWarps + (threadIdx.x >> 5); j < n_rows; j += stride) {
        if (j >= skip_from && j < skip_to) continue;
        const uint4* s = src + (size_t)__ldg(index + j) * pieces;
        uint4* d = dst + (size_t)j * pieces;
        for (int i0 = lane; i0 < pieces; i0 += 32 * 8) {
            uint4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (i0 + u * 32 < pieces) v[u] = __ldg(s + i0 + u * 32);
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (i0 + u * 32 < pieces) d[i0 + u * 32] = v[u];
        }
    }
}

}  // namespace

int launch_gather_rows(const void* src, const int32_t* index, int n_rows, size_t row_bytes, void* dst,
                       cudaStream_t stream, const int32_t* skip_from_dev, int skip_to) {
    IMX_REQUIRE(row_bytes % 4 == 0 && row_bytes > 0, "gather_rows: row size (%zu) must be a positive multiple of 4", row_bytes);
    IMX_REQUIRE(row_bytes % 16 != 0 || (((uintptr_t)src | (uintptr_t)dst) % 16) == 0,
                "gather_rows: 16-byte rows need 16-byte aligned buffers");
    if (n_rows == 0) return IMX_OK;
    const int words = (int)(row_bytes / 4);
    if (row_bytes % 16 == 0) {
        int grid = ceil_div(n_rows, kGatherWarps);
        if (grid > 148 * 8) grid = 148 * 8;
        gather_rows16_kernel<<<grid, kGatherWarps * 32, 0, stream>>>((const uint4*)src, index, n_rows, (int)(row_bytes / 16),
                                                                    (uint4*)dst, skip_from_dev, skip_to); IMX_LAUNCHED();
        IMX_CHECK_CUDA(cudaGetLastError());
        return IMX_OK;
    }
    IMX_REQUIRE(skip_from_dev == nullptr, "gather_rows: a skipped range needs rows that are multiples of 16 bytes");
    const int threads = words >= 1024 ? 256 : (words >= 128 ? 128 : 32);
    gather_rows_kernel<<<n_rows, threads, 0, stream>>>((const uint32_t*)src, index, words, (uint32_t*)dst); IMX_LAUNCHED();
    IMX_CHECK_CUDA(cudaGetLastError());
    return IMX_OK;
}

int launch_combine(const void* rows, const float* row_scale, const int32_t* inv_perm, int n, int k, int H,
                   const void* shared_rows, void* y, cudaStream_t stream, bool f32_out, const void* residual,
                   bool rows_f16, const float* shared_scale) {
    IMX_REQUIRE(k >= 1 && k <= kMaxK, "combine: top_k (%d) must be in 1..%d", k, kMaxK);
    IMX_REQUIRE(H % 4 == 0 && (!rows_f16 || H % 8 == 0), "combine: hidden (%d) must be a multiple of 4 (8 for fp16 rows)", H);
    if (n == 0) return IMX_OK;
    dim3 grid(n, ceil_div(H, kCCols * (rows_f16 ? 2 : 1)));
    const __nv_bfloat16* res = (const __nv_bfloat16*)residual;
    if (rows_f16 && f32_out) combine_kernel<true, true><<<grid, kCThreads, 0, stream>>>(rows, row_scale, inv_perm, k, H, shared_rows, y, res, shared_scale);
    else if (rows_f16) combine_kernel<false, true><<<grid, kCThreads, 0, stream>>>(rows, row_scale, inv_perm, k, H, shared_rows, y, res, shared_scale);
    else if (f32_out) combine_kernel<true, false><<<grid, kCThreads, 0, stream>>>(rows, row_scale, inv_perm, k, H, shared_rows, y, res, shared_scale);
    else combine_kernel<false, false><<<grid, kCThreads, 0, stream>>>(rows, row_scale, inv_perm, k, H, shared_rows, y, res, shared_scale); IMX_LAUNCHED();
    IMX_CHECK_CUDA(cudaGetLastError());
    return IMX_OK;
}

}  // namespace imx
