// Format-agnostic grouped expert products: a warp-per-output-row dequant-GEMV
// with shuffle reductions.  Handles every MLX format (affine 2/3/4/5/6/8 bit,
// mxfp8, nvfp4) and any shape; it is the path for formats/shapes the
// tensor-core kernels do not cover and the cross-check for those that they do.
//
//   first product  act[slot, i] = silu(gate_e[i,:] . a) * (up_e[i,:] . a)
//   second product out[slot, h] = row_scale[slot] * (down_e[h,:] . act[slot,:])
// (mlx/src/nn/moe.rs:26-32; each dot product is one row of the reference's
// `quantized_matmul(transpose=true)`, mlx/src/nn/linear.rs:51-63.)
#include "internal.h"
#include "qformat.cuh"

namespace imx {

namespace {

constexpr int kGThreads = 256;
constexpr int kGWarps = kGThreads / 32;
constexpr int kGRowsPerWarp = 8;
constexpr int kGRowsPerCta = kGWarps * kGRowsPerWarp;   // 64 output rows per CTA
constexpr int UR = kUnitRows;

struct Resolved {
    QMat a, b;        // SWIGLU: gate, up; else: down, unused
    int K;            // reduction length
    int n_out;        // output rows
};

template <bool SWIGLU>
__device__ __forceinline__ Resolved resolve(const ExpertSet& s, int e) {
    Resolved r;
    const bool extra = (e >= s.num_experts);
    if (SWIGLU) {
        if (extra) {
            r.a = s.x_gate;
            r.b = s.x_up;
        } else {
            r.a = s.gate;
            r.b = s.up;
            r.a.w += (size_t)e * s.gu_stride_w;
            r.b.w += (size_t)e * s.gu_stride_w;
            r.a.scales += (size_t)e * s.gu_stride_s;
            r.b.scales += (size_t)e * s.gu_stride_s;
            if (r.a.biases) {
                r.a.biases += (size_t)e * s.gu_stride_s;
                r.b.biases += (size_t)e * s.gu_stride_s;
            }
        }
        r.K = s.n_in;
        r.n_out = extra ? s.x_mid : s.n_mid;
    } else {
        if (extra) {
            r.a = s.x_down;
        } else {
            r.a = s.down;
            r.a.w += (size_t)e * s.dn_stride_w;
            r.a.scales += (size_t)e * s.dn_stride_s;
            if (r.a.biases) r.a.biases += (size_t)e * s.dn_stride_s;
        }
        r.b = r.a;
        r.K = extra ? s.x_mid : s.n_mid;
        r.n_out = s.n_in;
    }
    return r;
}

template <bool SWIGLU>
__global__ void __launch_bounds__(kGThreads) generic_grouped_kernel(GroupedArgs a, int rb_count) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half* s_in = reinterpret_cast<__half*>(smem_raw);      // [UR][K]

    const int unit_id = blockIdx.x / rb_count;
    const int rb = blockIdx.x % rb_count;
    if (unit_id >= *a.n_units) return;
    const WorkUnit u = a.units[unit_id];
    const Resolved R = resolve<SWIGLU>(a.set, u.expert);
    const QFormat f = a.set.fmt;
    if (rb * kGRowsPerCta >= R.n_out) return;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = R.K;
    // stage the unit's input rows
    for (int r = 0; r < UR; ++r) {
        const __half* src = nullptr;
        if (r < u.rows) {
            if (SWIGLU) {
                const int slot = u.slot0 + r;
                const int row = a.row_index ? a.row_index[slot] : slot;
                src = a.in + (size_t)row * a.set.n_in;
            } else {
                src = a.act + (size_t)(u.slot0 + r) * a.act_stride;
            }
        }
        for (int c = tid * 8; c < K; c += kGThreads * 8) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (src) v = *reinterpret_cast<const uint4*>(src + c);
            *reinterpret_cast<uint4*>(s_in + (size_t)r * K + c) = v;
        }
    }
    __syncthreads();

    for (int j = 0; j < kGRowsPerWarp; ++j) {
        const int row = rb * kGRowsPerCta + warp * kGRowsPerWarp + j;
        if (row >= R.n_out) break;
        const QRow ra = qrow(R.a, row, K, f);
        const QRow rb2 = qrow(R.b, row, K, f);
        float acc_a[UR], acc_b[UR];
#pragma unroll
        for (int r = 0; r < UR; ++r) acc_a[r] = acc_b[r] = 0.f;
        for (int k0 = lane * 8; k0 < K; k0 += 256) {
            float wa[8], wb[8];
            dequant8(ra, k0, f, wa);
            if (SWIGLU) dequant8(rb2, k0, f, wb);
#pragma unroll
            for (int r = 0; r < UR; ++r) {
                uint4 xv = *reinterpret_cast<const uint4*>(s_in + (size_t)r * K + k0);
                const __half2* xh = reinterpret_cast<const __half2*>(&xv);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float2 xf = __half22float2(xh[i]);
                    acc_a[r] = fmaf(wa[2 * i], xf.x, acc_a[r]);
                    acc_a[r] = fmaf(wa[2 * i + 1], xf.y, acc_a[r]);
                    if (SWIGLU) {
                        acc_b[r] = fmaf(wb[2 * i], xf.x, acc_b[r]);
                        acc_b[r] = fmaf(wb[2 * i + 1], xf.y, acc_b[r]);
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < UR; ++r) {
            acc_a[r] = warp_sum(acc_a[r]) * R.a.global_scale;
            if (SWIGLU) acc_b[r] = warp_sum(acc_b[r]) * R.b.global_scale;
        }
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < UR; ++r) {
                if (r >= u.rows) break;
                const int slot = u.slot0 + r;
                if (SWIGLU) {
                    a.act[(size_t)slot * a.act_stride + row] = f32_to_f16_sat(silu_f(acc_a[r]) * acc_b[r], a.status);
                } else {
                    const float sc = a.row_scale ? a.row_scale[slot] : 1.f;
                    a.out[(size_t)slot * a.set.n_in + row] = acc_a[r] * sc;
                }
            }
        }
    }
}

}  // namespace

int launch_generic_grouped(const GroupedArgs& a, cudaStream_t stream, cudaEvent_t mid) {
    const ExpertSet& s = a.set;
    IMX_REQUIRE(s.n_in % 8 == 0 && s.n_mid % 8 == 0 && (!s.has_extra || s.x_mid % 8 == 0),
                "experts: hidden/intermediate sizes must be multiples of 8");
    const int mid_max = s.has_extra && s.x_mid > s.n_mid ? s.x_mid : s.n_mid;
    if (a.max_units == 0) return IMX_OK;
    {
        const int rb = ceil_div(mid_max, kGRowsPerCta);
        const size_t smem = (size_t)UR * s.n_in * sizeof(__half);
        IMX_REQUIRE(smem <= 200 * 1024, "experts: hidden size %d too large for the generic path", s.n_in);
        IMX_CHECK_CUDA(cudaFuncSetAttribute(generic_grouped_kernel<true>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        generic_grouped_kernel<true><<<a.max_units * rb, kGThreads, smem, stream>>>(a, rb); IMX_LAUNCHED();
        IMX_CHECK_CUDA(cudaGetLastError());
        if (mid) IMX_CHECK_CUDA(cudaEventRecord(mid, stream));
    }
    {
        const int rb = ceil_div(s.n_in, kGRowsPerCta);
        const size_t smem = (size_t)UR * mid_max * sizeof(__half);
        IMX_REQUIRE(smem <= 200 * 1024, "experts: intermediate size %d too large for the generic path", mid_max);
        IMX_CHECK_CUDA(cudaFuncSetAttribute(generic_grouped_kernel<false>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        generic_grouped_kernel<false><<<a.max_units * rb, kGThreads, smem, stream>>>(a, rb); IMX_LAUNCHED();
        IMX_CHECK_CUDA(cudaGetLastError());
    }
    return IMX_OK;
}

}  // namespace imx
