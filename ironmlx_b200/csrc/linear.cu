// The layer calls of the path as single entry points over the expert kernels:
//
//   imx_quantized_matmul_ws  `QuantizedLinear::forward_with_stream`
//                            (mlx/src/nn/linear.rs:51-63): y = x . dequantize(W)^T.
//                            The second expert product IS this contraction (rows of
//                            fp16 activations against one quantized matrix), so the
//                            call runs that kernel alone as a one-expert problem:
//                            the tensor-map decode kernel for few rows, the tcgen05
//                            kernel from 32 rows up; shapes neither takes fall back
//                            to the scalar kernel of imx_quantized_matmul.
//   imx_expert_forward       `Expert::forward_with_stream` / `MLP::forward_with_stream`
//                            (mlx/src/nn/moe.rs:26-32, mlx/src/nn/mlp.rs:27-33):
//                            down(silu(gate(x)) * up(x)) for one expert over all rows.
//   imx_linear               `Linear::forward_with_stream` (mlx/src/nn/linear.rs:170-177):
//                            dense bf16 x . W^T (+ b) on mma.sync, fp32 accumulation.
//
// All take bf16 activations in and out, as the reference's layers do; scratch comes
// from the caller.
#include "internal.h"

namespace imx {

namespace {

// Everything a one-expert launch needs, in one kernel.  Blocks 0 .. m-1: the fp16 copy of a bf16 row in the
// 16-value block order the expert kernels of a format read (pairs 1 and 3 of every 8 stored values multiplied
// by pair_scale_odd, the tensor-map decode kernel's convention).  Block m: the identity slot order, the work
// units of the single expert (balanced, at most unit_rows slots each) and cleared scheduler words.
__global__ void __launch_bounds__(256)
prepare_one_kernel(const __nv_bfloat16* __restrict__ src, int m, int cols, __half* __restrict__ dst, const Order16 order,
                   int unit_rows, int32_t* __restrict__ offsets, int32_t* __restrict__ ident, WorkUnit* __restrict__ units,
                   int32_t* __restrict__ n_units, int32_t* __restrict__ sched, int sched_ints, float* __restrict__ psum) {
    if ((int)blockIdx.x < m) {
        const size_t r = blockIdx.x;
        const __nv_bfloat16* s = src + r * cols;
        for (int i = threadIdx.x; i < cols; i += blockDim.x) {
            const float v = __bfloat162float(s[(i & ~15) + order.o[i & 15]]);
            dst[r * cols + i] = __float2half_rn((i & 2) ? v * order.pair_scale_odd : v);
        }
        if (psum != nullptr) {
            // sums of every 16 values of the row as the expert kernels will read them (the tensor-map decode
            // kernel's second product takes its group sums from these)
            __syncthreads();
            const float unscale = 1.f / order.pair_scale_odd;
            for (int b = threadIdx.x; b < cols / 16; b += blockDim.x) {
                float acc = 0.f;
                for (int i = 0; i < 16; ++i) {
                    const float v = __half2float(dst[r * cols + b * 16 + i]);
                    acc += (i & 2) ? v * unscale : v;
                }
                psum[r * (cols / 16) + b] = acc;
            }
        }
        return;
    }
    const int tid = threadIdx.x;
    const int nu = (m + unit_rows - 1) / unit_rows;
    int per = (m + nu - 1) / nu;                       // equal shares, rounded up to whole blocks of 16 slots
    per = (per + 15) & ~15;
    if (per > unit_rows) per = unit_rows;
    for (int i = tid; i < m; i += blockDim.x) ident[i] = i;
    for (int c = tid; c < nu; c += blockDim.x) {
        WorkUnit u;
        u.expert = 0;
        u.slot0 = c * per;
        u.rows = min(per, m - c * per);
        u.pad = 0;
        units[c] = u;
    }
    for (int i = tid; i < sched_ints; i += blockDim.x) sched[i] = 0;
    if (tid == 0) {
        offsets[0] = 0;
        offsets[1] = m;
        n_units[0] = n_units[1] = nu;
    }
}

struct OneWs {
    int32_t* status;
    SchedWs sw;
    int32_t* n_units;
    float* partials;
    int32_t* offsets;     // [2]
    int32_t* ident;       // [m]
    WorkUnit* units;
    __half* x16;          // [m, in]
    __half* act;          // [m, mid]      (expert forward)
    float* psum;          // [m, K / 16 + 1]
    float* gsum_x;        // [m, in / 64 + 1]
    float* rows;          // [m, out] fp32 (or fp16 in the same buffer)
    int max_units;
    size_t bytes;
};

OneWs carve_one(int m, int in, int mid, int out, void* base) {
    OneWs w = {};
    Carver cv(base);
    w.status = cv.take<int32_t>(16);
    w.max_units = max_units_for(m, 1, 0);
    // as the second product alone the matrix is [out, in]: reduction over `in`, `out` output rows
    w.sw = mid > 0 ? carve_sched(cv, in, mid, 0) : carve_sched(cv, out, in, 0);
    w.n_units = cv.take<int32_t>(4);
    w.partials = cv.take<float>((size_t)kFlagWarps * 256);
    w.offsets = cv.take<int32_t>(4);
    w.ident = cv.take<int32_t>(m);
    w.units = cv.take<WorkUnit>(w.max_units);
    w.x16 = cv.take<__half>((size_t)m * in);
    if (mid > 0) w.act = cv.take<__half>((size_t)m * mid);
    const int kmax = mid > in ? mid : in;
    w.psum = cv.take<float>((size_t)m * (kmax / 16 + 1));
    w.gsum_x = cv.take<float>((size_t)m * (in / 64 + 1));
    w.rows = cv.take<float>((size_t)m * out);
    w.bytes = align_up(cv.off, 256);
    return w;
}

int check_scratch(void* scratch, size_t have, size_t need, const char* who) {
    if (scratch == nullptr || ((uintptr_t)scratch % 256) != 0 || have < need) {
        set_error("%s: 256-byte aligned scratch of %zu bytes needed, %zu given", who, need, have);
        return IMX_ERR_WORKSPACE;
    }
    return IMX_OK;
}

// The quantized matrix [n_out, in] as the "down" matrix of a one-expert set: hidden := n_out, intermediate := in.
int qmm_set(const imx_qtensor& w, int n_out, int in, const QFormat& f, ExpertSet* out) {
    imx_moe_config c = {};
    c.hidden = n_out;
    c.intermediate = in;
    ExpertSet s = {};
    s.fmt = f;
    s.num_experts = 1;
    s.n_in = n_out;
    s.n_mid = in;
    QMat m;
    m.w = (const uint8_t*)w.w;
    m.scales = (const uint8_t*)w.scales;
    m.biases = (const uint8_t*)w.biases;
    m.global_scale = w.global_scale == 0.f ? 1.f : w.global_scale;
    s.gate = s.up = s.down = m;        // only `down` is read
    s.dn_stride_w = (size_t)n_out * packed_row_bytes(in, f.bits);
    s.dn_stride_s = (size_t)n_out * scale_row_bytes(in, f);
    *out = s;
    return IMX_OK;
}

// Which kernel runs a [m, in] x [n_out, in]^T product alone; IMX_PATH_GENERIC = none of the expert kernels.
int qmm_path(const ExpertSet& s, int m) {
    if (m >= 32 && prefill_tc_supported(s, true)) return IMX_PATH_PREFILL;
    if (m <= 256 && (decode_tmap_supported(s) || decode_mma_supported(s) || decode_fp_supported(s))) return IMX_PATH_DECODE;
    if (prefill_tc_supported(s, true)) return IMX_PATH_PREFILL;
    return IMX_PATH_GENERIC;
}

// ── dense x . W^T (+ b) ──────────────────────────────────────────────────────
constexpr int kLT = 64, kLK = 32, kLPad = 8;
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 64 x 64 output tile per CTA of four warps (a 32 x 32 quarter each), K in steps of 32 through shared memory.
__global__ void __launch_bounds__(128)
linear_kernel(const __nv_bfloat16* __restrict__ x, int m, int k, const __nv_bfloat16* __restrict__ w, int n,
              const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ y) {
    __shared__ __align__(16) __nv_bfloat16 sa[kLT][kLK + kLPad];
    __shared__ __align__(16) __nv_bfloat16 sb[kLT][kLK + kLPad];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int m0 = blockIdx.y * kLT, n0 = blockIdx.x * kLT;
    const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;
    for (int k0 = 0; k0 < k; k0 += kLK) {
        // 64 rows x 32 values of each operand: 256 pieces of 8 values, two per thread
#pragma unroll
        for (int p = 0; p < 2; ++p) {
            const int piece = tid + p * 128, r = piece >> 2, c = (piece & 3) * 8;
            uint4 va = make_uint4(0, 0, 0, 0), vb = make_uint4(0, 0, 0, 0);
            if (k0 + c < k) {
                if (m0 + r < m) va = *reinterpret_cast<const uint4*>(x + (size_t)(m0 + r) * k + k0 + c);
                if (n0 + r < n) vb = *reinterpret_cast<const uint4*>(w + (size_t)(n0 + r) * k + k0 + c);
            }
            *reinterpret_cast<uint4*>(&sa[r][c]) = va;
            *reinterpret_cast<uint4*>(&sb[r][c]) = vb;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kLK; kk += 16) {
            uint32_t a[2][4], b[4][2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int r = wm + i * 16 + g;
                a[i][0] = *reinterpret_cast<const uint32_t*>(&sa[r][kk + 2 * t]);
                a[i][1] = *reinterpret_cast<const uint32_t*>(&sa[r + 8][kk + 2 * t]);
                a[i][2] = *reinterpret_cast<const uint32_t*>(&sa[r][kk + 8 + 2 * t]);
                a[i][3] = *reinterpret_cast<const uint32_t*>(&sa[r + 8][kk + 8 + 2 * t]);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = wn + j * 8 + g;
                b[j][0] = *reinterpret_cast<const uint32_t*>(&sb[c][kk + 2 * t]);
                b[j][1] = *reinterpret_cast<const uint32_t*>(&sb[c][kk + 8 + 2 * t]);
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) mma_bf16(acc[i][j], a[i][0], a[i][1], a[i][2], a[i][3], b[j][0], b[j][1]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int r = m0 + wm + i * 16 + g + 8 * h;
                const int c = n0 + wn + j * 8 + 2 * t;
                if (r < m) {
#pragma unroll
                    for (int e = 0; e < 2; ++e)
                        if (c + e < n) {
                            float v = acc[i][j][2 * h + e];
                            if (bias != nullptr) v += __bfloat162float(bias[c + e]);
                            y[(size_t)r * n + c + e] = __float2bfloat16_rn(v);
                        }
                }
            }
}

}  // namespace

}  // namespace imx

using namespace imx;

extern "C" {

int imx_quantized_matmul_scratch_bytes(int m, int n_out, int in, int group_size, int bits, int mode, size_t* bytes) {
    QFormat f;
    IMX_TRY(validate_format(mode, bits, group_size, &f));
    IMX_REQUIRE(bytes != nullptr && m >= 0 && n_out > 0 && in > 0, "quantized_matmul_scratch_bytes: bad arguments");
    *bytes = carve_one(m, in, 0, n_out, nullptr).bytes;
    return IMX_OK;
}

int imx_quantized_matmul_ws(const void* x, int m, const imx_qtensor* w, int n_out, int in, int group_size, int bits,
                            int mode, void* y, void* scratch, size_t scratch_bytes, void* stream_) {
    QFormat f;
    IMX_TRY(validate_format(mode, bits, group_size, &f));
    IMX_REQUIRE(x && w && y && m >= 0 && n_out > 0 && in > 0, "quantized_matmul: bad arguments");
    IMX_REQUIRE(w->w != nullptr && w->scales != nullptr && (f.mode != IMX_MODE_AFFINE || w->biases != nullptr),
                "quantized_matmul: weight, scales (and biases for affine) are required");
    if (m == 0) return IMX_OK;
    cudaStream_t stream = (cudaStream_t)stream_;
    ExpertSet set;
    IMX_TRY(qmm_set(*w, n_out, in, f, &set));
    const int path = ((uintptr_t)w->w % 16 == 0 && (uintptr_t)w->scales % 16 == 0 && (w->biases == nullptr || (uintptr_t)w->biases % 16 == 0))
                         ? qmm_path(set, m) : IMX_PATH_GENERIC;
    if (path == IMX_PATH_GENERIC)      // no expert kernel takes this shape: the scalar kernel
        return imx_quantized_matmul(x, m, w, n_out, in, 1, group_size, bits, mode, y, stream_);
    const OneWs ws = carve_one(m, in, 0, n_out, scratch);
    IMX_TRY(check_scratch(scratch, scratch_bytes, ws.bytes, "quantized_matmul"));
    int o[16];
    path_block_order(path, f, o);
    Order16 order;
    for (int i = 0; i < 16; ++i) order.o[i] = (int8_t)o[i];
    const bool tmap_second = path == IMX_PATH_DECODE && decode_tmap_supported(set);
    order.pair_scale_odd = tmap_second ? 0.0625f : 1.f;
    prepare_one_kernel<<<m + 1, 256, 0, stream>>>((const __nv_bfloat16*)x, m, in, ws.x16, order, unit_rows_for(path), ws.offsets,
                                                  ws.ident, ws.units, ws.n_units, ws.sw.sched, ws.sw.n_ints,
                                                  tmap_second ? ws.psum : nullptr); IMX_LAUNCHED();
    IMX_CHECK_CUDA(cudaGetLastError());
    GroupedArgs ga = {};
    ga.set = set;
    ga.second_only = 1;
    ga.n_slots = m;
    ga.units = ws.units;
    ga.n_units = ws.n_units;
    ga.max_units = ws.max_units;
    use_sched(ga, ws.sw);
    ga.partials = ws.partials;
    ga.psum = ws.psum;
    ga.act = ws.x16;                 // the second product reads its activations here
    ga.act_stride = in;
    ga.out = ws.rows;
    ga.status = ws.status;
    IMX_TRY(run_experts(path, ga, stream));
    return launch_combine(ws.rows, nullptr, ws.ident, m, 1, n_out, nullptr, y, stream);
}

int imx_expert_scratch_bytes(const imx_moe_config* cfg, int m, size_t* bytes) {
    QFormat f;
    IMX_TRY(check_config(cfg, &f));
    IMX_REQUIRE(bytes != nullptr && m >= 0, "expert_scratch_bytes: bad arguments");
    *bytes = carve_one(m, cfg->hidden, cfg->intermediate, cfg->hidden, nullptr).bytes;
    return IMX_OK;
}

int imx_expert_forward(const imx_moe_config* cfg, const imx_qtensor* gate_up, const imx_qtensor* down, const void* x,
                       int m, void* y, void* scratch, size_t scratch_bytes, void* stream_) {
    QFormat f;
    IMX_TRY(check_config(cfg, &f));
    IMX_REQUIRE(gate_up && down && m >= 0, "expert_forward: gate_up and down are required");
    if (m == 0) return IMX_OK;
    IMX_REQUIRE(x && y, "expert_forward: x and y are required");
    imx_moe_config c = *cfg;
    c.num_experts = 1;
    c.top_k = 1;
    c.shared_intermediate = 0;
    const OneWs ws = carve_one(m, c.hidden, c.intermediate, c.hidden, scratch);
    IMX_TRY(check_scratch(scratch, scratch_bytes, ws.bytes, "expert_forward"));
    cudaStream_t stream = (cudaStream_t)stream_;
    ExpertSet set;
    IMX_TRY(make_expert_set(c, f, *gate_up, *down, 1, nullptr, &set));
    int path;
    IMX_TRY(pick_path(c, set, (long)m, &path));
    int o[16];
    path_block_order(path, f, o);
    Order16 order;
    for (int i = 0; i < 16; ++i) order.o[i] = (int8_t)o[i];
    const bool tmap = path == IMX_PATH_DECODE && decode_tmap_supported(set);
    order.pair_scale_odd = tmap ? 0.0625f : 1.f;
    prepare_one_kernel<<<m + 1, 256, 0, stream>>>((const __nv_bfloat16*)x, m, c.hidden, ws.x16, order, unit_rows_for(path),
                                                  ws.offsets, ws.ident, ws.units, ws.n_units, ws.sw.sched, ws.sw.n_ints,
                                                  nullptr); IMX_LAUNCHED();
    IMX_CHECK_CUDA(cudaGetLastError());
    const bool rows_f16 = is_prefill(path);
    GroupedArgs ga = {};
    ga.set = set;
    ga.in = ws.x16;
    ga.n_slots = m;
    ga.units = ws.units;
    ga.n_units = ws.n_units;
    ga.max_units = ws.max_units;
    use_sched(ga, ws.sw);
    ga.partials = ws.partials;
    ga.psum = ws.psum;
    ga.gsum_x = ws.gsum_x;
    ga.n_in_rows = m;
    ga.act = ws.act;
    ga.act_stride = c.intermediate;
    ga.out = ws.rows;
    ga.out16 = rows_f16 ? reinterpret_cast<__half*>(ws.rows) : nullptr;
    ga.status = ws.status;
    IMX_TRY(run_experts(path, ga, stream));
    return launch_combine(ws.rows, nullptr, ws.ident, m, 1, c.hidden, nullptr, y, stream, false, nullptr, rows_f16);
}

int imx_linear(const void* x, int m, int in, const void* w, int n_out, const void* bias, void* y, void* stream) {
    IMX_REQUIRE(x && w && y && m >= 0 && in > 0 && n_out > 0, "linear: bad arguments");
    IMX_REQUIRE(in % 8 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0,
                "linear: input dimension (%d) must be a multiple of 8 and x, w 16-byte aligned", in);
    if (m == 0) return IMX_OK;
    const dim3 grid((unsigned)ceil_div(n_out, kLT), (unsigned)ceil_div(m, kLT));
    linear_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, m, in, (const __nv_bfloat16*)w, n_out,
                                                          (const __nv_bfloat16*)bias, (__nv_bfloat16*)y); IMX_LAUNCHED();
    IMX_CHECK_CUDA(cudaGetLastError());
    return IMX_OK;
}

}  // extern "C"
