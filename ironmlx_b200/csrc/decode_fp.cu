// Decode-regime grouped expert products for the block-scaled float formats
// (mxfp8: e4m3 values, one ue8m0 scale per 32; nvfp4: e2m1 values, one e4m3
// scale per 16 and an fp32 tensor scale): the per-expert `quantized_matmul`
// calls of mlx/src/nn/moe.rs:26-32 with `mode` = "mxfp8" / "nvfp4"
// (mlx/src/nn/linear.rs:33-49, mlx/src/ops.rs:688-693).
//
// A bandwidth-bound kernel on the skeleton of the affine decode kernel
// (decode_mma.cu): every selected expert's packed weights are streamed exactly
// once with 16-byte / 8-byte loads that bypass L1, through a register ring that
// runs across task boundaries; tokens sit on the n = 8 side of
// mma.m16n8k16 (fp16 x fp16 -> fp32).
//
//   * a lane converts its 16 consecutive values of a row with `cvt.rn.f16x2`
//     (e4m3x2 / e2m1x2: exact) and multiplies them by their block scale in fp16:
//       nvfp4  e2m1 x e4m3 needs at most 5 significant bits and stays inside
//              fp16's normal range: the product is exact; the fp32 tensor
//              scale is applied in the epilogue;
//       mxfp8  the scale is a power of two; it is applied relative to the
//              largest scale exponent r of the weight row, 2^(s - r) <= 1
//              (exact down to 2^-24 of the row's largest magnitude), and
//              2^(r - 127) is applied in the epilogue in fp32.
//     The scaled values feed the MMAs directly, so one accumulator runs over
//     the whole reduction length (two, alternating, to halve the dependent
//     chain) and no per-group fold is needed.
//   * task = (work unit of <= 8 slots of one expert, pair of 16-row tiles):
//     gate tile + up tile (SwiGLU in registers) or two down tiles; every warp
//     owns a contiguous, balanced range of tasks: no shared memory, no block
//     barriers, no atomics, deterministic.
//   * the reduction index is in natural order (activation rows are read as the
//     router wrote them).
#include "decode_common.cuh"

namespace imx {

namespace {

using namespace decode;

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
// Two CTAs of eight warps per SM with a ring of two iterations each (128 registers): measured against one CTA with
// four iterations in flight (238 registers), c4 decode: 441 -> 389 us (mxfp8), 284 -> 219 us (nvfp4) per step.
constexpr int kStages = 2;          // register prefetch depth (iterations of 128 values)
constexpr int kCtasPerSm = 2;

// MX = true: mxfp8, else nvfp4.
template <bool MX>
struct Fp {
    static constexpr int WORDS = MX ? 4 : 2;                 // words of a lane's 16 values
    static constexpr int SWORDS = MX ? 1 : 2;                // scale words of one iteration of a row
    static constexpr int ROW_BYTES_PER_VALUE_NUM = MX ? 8 : 4;   // bits per value
    static constexpr int GROUP = MX ? 32 : 16;
};

template <bool MX>
struct FpStage {
    uint32_t w[2][2][2][Fp<MX>::WORDS];   // [tile][row half][step][words]
    uint32_t s[2][2][Fp<MX>::SWORDS];     // [tile][row half]: the iteration's scale bytes of the row
};

struct FpTask {
    const uint8_t* w[2][2];      // [tile][row g / row g+8]: packed row, already offset by the lane's t
    const uint8_t* s[2][2];      // scale rows
    const __half* act_in;        // this lane's activation row (slot g of the unit) or nullptr
    int n_it;                    // iterations of 128 values
    int rows;                    // valid slots in the unit
    int slot0;
    int row0[2];                 // first output row of each tile
    float rowf[2][2];            // epilogue factor of rows g, g+8 of each tile
    int rexp[2][2];              // mxfp8: largest scale exponent of those rows
};

template <bool MX, bool SWIGLU>
__device__ __forceinline__ void setup_task(const GroupedArgs& a, int task, int pairs_per_unit, int g, int t, FpTask& c) {
    const ExpertSet& S = a.set;
    const int unit_id = task / pairs_per_unit;
    const int pair = task - unit_id * pairs_per_unit;
    const WorkUnit u = a.units[unit_id];
    const bool extra = u.expert >= S.num_experts;
    const int K = SWIGLU ? S.n_in : (extra ? S.x_mid : S.n_mid);
    const int n_out = SWIGLU ? (extra ? S.x_mid : S.n_mid) : S.n_in;
    c.n_it = K >> 7;
    c.rows = u.rows;
    c.slot0 = u.slot0;
    c.row0[0] = SWIGLU ? pair * 16 : pair * 32;
    c.row0[1] = SWIGLU ? pair * 16 : pair * 32 + 16;
    if (c.row0[0] >= n_out) {      // the unit's expert has fewer tile pairs than the widest one
        c.n_it = 0;
        return;
    }
    const size_t row_w = (size_t)K * Fp<MX>::ROW_BYTES_PER_VALUE_NUM / 8;
    const size_t row_s = (size_t)K / Fp<MX>::GROUP;
    QMat m[2];
    if (SWIGLU) {
        m[0] = extra ? S.x_gate : S.gate;
        m[1] = extra ? S.x_up : S.up;
        if (!extra) {
            for (int i = 0; i < 2; ++i) {
                m[i].w += (size_t)u.expert * S.gu_stride_w;
                m[i].scales += (size_t)u.expert * S.gu_stride_s;
            }
        }
    } else {
        m[0] = extra ? S.x_down : S.down;
        if (!extra) {
            m[0].w += (size_t)u.expert * S.dn_stride_w;
            m[0].scales += (size_t)u.expert * S.dn_stride_s;
        }
        m[1] = m[0];
    }
#pragma unroll
    for (int T = 0; T < 2; ++T) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const size_t r = (size_t)(c.row0[T] + g + 8 * h);
            c.w[T][h] = m[T].w + r * row_w + (size_t)t * (16 * Fp<MX>::ROW_BYTES_PER_VALUE_NUM / 8);
            c.s[T][h] = m[T].scales + r * row_s;
            if (MX) {
                // largest scale byte of the row: the four lanes of a quad share the row, each scans a quarter
                uint32_t mx = 0;
                for (size_t i = (size_t)t * 4; i < row_s; i += 16) mx = __vmaxu4(mx, __ldg(reinterpret_cast<const uint32_t*>(c.s[T][h] + i)));
                mx = max(mx & 0xffu, max((mx >> 8) & 0xffu, max((mx >> 16) & 0xffu, mx >> 24)));
                mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                c.rexp[T][h] = (int)mx;
                c.rowf[T][h] = ue8m0_to_f32(mx);
            } else {
                c.rexp[T][h] = 0;
                c.rowf[T][h] = m[T].global_scale;
            }
        }
    }
    c.act_in = nullptr;
    if (g < u.rows) {
        const int slot = u.slot0 + g;
        if (SWIGLU) {
            const int row = a.row_index ? a.row_index[slot] : slot;
            c.act_in = a.in + (size_t)row * S.n_in + t * 16;
        } else {
            c.act_in = a.act + (size_t)slot * a.act_stride + t * 16;
        }
    }
}

template <bool MX>
__device__ __forceinline__ void fetch(FpStage<MX>& st, const FpTask& c, int it, int t) {
    constexpr int W = Fp<MX>::WORDS;
    const size_t koff = (size_t)it * (128 * Fp<MX>::ROW_BYTES_PER_VALUE_NUM / 8);
#pragma unroll
    for (int T = 0; T < 2; ++T)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int s = 0; s < 2; ++s)
                ldg_stream<W>(st.w[T][h][s], c.w[T][h] + koff + (size_t)s * (64 * Fp<MX>::ROW_BYTES_PER_VALUE_NUM / 8));
            if (MX) {
                st.s[T][h][0] = __ldg(reinterpret_cast<const uint32_t*>(c.s[T][h]) + it);      // 4 scales of 128 values
            } else {
                const uint2 v = __ldg(reinterpret_cast<const uint2*>(c.s[T][h]) + it);         // 8 scales of 128 values
                st.s[T][h][0] = v.x;
                st.s[T][h][1] = v.y;
            }
        }
    (void)t;
}

// 2^d (d <= 0) as fp16 in both halves; zero below 2^-24.
__device__ __forceinline__ uint32_t pow2_h2(int d) {
    uint32_t b = 0;
    if (d >= -14) b = (uint32_t)(d + 15) << 10;
    else if (d >= -24) b = 1u << (d + 24);
    return b | (b << 16);
}
__device__ __forceinline__ uint32_t hmul2_bits(uint32_t a, uint32_t b) {
    const __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
}

// The lane's 16 values of one row and step as eight fp16 pairs, scaled: v[2m], v[2m+1] feed MMA m.
template <bool MX>
__device__ __forceinline__ void convert(const uint32_t* w, uint32_t scale_h2, uint32_t (&v)[8]) {
    if (MX) {
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            uint32_t r0, r1;
            asm("{\n\t.reg .b16 lo, hi;\n\t"
                "mov.b32 {lo, hi}, %2;\n\t"
                "cvt.rn.f16x2.e4m3x2 %0, lo;\n\t"
                "cvt.rn.f16x2.e4m3x2 %1, hi;\n\t}"
                : "=r"(r0), "=r"(r1)
                : "r"(w[m]));
            v[2 * m] = hmul2_bits(r0, scale_h2);
            v[2 * m + 1] = hmul2_bits(r1, scale_h2);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            uint32_t r[4];
            asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
                "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
                "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
                "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
                "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
                "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                : "r"(w[j]));
#pragma unroll
            for (int e = 0; e < 4; ++e) v[4 * j + e] = hmul2_bits(r[e], scale_h2);
        }
    }
}

// Block scale of (row, step s) for lane t as a half2 pair.
template <bool MX>
__device__ __forceinline__ uint32_t scale_of(const uint32_t* sw, int s, int t, int rexp) {
    if (MX) {
        // bytes: group (s, t >> 1) of the iteration's four
        const uint32_t b = (sw[0] >> (8 * (2 * s + (t >> 1)))) & 0xffu;
        return pow2_h2((int)b - rexp);
    }
    const uint32_t b = (sw[s] >> (8 * t)) & 0xffu;
    uint32_t h;
    asm("{\n\t.reg .b16 x;\n\tcvt.u16.u32 x, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, x;\n\t}" : "=r"(h) : "r"(b));
    uint32_t both;
    asm("prmt.b32 %0, %1, %1, 0x1010;" : "=r"(both) : "r"(h));
    return both;
}

template <bool MX>
__device__ __forceinline__ void compute(const FpStage<MX>& st, const FpTask& c, int it, int t, float (&acc)[2][2][4]) {
    uint32_t bf[2][8];
#pragma unroll
    for (int s = 0; s < 2; ++s) {
        if (c.act_in != nullptr) {
            const uint4* p = reinterpret_cast<const uint4*>(c.act_in + (size_t)it * 128 + s * 64);
            const uint4 v0 = __ldg(p), v1 = __ldg(p + 1);
            bf[s][0] = v0.x; bf[s][1] = v0.y; bf[s][2] = v0.z; bf[s][3] = v0.w;
            bf[s][4] = v1.x; bf[s][5] = v1.y; bf[s][6] = v1.z; bf[s][7] = v1.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) bf[s][i] = 0u;
        }
    }
#pragma unroll
    for (int s = 0; s < 2; ++s) {
#pragma unroll
        for (int T = 0; T < 2; ++T) {
            uint32_t lo[8], hi[8];
            convert<MX>(st.w[T][0][s], scale_of<MX>(st.s[T][0], s, t, c.rexp[T][0]), lo);
            convert<MX>(st.w[T][1][s], scale_of<MX>(st.s[T][1], s, t, c.rexp[T][1]), hi);
#pragma unroll
            for (int m = 0; m < 4; ++m)
                mma_f16(acc[T][m & 1], lo[2 * m], hi[2 * m], lo[2 * m + 1], hi[2 * m + 1], bf[s][2 * m], bf[s][2 * m + 1]);
        }
    }
}

template <bool SWIGLU>
__device__ __forceinline__ void finish(const GroupedArgs& a, const FpTask& c, float (&acc)[2][2][4], int g, int t) {
    if (c.n_it > 0) {
        float r[2][4];
#pragma unroll
        for (int T = 0; T < 2; ++T)
#pragma unroll
            for (int i = 0; i < 4; ++i) r[T][i] = (acc[T][0][i] + acc[T][1][i]) * c.rowf[T][i >> 1];
        if (SWIGLU) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int slot_l = 2 * t + (i & 1);
                const int row = c.row0[0] + g + 8 * (i >> 1);
                if (slot_l < c.rows)
                    a.act[(size_t)(c.slot0 + slot_l) * a.act_stride + row] = f32_to_f16_sat(silu_f(r[0][i]) * r[1][i], a.status);
            }
        } else {
#pragma unroll
            for (int T = 0; T < 2; ++T)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int slot_l = 2 * t + (i & 1);
                    const int row = c.row0[T] + g + 8 * (i >> 1);
                    if (slot_l < c.rows) {
                        const int slot = c.slot0 + slot_l;
                        const float sc = a.row_scale ? a.row_scale[slot] : 1.f;
                        a.out[(size_t)slot * a.set.n_in + row] = r[T][i] * sc;
                    }
                }
        }
    }
#pragma unroll
    for (int T = 0; T < 2; ++T)
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[T][h][i] = 0.f;
}

template <bool MX, bool SWIGLU>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
decode_fp_kernel(const GroupedArgs a, const int pairs_per_unit) {
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const long gw = (long)blockIdx.x * kWarps + (threadIdx.x >> 5);
    const long nw = (long)gridDim.x * kWarps;
    const long n_tasks = (long)(*a.n_units) * pairs_per_unit;
    const int task_lo = (int)(gw * n_tasks / nw);
    const int task_hi = (int)((gw + 1) * n_tasks / nw);
    if (task_lo >= task_hi) return;

    FpTask fc, cc;                  // fetch cursor, compute cursor
    int f_task = task_lo, f_it = 0;
    int c_task = task_lo, c_it = 0;
    setup_task<MX, SWIGLU>(a, f_task, pairs_per_unit, g, t, fc);
    cc = fc;
    auto advance_fetch = [&]() {    // skips tasks with nothing to stream
        while (f_task < task_hi && f_it >= fc.n_it) {
            ++f_task;
            f_it = 0;
            if (f_task < task_hi) setup_task<MX, SWIGLU>(a, f_task, pairs_per_unit, g, t, fc);
        }
    };
    float acc[2][2][4];
#pragma unroll
    for (int T = 0; T < 2; ++T)
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[T][h][i] = 0.f;
    auto advance_compute = [&]() {
        while (c_task < task_hi && c_it >= cc.n_it) {
            finish<SWIGLU>(a, cc, acc, g, t);
            ++c_task;
            c_it = 0;
            if (c_task < task_hi) setup_task<MX, SWIGLU>(a, c_task, pairs_per_unit, g, t, cc);
        }
    };
    advance_fetch();
    advance_compute();

    FpStage<MX> ring[kStages];
#pragma unroll
    for (int s = 0; s < kStages - 1; ++s) {
        if (f_task < task_hi) {
            fetch<MX>(ring[s], fc, f_it, t);
            ++f_it;
            advance_fetch();
        }
    }
    while (c_task < task_hi) {
#pragma unroll
        for (int s = 0; s < kStages; ++s) {
            if (c_task < task_hi) {
                if (f_task < task_hi) {
                    fetch<MX>(ring[(s + kStages - 1) % kStages], fc, f_it, t);
                    ++f_it;
                    advance_fetch();
                }
                compute<MX>(ring[s], cc, c_it, t, acc);
                ++c_it;
                advance_compute();
            }
        }
    }
}

template <bool MX>
int launch_mode(const GroupedArgs& a, cudaStream_t stream, cudaEvent_t mid) {
    const ExpertSet& s = a.set;
    int dev = 0, sms = 148;
    IMX_CHECK_CUDA(cudaGetDevice(&dev));
    IMX_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int mid_max = s.has_extra && s.x_mid > s.n_mid ? s.x_mid : s.n_mid;
    if (!a.second_only) {
        decode_fp_kernel<MX, true><<<sms * kCtasPerSm, kThreads, 0, stream>>>(a, mid_max / 16); IMX_LAUNCHED();
        IMX_CHECK_CUDA(cudaGetLastError());
    }
    if (mid) IMX_CHECK_CUDA(cudaEventRecord(mid, stream));
    decode_fp_kernel<MX, false><<<sms * kCtasPerSm, kThreads, 0, stream>>>(a, s.n_in / 32); IMX_LAUNCHED();
    IMX_CHECK_CUDA(cudaGetLastError());
    return IMX_OK;
}

}  // namespace

bool decode_fp_supported(const ExpertSet& s) {
    const QFormat& f = s.fmt;
    if (f.mode == IMX_MODE_MXFP8) {
        if (f.bits != 8 || f.group != 32) return false;
    } else if (f.mode == IMX_MODE_NVFP4) {
        if (f.bits != 4 || f.group != 16) return false;
    } else {
        return false;
    }
    // iterations of 128 values (a row's scale bytes of one iteration are one aligned 4- or 8-byte word)
    if (s.n_in % 128 || s.n_mid % 128) return false;
    if (s.has_extra && s.x_mid % 128) return false;
    return true;
}

int launch_decode_fp(const GroupedArgs& a, cudaStream_t stream, cudaEvent_t mid) {
    IMX_REQUIRE(decode_fp_supported(a.set), "decode path (mxfp8 / nvfp4): format/shape not supported");
    if (a.max_units == 0) return IMX_OK;
    return a.set.fmt.mode == IMX_MODE_MXFP8 ? launch_mode<true>(a, stream, mid) : launch_mode<false>(a, stream, mid);
}

}  // namespace imx
