// Decode-regime grouped expert products (few tokens per expert): a
// bandwidth-bound dequant kernel that streams each selected expert's packed
// weights exactly once and feeds the tensor cores with tokens on the n=8 side
// of mma.m16n8k16 (fp16 operands, fp32 accumulation).
//
// Replaces, per expert, the three `quantized_matmul` calls plus silu/multiply
// of mlx/src/nn/moe.rs:26-32 (and mlx/src/nn/mlp.rs:27-33 for the shared
// expert), for affine 2/4/8-bit weights with group size 64 or 128.
//
// How the arithmetic is arranged
//   * A operand = the raw integer codes q, turned into fp16 with one
//     shift+lop3 (or one prmt) per two codes by planting them in the mantissa
//     of a constant (64+q for 2/4-bit, 1024+q for 8-bit): exact, no rounding.
//   * B operand = fp16 activations of the unit's <= 8 slots.
//   * Per 64 codes (one group) the fp32 partial sums are folded as
//         acc += scale * sum(x*(off+q)) + (bias - off*scale) * sum(x)
//     so the result equals x . (scale*q + bias) with fp32 accumulation and no
//     rounding of the dequantized weight.  sum(x) comes from one extra MMA
//     per 16 codes whose A operand is all ones: it lands in exactly the
//     accumulator layout the fold needs.
//   * The reduction index inside each block of 16 is permuted (sums do not
//     care) so that the codes a thread needs for its A fragments are the
//     contiguous bytes it loaded, and the matching B fragments are 32
//     contiguous bytes of a pre-permuted activation row.
//
// How the work is arranged
//   * task = (work unit of <= 8 slots of one expert, pair of 16-row tiles):
//     gate tile + up tile for the first product (SwiGLU in registers), two
//     consecutive tiles for the second.  Tasks are independent and every
//     warp owns a contiguous, balanced range of them: no shared memory, no
//     block barriers, no atomics, deterministic.
//   * each lane streams its rows with 8/16-byte loads that bypass L1,
//     prefetched kStages iterations (128 codes each) ahead through a register
//     ring that runs across task boundaries; activations come through L1.
#include "internal.h"

namespace imx {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kStages = 4;          // register prefetch depth (iterations of 128 codes)

// ── per-bit-width code handling ──────────────────────────────────────────────
// order(p) = which of the 16 reduction indices of a block sits at position p
// of the permuted activation row; MMA m (0..3) of a block consumes positions
// 4m..4m+3: (4m,4m+1) -> fragment register 0, (4m+2,4m+3) -> register 1.
template <int BITS>
struct Codec;

template <>
struct Codec<4> {
    static constexpr int WORDS = 2;
    static constexpr float OFFSET = 64.f;
    // {0,4,1,5, 2,6,3,7, 8,12,9,13, 10,14,11,15}
    __host__ __device__ static constexpr int order(int p) {
        return 8 * (p >> 3) + 2 * ((p >> 2) & 1) + ((p >> 1) & 1) + 4 * (p & 1);
    }
    // fragment registers (r0: positions 4m,4m+1; r1: 4m+2,4m+3) from the raw words
    template <int M>
    __device__ static __forceinline__ void frag(const uint32_t* w, uint32_t& r0, uint32_t& r1) {
        const uint32_t v = w[M >> 1];
        constexpr int J = 2 * (M & 1);   // nibble pairs (J, J+4) and (J+1, J+5)
        const uint32_t s0 = J == 0 ? (v << 4) : (v >> 4);   // J = 0 or 2
        const uint32_t s1 = J == 0 ? v : (v >> 8);          // J+1 = 1 or 3
        asm("lop3.b32 %0, %1, 0x00f000f0, 0x54005400, 0xea;" : "=r"(r0) : "r"(s0));
        asm("lop3.b32 %0, %1, 0x00f000f0, 0x54005400, 0xea;" : "=r"(r1) : "r"(s1));
    }
};

template <>
struct Codec<8> {
    static constexpr int WORDS = 4;
    static constexpr float OFFSET = 1024.f;
    // {0,2,1,3, 4,6,5,7, 8,10,9,11, 12,14,13,15}
    __host__ __device__ static constexpr int order(int p) {
        return 4 * (p >> 2) + 2 * (p & 1) + ((p >> 1) & 1);
    }
    template <int M>
    __device__ static __forceinline__ void frag(const uint32_t* w, uint32_t& r0, uint32_t& r1) {
        const uint32_t v = w[M];
        asm("prmt.b32 %0, %1, 0x64646464, 0x4240;" : "=r"(r0) : "r"(v));   // bytes (0, 2)
        asm("prmt.b32 %0, %1, 0x64646464, 0x4341;" : "=r"(r1) : "r"(v));   // bytes (1, 3)
    }
};

template <>
struct Codec<2> {
    static constexpr int WORDS = 1;
    static constexpr float OFFSET = 64.f;
    // {0,8,1,9, 2,10,3,11, 4,12,5,13, 6,14,7,15}
    __host__ __device__ static constexpr int order(int p) {
        return 2 * (p >> 2) + ((p >> 1) & 1) + 8 * (p & 1);
    }
    // field J (bits [2J, 2J+2)) moved to bits [4, 6) of its half-word
    template <int J>
    __device__ static __forceinline__ uint32_t to_bit4(uint32_t v) {
        if constexpr (2 * J >= 4) return v >> (2 * J - 4);
        else return v << (4 - 2 * J);
    }
    template <int M>
    __device__ static __forceinline__ void frag(const uint32_t* w, uint32_t& r0, uint32_t& r1) {
        const uint32_t v = w[0];
        const uint32_t s0 = to_bit4<2 * M>(v);       // field pairs (J, J+8)
        const uint32_t s1 = to_bit4<2 * M + 1>(v);
        asm("lop3.b32 %0, %1, 0x00300030, 0x54005400, 0xea;" : "=r"(r0) : "r"(s0));
        asm("lop3.b32 %0, %1, 0x00300030, 0x54005400, 0xea;" : "=r"(r1) : "r"(s1));
    }
};

__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int WORDS>
__device__ __forceinline__ void ldg_stream(uint32_t* dst, const uint8_t* p) {
    if constexpr (WORDS == 1) {
        asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(dst[0]) : "l"(p));
    } else if constexpr (WORDS == 2) {
        asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(dst[0]), "=r"(dst[1]) : "l"(p));
    } else {
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(dst[0]), "=r"(dst[1]), "=r"(dst[2]), "=r"(dst[3])
                     : "l"(p));
    }
}

// Everything a warp needs to know about the task it is fetching/computing.
struct TaskCtx {
    const uint8_t* w[2][2];      // [tile][row g / row g+8]: packed row, already offset by lane's t
    const uint8_t* s[2][2];      // scales rows
    const uint8_t* b[2][2];      // biases rows
    const __half* act_in;        // this lane's activation row (slot g of the unit) or nullptr
    int n_it;                    // iterations of 128 codes
    int rows;                    // valid slots in the unit
    int slot0;
    int row0[2];                 // first output row of each tile
    int valid;                   // tile rows exist for this expert
    float gs[2];                 // tensor scales (1 for affine)
};

template <int BITS, bool SWIGLU>
__device__ __forceinline__ void setup_task(const GroupedArgs& a, int task, int pairs_per_unit, int g, int t,
                                           bool g128, TaskCtx& c) {
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
    c.valid = c.row0[0] < n_out;
    if (!c.valid) {
        c.n_it = 0;
        return;
    }
    const size_t row_w = (size_t)K * BITS / 8;
    const size_t row_s = (size_t)(K / (g128 ? 128 : 64)) * 2;
    QMat m[2];
    if (SWIGLU) {
        m[0] = extra ? S.x_gate : S.gate;
        m[1] = extra ? S.x_up : S.up;
        if (!extra) {
            for (int i = 0; i < 2; ++i) {
                m[i].w += (size_t)u.expert * S.gu_stride_w;
                m[i].scales += (size_t)u.expert * S.gu_stride_s;
                m[i].biases += (size_t)u.expert * S.gu_stride_s;
            }
        }
    } else {
        m[0] = extra ? S.x_down : S.down;
        if (!extra) {
            m[0].w += (size_t)u.expert * S.dn_stride_w;
            m[0].scales += (size_t)u.expert * S.dn_stride_s;
            m[0].biases += (size_t)u.expert * S.dn_stride_s;
        }
        m[1] = m[0];
    }
#pragma unroll
    for (int T = 0; T < 2; ++T) {
        c.gs[T] = m[T].global_scale;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const size_t r = (size_t)(c.row0[T] + g + 8 * h);
            c.w[T][h] = m[T].w + r * row_w + (size_t)t * (16 * BITS / 8);
            c.s[T][h] = m[T].scales + r * row_s;
            c.b[T][h] = m[T].biases + r * row_s;
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

template <int BITS>
struct Stage {
    uint32_t w[2][2][2][Codec<BITS>::WORDS];   // [tile][row half][step][words]
    uint32_t s[2][2];                          // [tile][row half]: bf16 scale of step 0 | step 1 << 16
    uint32_t b[2][2];
};

template <int BITS>
__device__ __forceinline__ void fetch(Stage<BITS>& st, const TaskCtx& c, int it, bool g128) {
    constexpr int W = Codec<BITS>::WORDS;
    const size_t koff = (size_t)it * (128 * BITS / 8);
#pragma unroll
    for (int T = 0; T < 2; ++T)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int s = 0; s < 2; ++s) ldg_stream<W>(st.w[T][h][s], c.w[T][h] + koff + (size_t)s * (64 * BITS / 8));
            if (g128) {
                const uint32_t sv = __ldg(reinterpret_cast<const uint16_t*>(c.s[T][h]) + it);
                const uint32_t bv = __ldg(reinterpret_cast<const uint16_t*>(c.b[T][h]) + it);
                st.s[T][h] = sv | (sv << 16);
                st.b[T][h] = bv | (bv << 16);
            } else {
                st.s[T][h] = __ldg(reinterpret_cast<const uint32_t*>(c.s[T][h]) + it);
                st.b[T][h] = __ldg(reinterpret_cast<const uint32_t*>(c.b[T][h]) + it);
            }
        }
}

template <int BITS, int M>
__device__ __forceinline__ void mma_tile(float (&tmp)[4], const uint32_t* wlo, const uint32_t* whi,
                                         const uint32_t* bf) {
    uint32_t a0, a1, a2, a3;
    Codec<BITS>::template frag<M>(wlo, a0, a2);
    Codec<BITS>::template frag<M>(whi, a1, a3);
    mma_f16(tmp, a0, a1, a2, a3, bf[2 * M], bf[2 * M + 1]);
}

template <int BITS>
__device__ __forceinline__ void compute(const Stage<BITS>& st, const TaskCtx& c, int it, float (&acc)[2][4]) {
    // activations of this iteration: 2 steps x 32 bytes (this lane's slot, its 16 codes per step)
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
    constexpr uint32_t ONES = 0x3c003c00u;   // fp16 (1, 1)
#pragma unroll
    for (int s = 0; s < 2; ++s) {
        float xs[4] = {0.f, 0.f, 0.f, 0.f};   // sum of x over the group, per (row, slot) of the C layout
#pragma unroll
        for (int m = 0; m < 4; ++m) mma_f16(xs, ONES, ONES, ONES, ONES, bf[s][2 * m], bf[s][2 * m + 1]);
#pragma unroll
        for (int T = 0; T < 2; ++T) {
            float tmp[4] = {0.f, 0.f, 0.f, 0.f};
            mma_tile<BITS, 0>(tmp, st.w[T][0][s], st.w[T][1][s], bf[s]);
            mma_tile<BITS, 1>(tmp, st.w[T][0][s], st.w[T][1][s], bf[s]);
            mma_tile<BITS, 2>(tmp, st.w[T][0][s], st.w[T][1][s], bf[s]);
            mma_tile<BITS, 3>(tmp, st.w[T][0][s], st.w[T][1][s], bf[s]);
            const float s_lo = __uint_as_float(s == 0 ? (st.s[T][0] << 16) : (st.s[T][0] & 0xffff0000u));
            const float s_hi = __uint_as_float(s == 0 ? (st.s[T][1] << 16) : (st.s[T][1] & 0xffff0000u));
            const float b_lo = __uint_as_float(s == 0 ? (st.b[T][0] << 16) : (st.b[T][0] & 0xffff0000u));
            const float b_hi = __uint_as_float(s == 0 ? (st.b[T][1] << 16) : (st.b[T][1] & 0xffff0000u));
            const float bp_lo = fmaf(-Codec<BITS>::OFFSET, s_lo, b_lo);
            const float bp_hi = fmaf(-Codec<BITS>::OFFSET, s_hi, b_hi);
            acc[T][0] += fmaf(s_lo, tmp[0], bp_lo * xs[0]);
            acc[T][1] += fmaf(s_lo, tmp[1], bp_lo * xs[1]);
            acc[T][2] += fmaf(s_hi, tmp[2], bp_hi * xs[2]);
            acc[T][3] += fmaf(s_hi, tmp[3], bp_hi * xs[3]);
        }
    }
}

// position of reduction index i (0..15) inside the permuted block of 16
template <int BITS>
__device__ __forceinline__ int permuted_pos(int i) {
    uint64_t lut = 0;
#pragma unroll
    for (int p = 0; p < 16; ++p) lut |= (uint64_t)p << (4 * Codec<BITS>::order(p));
    return (int)((lut >> (4 * i)) & 0xf);
}

template <int BITS, bool SWIGLU>
__device__ __forceinline__ void epilogue(const GroupedArgs& a, const TaskCtx& c, float (&acc)[2][4], int g, int t) {
    if (c.valid) {
        if (SWIGLU) {
            // gate tile = acc[0], up tile = acc[1], same (row, slot) positions
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int slot_l = 2 * t + (i & 1);
                const int row = c.row0[0] + g + 8 * (i >> 1);
                if (slot_l < c.rows) {
                    const float v = silu_f(acc[0][i] * c.gs[0]) * (acc[1][i] * c.gs[1]);
                    // stored in the permuted order the second product reads
                    const int col = (row & ~15) + permuted_pos<BITS>(row & 15);
                    a.act[(size_t)(c.slot0 + slot_l) * a.act_stride + col] = f32_to_f16_sat(v);
                }
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
                        a.out[(size_t)slot * a.set.n_in + row] = acc[T][i] * c.gs[T] * sc;
                    }
                }
        }
    }
#pragma unroll
    for (int T = 0; T < 2; ++T)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[T][i] = 0.f;
}

template <int BITS, bool SWIGLU>
__global__ void __launch_bounds__(kThreads, 1)
decode_mma_kernel(const GroupedArgs a, const int pairs_per_unit, const int g128) {
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const long gw = (long)blockIdx.x * kWarps + (threadIdx.x >> 5);
    const long nw = (long)gridDim.x * kWarps;
    const long n_tasks = (long)(*a.n_units) * pairs_per_unit;
    const int task_lo = (int)(gw * n_tasks / nw);
    const int task_hi = (int)((gw + 1) * n_tasks / nw);
    if (task_lo >= task_hi) return;

    TaskCtx fc, cc;                 // fetch cursor, compute cursor
    int f_task = task_lo, f_it = 0;
    int c_task = task_lo, c_it = 0;
    setup_task<BITS, SWIGLU>(a, f_task, pairs_per_unit, g, t, g128, fc);
    cc = fc;
    // skip tasks with nothing to stream
    auto advance_fetch = [&]() {
        while (f_task < task_hi && f_it >= fc.n_it) {
            ++f_task;
            f_it = 0;
            if (f_task < task_hi) setup_task<BITS, SWIGLU>(a, f_task, pairs_per_unit, g, t, g128, fc);
        }
    };
    float acc[2][4];
#pragma unroll
    for (int T = 0; T < 2; ++T)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[T][i] = 0.f;
    auto advance_compute = [&]() {
        while (c_task < task_hi && c_it >= cc.n_it) {
            epilogue<BITS, SWIGLU>(a, cc, acc, g, t);
            ++c_task;
            c_it = 0;
            if (c_task < task_hi) setup_task<BITS, SWIGLU>(a, c_task, pairs_per_unit, g, t, g128, cc);
        }
    };
    advance_fetch();
    advance_compute();

    Stage<BITS> ring[kStages];
#pragma unroll
    for (int s = 0; s < kStages - 1; ++s) {
        if (f_task < task_hi) {
            fetch<BITS>(ring[s], fc, f_it, g128);
            ++f_it;
            advance_fetch();
        }
    }
    while (c_task < task_hi) {
#pragma unroll
        for (int s = 0; s < kStages; ++s) {
            if (c_task < task_hi) {
                if (f_task < task_hi) {
                    fetch<BITS>(ring[(s + kStages - 1) % kStages], fc, f_it, g128);
                    ++f_it;
                    advance_fetch();
                }
                compute<BITS>(ring[s], cc, c_it, acc);
                ++c_it;
                advance_compute();
            }
        }
    }
}

template <int BITS>
int launch_bits(const GroupedArgs& a, int g128, cudaStream_t stream, cudaEvent_t mid) {
    const ExpertSet& s = a.set;
    int dev = 0, sms = 148;
    IMX_CHECK_CUDA(cudaGetDevice(&dev));
    IMX_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int mid_max = s.has_extra && s.x_mid > s.n_mid ? s.x_mid : s.n_mid;
    const int grid = sms;                       // one resident CTA of 8 warps per SM
    decode_mma_kernel<BITS, true><<<grid, kThreads, 0, stream>>>(a, mid_max / 16, g128);
    IMX_CHECK_CUDA(cudaGetLastError());
    if (mid) IMX_CHECK_CUDA(cudaEventRecord(mid, stream));
    decode_mma_kernel<BITS, false><<<grid, kThreads, 0, stream>>>(a, s.n_in / 32, g128);
    IMX_CHECK_CUDA(cudaGetLastError());
    return IMX_OK;
}

}  // namespace

// 16-index block order of the activation rows the kernels of a bit width read
// (identity when the width has no tensor-core decode path).
void decode_block_order(int bits, int order[16]) {
    for (int i = 0; i < 16; ++i) order[i] = i;
    if (bits == 4) for (int i = 0; i < 16; ++i) order[i] = Codec<4>::order(i);
    if (bits == 8) for (int i = 0; i < 16; ++i) order[i] = Codec<8>::order(i);
    if (bits == 2) for (int i = 0; i < 16; ++i) order[i] = Codec<2>::order(i);
}

bool decode_mma_supported(const ExpertSet& s) {
    const QFormat& f = s.fmt;
    if (f.mode != IMX_MODE_AFFINE) return false;
    if (f.bits != 2 && f.bits != 4 && f.bits != 8) return false;
    if (f.group != 64 && f.group != 128) return false;
    if (s.n_in % 128 || s.n_mid % 128) return false;
    if (s.has_extra && s.x_mid % 128) return false;
    return true;
}

int launch_decode_mma(const GroupedArgs& a, cudaStream_t stream, cudaEvent_t mid) {
    IMX_REQUIRE(decode_mma_supported(a.set), "decode path: format/shape not supported");
    if (a.max_units == 0) return IMX_OK;
    const int g128 = a.set.fmt.group == 128;
    switch (a.set.fmt.bits) {
        case 4: return launch_bits<4>(a, g128, stream, mid);
        case 8: return launch_bits<8>(a, g128, stream, mid);
        default: return launch_bits<2>(a, g128, stream, mid);
    }
}

}  // namespace imx
