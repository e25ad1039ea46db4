// Pieces shared by the two decode-regime expert kernels (register-pipelined
// and TMA-pipelined): integer-code -> fp16 fragment builders, the m16n8k16
// MMA wrapper, per-task pointer set-up and the epilogues.
#pragma once
#include "internal.h"

namespace imx {
namespace decode {

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
                    a.act[(size_t)(c.slot0 + slot_l) * a.act_stride + col] = f32_to_f16_sat(v, a.status);
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


}  // namespace decode
}  // namespace imx
