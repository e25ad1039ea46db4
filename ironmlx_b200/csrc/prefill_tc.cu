// Prefill-regime grouped expert products on the 5th-generation tensor cores,
// every MLX weight format the block accepts at these sizes (affine 2/4/8-bit,
// mxfp8, nvfp4):
//
//   first product   act[slot, :] = silu(x W_gate^T) * (x W_up^T)       (moe.rs:26-30)
//   second product  out[slot, :] = row_scale[slot] * (act W_down^T)    (moe.rs:31, 155-161)
//
// each the grouped form of `quantized_matmul(transpose = true)`
// (mlx/src/nn/linear.rs:51-63), with `tcgen05.mma` (kind::f16, fp16 x fp16 ->
// fp32) and the accumulator in tensor memory.
//
// The WEIGHTS are the A operand (M = 128 weight rows, one tensor-memory lane
// each), the sorted slots of one expert are the N side (N = the unit's rows
// rounded up to 16, at most 128), K in steps of 64.  The packed weights are
// dequantized by producer warps straight into TENSOR MEMORY (`tcgen05.st`), and
// the MMA takes A from there: the dequantized tile never passes through shared
// memory, which the 128 x 128 tile of an smem-smem MMA saturates (the measured
// limit of the kernel this one replaces).  Shared memory carries only what the
// copy engine brings: the activation tile (B operand, 128-byte swizzle) and
// the packed codes.  A variant with the dequantized tile in shared memory
// (TS = false) is kept as a cross-check.
//
// One persistent CTA per SM, 16 warps, specialised:
//   warp 0        issues the MMAs (one elected lane), commits a stage back to
//                 the loader and the finished accumulator to the epilogue (two
//                 accumulators: the epilogue of tile i overlaps the MMAs of i+1)
//   warp 1        allocates / frees tensor memory
//   warp 2        loader: tiled TMA copies of the activation tile, the packed
//                 codes (two boxes of 64 rows) per K step and, once per tile,
//                 the tile's scale (and bias) rows
//   warps 4..7    epilogue: tcgen05.ld of their 32 lanes; lane = weight row,
//                 column = slot.  First product: gate row j sits on lane
//                 16 q + l, the matching up row on lane 16 q + l + 16 of the same
//                 warp, so SwiGLU needs one shuffle exchange and no shared memory
//   warps 8..15   producers, two groups of four warps on alternating K steps; a
//                 thread owns one weight row: its 16/32/64 bytes of codes ->
//                 64 fp16 values (exact codes, one HFMA2 / HMUL2 with the
//                 group's scale) -> one tcgen05.st of 32 columns
// Every wait is bounded; on expiry the CTA records a status, every role leaves
// its loop and tensor memory is freed.  No thread-block clusters, no multicast.
//
// Scales: affine rounds s*q+b once to fp16.  nvfp4: q * (e4m3 block scale) is
// exact in fp16, the fp32 tensor scale is applied in the epilogue.  mxfp8: the
// e4m3 value times 2^(s - r), r the largest scale exponent of the weight row,
// is exact in fp16 (down to 2^-24 of the row's largest magnitude); 2^(r - 127)
// is applied per row in the epilogue.
#include <cuda.h>

#include <cstring>
#include <type_traits>

#include "decode_common.cuh"

namespace imx {

namespace {

using namespace decode;

constexpr int kTileK = 64;
constexpr int kXBytes = 128 * kTileK * 2;          // activation tile, 16 KB
constexpr int kWBytes = 128 * kTileK * 2;          // dequantized weight tile (TS = false only), 16 KB
constexpr int kMaxStages = 8;
constexpr int kSpin = 1 << 22;
constexpr uint32_t kTmemCols = 512;                // two 128-column accumulators + the ring of A tiles
constexpr uint32_t kTmemA = 256;                   // first column of the A ring (32 columns per stage)
constexpr int kThreadsTc = 640;                    // 20 warps: 4 control, 4 + 4 epilogue, 8 producers

enum { FMT_A4 = 0, FMT_A8 = 1, FMT_A2 = 2, FMT_MXFP8 = 3, FMT_NVFP4 = 4 };
__host__ __device__ constexpr int q_row_bytes(int fmt) {       // packed bytes of one row per K step
    return fmt == FMT_A8 || fmt == FMT_MXFP8 ? 64 : (fmt == FMT_A2 ? 16 : 32);
}

// Per-role cycle counters of CTA 0, compiled in only for timing experiments (-DIMX_TC_PROFILE).
#ifdef IMX_TC_PROFILE
__device__ unsigned long long g_tc_prof[2][16];
#define PROF_DECL long long _pt = 0, _p0 = clock64(), _pw[3] = {0, 0, 0};
#define PROF_BEGIN _pt = clock64();
#define PROF_END(i) _pw[i] += clock64() - _pt;
#define PROF_FLUSH(role)                                                                     \
    if (lane == 0 && blockIdx.x == 0) {                                                      \
        for (int _i = 0; _i < 3; ++_i) g_tc_prof[SWIGLU ? 1 : 0][(role) * 4 + _i] = _pw[_i]; \
        g_tc_prof[SWIGLU ? 1 : 0][(role) * 4 + 3] = clock64() - _p0;                         \
    }
#else
#define PROF_DECL
#define PROF_BEGIN
#define PROF_END(i)
#define PROF_FLUSH(role)
#endif

struct Bars {                                      // shared-memory control block
    uint64_t qfull[kMaxStages];                    // activation tile + packed codes landed (TMA bytes)
    uint64_t full[kMaxStages];                     // weights of the stage dequantized
    uint64_t empty[kMaxStages];                    // MMAs that read the stage retired
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint64_t sfull[2];                             // scales of a tile landed
    uint64_t sempty[2];                            // ... and were consumed by all producer warps
    uint32_t tmem_base;
    int abort;
};

struct TcMaps {
    CUtensorMap x;                                 // slot-ordered activations
    CUtensorMap w[3], s[3], b[3];                  // [0] stacked routed matrix, [1]/[2] the extra expert's
};

struct TcParams {
    int nt_r, nt_x;                                // weight-row tiles per unit: routed / extra expert
    int stages;
    int stage_bytes;
    int sc_bytes;                                  // one tile's scale buffer
    int panel_bytes;                               // resident activation panel (0: streamed per stage)
    int lg_group;                                  // log2 of the group size
    unsigned long long pos_lut;                    // position of reduction index i inside its block of 16, 4 bits each
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait; false (and the abort flag set) when it gives up or someone else did.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (int spin = 0; spin < kSpin; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 1023) == 1023 && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// K-major, 128-byte swizzle: rows of 128 bytes, atoms of 8 rows (1024 bytes).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// kind::f16 instruction descriptor: D fp32, A/B fp16 K-major, M = 128, N = n
__device__ __forceinline__ uint32_t idesc_for(int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
// D[tmem_d] (+)= A[tmem_a] * B[smem]: A from tensor memory
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_ss(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// 16 lanes x 64 columns: thread t gets, for each block j of 8 columns, lane t/4 columns 8j + 2(t%4), +1
// (v[4j], v[4j+1]) and lane t/4 + 8, same columns (v[4j+2], v[4j+3])
__device__ __forceinline__ void tmem_ld_16x64(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.16x256b.x8.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// 32 consecutive columns of this thread's lane <- v
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
          "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
          "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
// two fp32 -> packed fp16 (lo, hi), clamped to the finite range: one instruction
__device__ __forceinline__ uint32_t pack_f16_sat(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}
// silu with the approximate exponential and reciprocal (relative error ~1e-6, far inside the fp16 rounding that follows)
__device__ __forceinline__ float silu_fast(float g) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.4426950408889634f * g));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return g * r;
}
__device__ __forceinline__ void st_global_u16(void* p, uint32_t v) {
    asm volatile("st.global.u16 [%0], %1;" ::"l"(p), "h"((uint16_t)v) : "memory");
}
__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 bits_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ __half2 bf16_to_half2(uint32_t b) {
    return __float2half2_rn(__uint_as_float(b << 16));
}

// A ring position: stage slot and phase of the n-th K step of the CTA.
struct Ring {
    int s;
    uint32_t ph;
    __device__ __forceinline__ void advance(int by, int stages) {
        s += by;
        while (s >= stages) {
            s -= stages;
            ph ^= 1u;
        }
    }
};

// What a tile is made of: one 128-row weight tile x (a part of) the sorted slots of one work unit.
struct TileInfo {
    int expert, slot0, rows, ntile, extra;
    int K;
    int first;              // first tile of its work item (XR: the activation panel is loaded with it)
};

// Walks this CTA's tiles.  Work units hold up to 256 slots.  SPLIT: the kernel's tiles take at most 128
// slots, so a larger unit is cut into two halves (multiples of 16 rows).  XR = false: a work item is one
// (unit part, weight tile), items dealt round-robin.  XR = true: a work item is a unit part with all its
// weight tiles in turn (its activation panel stays in shared memory).  nt_r / nt_x: weight tiles per unit of
// the routed experts / the extra expert.  body(tile, index) returns false to stop.
template <bool SWIGLU, bool XR, bool SPLIT, typename F>
__device__ __forceinline__ void for_each_tile(const GroupedArgs& a, int nt_r, int nt_x, F&& body) {
    const int n_r = a.n_units[1], n_x = a.n_units[0] - n_r;
    const int tiles_r = n_r * nt_r;
    const int parts = SPLIT ? 2 : 1;
    const int total = (XR ? n_r + n_x : tiles_r + n_x * nt_x) * parts;
    int it = 0;
    for (int w0 = blockIdx.x; w0 < total; w0 += gridDim.x) {
        const int part = SPLIT ? (w0 & 1) : 0;
        const int w = SPLIT ? (w0 >> 1) : w0;
        int unit, nt0, ntn = 1;
        if (XR) {
            unit = w;
            nt0 = 0;
            ntn = w < n_r ? nt_r : nt_x;
        } else if (w < tiles_r) {
            unit = w / nt_r;
            nt0 = w - unit * nt_r;
        } else {
            const int l = w - tiles_r;
            unit = n_r + l / nt_x;
            nt0 = l - (l / nt_x) * nt_x;
        }
        const WorkUnit u = a.units[unit];
        TileInfo t;
        t.expert = u.expert;
        t.slot0 = u.slot0;
        t.rows = u.rows;
        if (SPLIT) {
            const int h0 = u.rows <= 128 ? u.rows : (((u.rows + 1) >> 1) + 15) & ~15;
            if (part == 1) {
                t.slot0 = u.slot0 + h0;
                t.rows = u.rows - h0;
            } else {
                t.rows = h0;
            }
            if (t.rows <= 0) continue;
        }
        t.extra = u.expert >= a.set.num_experts;
        t.K = SWIGLU ? a.set.n_in : (t.extra ? a.set.x_mid : a.set.n_mid);
        for (int nt = nt0; nt < nt0 + ntn; ++nt, ++it) {
            t.ntile = nt;
            t.first = nt == nt0;
            if (!body(t, it)) return;
        }
    }
}

// Tensor-map index and first row of the two 64-row halves of 128-row weight tile `sub` of an expert.
template <bool SWIGLU>
__device__ __forceinline__ void tile_rows(const GroupedArgs& a, const TileInfo& t, int sub, int& mi0, int& mi1, int& row0, int& row1) {
    if (SWIGLU) {
        if (t.extra) { mi0 = 1; mi1 = 2; row0 = row1 = sub * 64; }
        else { mi0 = mi1 = 0; row0 = t.expert * 2 * a.set.n_mid + sub * 64; row1 = row0 + a.set.n_mid; }
    } else {
        mi0 = mi1 = t.extra ? 1 : 0;
        row0 = (t.extra ? 0 : t.expert * a.set.n_in) + sub * 128;
        row1 = row0 + 64;
    }
}

// Row of the 128-row tile (0..127: the order of the two TMA boxes: first product 64 gate rows, then the 64
// matching up rows) a tensor-memory lane holds.  First product: in every group of 16 lanes the first 8 hold
// gate rows and the other 8 the matching up rows, so that a 16-lane tensor-memory load hands a thread the gate
// and the up value of the same (row, slot) and SwiGLU needs no exchange between threads.
template <bool SWIGLU>
__device__ __forceinline__ int tile_row_of_lane(int lane128) {
    if (!SWIGLU) return lane128;
    const int grp = lane128 >> 4, w = lane128 & 15;
    return ((w >> 3) << 6) + grp * 8 + (w & 7);
}

// ── dequantization of one weight row's K step: 64 values -> 32 registers of fp16 pairs ──
// q: shared address of the row's packed bytes (chunk c of 16 bytes at q + ((c ^ swz) << 4)).
template <int FMT>
struct Dequant;

template <>
struct Dequant<FMT_A4> {
    // scale/bias of a half step (32 values) given as half2 pairs
    static __device__ __forceinline__ void run(uint32_t q, uint32_t swz, const __half2 (&sc)[2], const __half2 (&bi)[2],
                                               uint32_t (&out)[32]) {
        const __half2 c1024 = __float2half2_rn(1024.f), c64 = __float2half2_rn(64.f);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const uint4 v4 = lds128(q + ((c ^ swz) << 4));
            const uint32_t words[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                // eight codes of a word -> (0,4) (1,5) (2,6) (3,7): the order the activation rows use
                uint32_t r[4];
                const uint32_t v = words[j], v8 = v >> 8;
                asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(r[0]) : "r"(v));
                asm("lop3.b32 %0, %1, 0x00f000f0, 0x54005400, 0xea;" : "=r"(r[1]) : "r"(v));
                asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(r[2]) : "r"(v8));
                asm("lop3.b32 %0, %1, 0x00f000f0, 0x54005400, 0xea;" : "=r"(r[3]) : "r"(v8));
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const __half2 qh = __hsub2(bits_h2(r[e]), (e & 1) ? c64 : c1024);      // exact code
                    out[(c * 4 + j) * 4 + e] = h2_bits(__hfma2(qh, sc[c], bi[c]));      // scale*q + bias
                }
            }
        }
    }
};

template <>
struct Dequant<FMT_A8> {
    static __device__ __forceinline__ void run(uint32_t q, uint32_t swz, const __half2 (&sc)[2], const __half2 (&bi)[2],
                                               uint32_t (&out)[32]) {
        const __half2 c1024 = __float2half2_rn(1024.f);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint4 v4 = lds128(q + ((c ^ swz) << 4));
            const uint32_t words[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                // four codes of a word -> (0,2) (1,3)
                uint32_t r0, r1;
                asm("prmt.b32 %0, %1, 0x64646464, 0x4240;" : "=r"(r0) : "r"(words[j]));
                asm("prmt.b32 %0, %1, 0x64646464, 0x4341;" : "=r"(r1) : "r"(words[j]));
                out[(c * 4 + j) * 2 + 0] = h2_bits(__hfma2(__hsub2(bits_h2(r0), c1024), sc[c >> 1], bi[c >> 1]));
                out[(c * 4 + j) * 2 + 1] = h2_bits(__hfma2(__hsub2(bits_h2(r1), c1024), sc[c >> 1], bi[c >> 1]));
            }
        }
    }
};

template <>
struct Dequant<FMT_A2> {
    static __device__ __forceinline__ void run(uint32_t q, uint32_t swz, const __half2 (&sc)[2], const __half2 (&bi)[2],
                                               uint32_t (&out)[32]) {
        (void)swz;
        const __half2 c1024 = __float2half2_rn(1024.f);
        const uint4 v4 = lds128(q);
        const uint32_t words[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            // sixteen codes of a word -> (J, J+8), J = 0..7
#pragma unroll
            for (int J = 0; J < 8; ++J) {
                uint32_t r;
                const uint32_t v = words[j] >> (2 * J);
                asm("lop3.b32 %0, %1, 0x00030003, 0x64006400, 0xea;" : "=r"(r) : "r"(v));
                out[j * 8 + J] = h2_bits(__hfma2(__hsub2(bits_h2(r), c1024), sc[j >> 1], bi[j >> 1]));
            }
        }
    }
};

template <>
struct Dequant<FMT_MXFP8> {
    // mult[h]: 2^(s - r) of the half step's group as a half2
    static __device__ __forceinline__ void run(uint32_t q, uint32_t swz, const __half2 (&mult)[2], const __half2 (&)[2],
                                               uint32_t (&out)[32]) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint4 v4 = lds128(q + ((c ^ swz) << 4));
            const uint32_t words[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t r0, r1;
                asm("{\n\t.reg .b16 lo, hi;\n\t"
                    "mov.b32 {lo, hi}, %2;\n\t"
                    "cvt.rn.f16x2.e4m3x2 %0, lo;\n\t"
                    "cvt.rn.f16x2.e4m3x2 %1, hi;\n\t}"
                    : "=r"(r0), "=r"(r1)
                    : "r"(words[j]));
                out[(c * 4 + j) * 2 + 0] = h2_bits(__hmul2(bits_h2(r0), mult[c >> 1]));
                out[(c * 4 + j) * 2 + 1] = h2_bits(__hmul2(bits_h2(r1), mult[c >> 1]));
            }
        }
    }
};

template <>
struct Dequant<FMT_NVFP4> {
    // sc4: the four e4m3 block scales of the step (one per 16 values), low byte first
    static __device__ __forceinline__ void run(uint32_t q, uint32_t swz, uint32_t sc4, uint32_t (&out)[32]) {
        uint32_t s01, s23;
        asm("{\n\t.reg .b16 lo, hi;\n\t"
            "mov.b32 {lo, hi}, %2;\n\t"
            "cvt.rn.f16x2.e4m3x2 %0, lo;\n\t"
            "cvt.rn.f16x2.e4m3x2 %1, hi;\n\t}"
            : "=r"(s01), "=r"(s23)
            : "r"(sc4));
        uint32_t sb[4];
        asm("prmt.b32 %0, %1, %1, 0x1010;" : "=r"(sb[0]) : "r"(s01));
        asm("prmt.b32 %0, %1, %1, 0x3232;" : "=r"(sb[1]) : "r"(s01));
        asm("prmt.b32 %0, %1, %1, 0x1010;" : "=r"(sb[2]) : "r"(s23));
        asm("prmt.b32 %0, %1, %1, 0x3232;" : "=r"(sb[3]) : "r"(s23));
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const uint4 v4 = lds128(q + ((c ^ swz) << 4));
            const uint32_t words[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                // a word = 8 values = half a block of 16: blocks 2c (j < 2) and 2c + 1
                uint32_t r[4];
                asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
                    "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
                    "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
                    "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
                    "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
                    "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
                    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                    : "r"(words[j]));
                const __half2 s = bits_h2(sb[2 * c + (j >> 1)]);
#pragma unroll
                for (int e = 0; e < 4; ++e) out[(c * 4 + j) * 4 + e] = h2_bits(__hmul2(bits_h2(r[e]), s));
            }
        }
    }
};

// 2^d (d <= 0) as an fp16 bit pattern in both halves; below 2^-24 it is zero.
__device__ __forceinline__ __half2 pow2_half2(int d) {
    uint32_t b = 0;
    if (d >= -14) b = (uint32_t)(d + 15) << 10;
    else if (d >= -24) b = 1u << (d + 24);
    return bits_h2(b | (b << 16));
}

// largest byte of n16 16-byte pieces
__device__ __forceinline__ uint32_t max_byte(uint4 v, uint32_t m) {
    m = __vmaxu4(m, v.x);
    m = __vmaxu4(m, v.y);
    m = __vmaxu4(m, v.z);
    return __vmaxu4(m, v.w);
}
__device__ __forceinline__ uint32_t hmax_bytes(uint32_t m) {
    m = max(m & 0xffu, max((m >> 8) & 0xffu, max((m >> 16) & 0xffu, m >> 24)));
    return m;
}

// WIDE: tiles of up to 256 slots (N = 256 per MMA: the issue cost of a tcgen05.mma, about 110 cycles whatever
// its N, is then covered by the 128 cycles it runs) with one accumulator of 256 columns and eight epilogue
// warps; otherwise tiles of up to 128 slots and two accumulators, the epilogue of tile i overlapping the MMAs
// of tile i+1.  XR: the unit part's activation panel stays in shared memory for all its weight tiles.
template <bool SWIGLU, int FMT, bool TS, bool WIDE, bool XR>
__global__ void __launch_bounds__(kThreadsTc, 1)
prefill_tc_kernel(const GroupedArgs a, const TcParams p, const __grid_constant__ TcMaps maps) {
    static_assert(!WIDE || (TS && !XR), "wide tiles: tensor-memory operand, streamed activations");
    constexpr int QROW = q_row_bytes(FMT);
    constexpr int QBYTES = 128 * QROW;                       // packed codes of one 128-row tile per K step
    constexpr bool AFFINE = FMT == FMT_A4 || FMT == FMT_A8 || FMT == FMT_A2;
    constexpr int XB = WIDE ? 2 * kXBytes : kXBytes;         // activation tile of a stage
    constexpr uint32_t Q_OFF = XR ? 0u : (uint32_t)(XB + (TS ? 0 : kWBytes));
    constexpr int NB = WIDE ? 1 : 2;                         // accumulator buffers
    constexpr int DCOLS = WIDE ? 256 : 128;                  // columns of one accumulator
    constexpr bool SPLIT = !WIDE;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    // [activation panel (XR)][stages][2 tiles' scale buffers][control block]
    Bars* bars = reinterpret_cast<Bars*>(base + (size_t)p.panel_bytes + (size_t)p.stages * p.stage_bytes + 2 * (size_t)p.sc_bytes);
    const uint32_t panel = smem_u32(base);
    const uint32_t sbase = panel + (uint32_t)p.panel_bytes;
    const uint32_t sc_base = sbase + (uint32_t)(p.stages * p.stage_bytes);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    volatile int* abort_flag = &bars->abort;
    const int stages = p.stages;

    if (tid == 0) {
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(smem_u32(&bars->qfull[s]), 1);
            mbar_init(smem_u32(&bars->full[s]), 4);
            mbar_init(smem_u32(&bars->empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bars->acc_full[b]), 1);
            mbar_init(smem_u32(&bars->acc_empty[b]), WIDE ? 8 : 4);
            mbar_init(smem_u32(&bars->sfull[b]), 1);
            mbar_init(smem_u32(&bars->sempty[b]), 8);
        }
        bars->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;

    if (warp == 0) {
        // ── MMA issuer ──────────────────────────────────────────────────────
        Ring r = {0, 0u};
        PROF_DECL
        for_each_tile<SWIGLU, XR, SPLIT>(a, p.nt_r, p.nt_x, [&](const TileInfo& t, int it) -> bool {
            const int buf = it % NB, round = it / NB;
            PROF_BEGIN
            if (!mbar_wait(smem_u32(&bars->acc_empty[buf]), (uint32_t)(round & 1) ^ 1u, abort_flag)) return false;
            PROF_END(0)
            tc_fence_after();
            const int ksteps = t.K / kTileK;
            const uint32_t idesc = idesc_for((t.rows + 15) & ~15);
            const uint32_t d = tmem + (uint32_t)(buf * DCOLS);
            for (int ks = 0; ks < ksteps; ++ks) {
                PROF_BEGIN
                if (!mbar_wait(smem_u32(&bars->full[r.s]), r.ph, abort_flag)) return false;
                PROF_END(1)
                tc_fence_after();
                PROF_BEGIN
                if (lane == 0) {
                    const uint32_t stage = sbase + (uint32_t)(r.s * p.stage_bytes);
                    const uint64_t dx = smem_desc(XR ? panel + (uint32_t)(ks * kXBytes) : stage);
#pragma unroll
                    for (int kk = 0; kk < kTileK / 16; ++kk) {
                        const uint32_t acc = (ks > 0 || kk > 0) ? 1u : 0u;
                        if (TS) umma_ts(d, tmem + kTmemA + (uint32_t)(r.s * 32 + kk * 8), dx + 2 * kk, idesc, acc);
                        else umma_ss(d, smem_desc(stage + XB) + 2 * kk, dx + 2 * kk, idesc, acc);
                    }
                    umma_commit(smem_u32(&bars->empty[r.s]));                // stage free once these MMAs retire
                    if (ks == ksteps - 1) umma_commit(smem_u32(&bars->acc_full[buf]));
                }
                __syncwarp();
                PROF_END(2)
                r.advance(1, stages);
            }
            return true;
        });
        PROF_FLUSH(0)
    } else if (warp == 2) {
        // ── loader (TMA): activation tile, packed codes, scales ─────────────
        Ring r = {0, 0u};
        PROF_DECL
        for_each_tile<SWIGLU, XR, SPLIT>(a, p.nt_r, p.nt_x, [&](const TileInfo& t, int it) -> bool {
            const int ksteps = t.K / kTileK;
            int mi0, mi1, row0, row1;
            tile_rows<SWIGLU>(a, t, t.ntile, mi0, mi1, row0, row1);
            const int sbuf = it & 1;
            PROF_BEGIN
            if (!mbar_wait(smem_u32(&bars->sempty[sbuf]), (uint32_t)((it >> 1) & 1) ^ 1u, abort_flag)) return false;
            PROF_END(0)
            if (lane == 0) {
                // bytes of one row of scales for this reduction length
                const uint32_t srow = (uint32_t)(t.K >> p.lg_group) * (AFFINE ? 2u : 1u);
                const uint32_t bar = smem_u32(&bars->sfull[sbuf]);
                const uint32_t dst = sc_base + (uint32_t)(sbuf * p.sc_bytes);
                mbar_expect_tx(bar, (AFFINE ? 4u : 2u) * 64u * srow);
                tma_load_2d(dst, &maps.s[mi0], 0, row0, bar);
                tma_load_2d(dst + 64 * srow, &maps.s[mi1], 0, row1, bar);
                if (AFFINE) {
                    tma_load_2d(dst + 128 * srow, &maps.b[mi0], 0, row0, bar);
                    tma_load_2d(dst + 192 * srow, &maps.b[mi1], 0, row1, bar);
                }
            }
            __syncwarp();
            // activation rows this tile needs: one box of 128 slots, a second one past 128 rows
            const bool two = WIDE && t.rows > 128;
            for (int ks = 0; ks < ksteps; ++ks) {
                PROF_BEGIN
                if (!mbar_wait(smem_u32(&bars->empty[r.s]), r.ph ^ 1u, abort_flag)) return false;
                PROF_END(1)
                if (lane == 0) {
                    const uint32_t bar = smem_u32(&bars->qfull[r.s]);
                    const uint32_t stage = sbase + (uint32_t)(r.s * p.stage_bytes);
                    // XR: the panel's chunk ks is loaded with the part's first tile; the MMAs that read the
                    // previous part's chunk retired before this stage's slot came free (stages <= K steps)
                    const bool with_x = !XR || t.first;
                    mbar_expect_tx(bar, (uint32_t)(QBYTES + (with_x ? (two ? 2 * kXBytes : kXBytes) : 0)));
                    if (with_x) {
                        const uint32_t xdst = XR ? panel + (uint32_t)(ks * kXBytes) : stage;
                        tma_load_2d(xdst, &maps.x, ks * kTileK, t.slot0, bar);
                        if (two) tma_load_2d(xdst + kXBytes, &maps.x, ks * kTileK, t.slot0 + 128, bar);
                    }
                    tma_load_2d(stage + Q_OFF, &maps.w[mi0], ks * QROW, row0, bar);
                    tma_load_2d(stage + Q_OFF + QBYTES / 2, &maps.w[mi1], ks * QROW, row1, bar);
                }
                __syncwarp();
                r.advance(1, stages);
            }
            return true;
        });
        PROF_FLUSH(1)
    } else if ((warp >= 4 && warp < 8) || warp >= 16) {
        // ── epilogue ────────────────────────────────────────────────────────
        const int q = warp & 3;                                 // tensor-memory lane quarter
        const int eh = warp >= 16 ? 1 : 0;                      // WIDE: which half of the tile's slots; else: which accumulator
        const int lane128 = q * 32 + lane;
        PROF_DECL
        for_each_tile<SWIGLU, XR, SPLIT>(a, p.nt_r, p.nt_x, [&](const TileInfo& t, int it) -> bool {
            const int buf = it % NB, round = it / NB;
            if (!WIDE && buf != eh) return true;                    // two accumulators: one set of four warps each
            const ExpertSet& S = a.set;
            // Per-row output factors (before the accumulator is waited for: global loads): nvfp4's tensor scale,
            // mxfp8's 2^(largest scale exponent of the row - 127).
            auto row_factor = [&](const QMat& m, size_t estride, int r_in) -> float {
                if (AFFINE) return 1.f;
                if (FMT == FMT_NVFP4) return m.global_scale;
                const int srow = t.K >> 5;                          // one ue8m0 byte per 32 values
                const uint8_t* sp = m.scales + (t.extra ? 0 : (size_t)t.expert * estride) + (size_t)r_in * srow;
                uint32_t mx = 0;
                for (int i = 0; i < srow; i += 16) mx = max_byte(__ldg(reinterpret_cast<const uint4*>(sp + i)), mx);
                return ue8m0_to_f32(hmax_bytes(mx));
            };
            float rf[4] = {1.f, 1.f, 1.f, 1.f};                     // first product: [lane group][gate, up]; second: [0]
            if (SWIGLU) {
#pragma unroll
                for (int gs = 0; gs < 2; ++gs) {
                    const int idx = t.ntile * 64 + (2 * q + gs) * 8 + (lane >> 2);
                    rf[2 * gs] = row_factor(t.extra ? S.x_gate : S.gate, S.gu_stride_s, idx);
                    rf[2 * gs + 1] = row_factor(t.extra ? S.x_up : S.up, S.gu_stride_s, idx);
                }
            } else {
                rf[0] = row_factor(t.extra ? S.x_down : S.down, S.dn_stride_s, t.ntile * 128 + lane128);
            }
            PROF_BEGIN
            if (!mbar_wait(smem_u32(&bars->acc_full[buf]), (uint32_t)(round & 1), abort_flag)) return false;
            PROF_END(0)
            tc_fence_after();
            PROF_BEGIN
            float peak = 0.f;                                       // largest magnitude this thread rounds to fp16 in the tile
            const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * DCOLS);
            auto release = [&]() {                                  // all of this warp's TMEM reads are done
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars->acc_empty[buf]));
            };
            if (SWIGLU) {
                // pieces of 64 slots x 16 lanes: 8 gate rows and the 8 matching up rows; a thread finishes row
                // lane/4 of the piece for the slots 8 j + 2 (lane % 4), +1
                const int n64 = (t.rows + 63) >> 6;
                const int c_lo = WIDE ? eh * 2 : 0, c_hi = WIDE ? min(n64, eh * 2 + 2) : n64;
                if (c_lo >= c_hi) release();
                for (int c = c_lo; c < c_hi; ++c) {
#pragma unroll
                    for (int gs = 0; gs < 2; ++gs) {
                        uint32_t v[32];
                        tmem_ld_16x64(taddr + ((uint32_t)(gs * 16) << 16) + (uint32_t)(c * 64), v);
                        if (c == c_hi - 1 && gs == 1) release();
                        uint32_t o[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            float g0 = __uint_as_float(v[4 * j]), g1 = __uint_as_float(v[4 * j + 1]);
                            float u0 = __uint_as_float(v[4 * j + 2]), u1 = __uint_as_float(v[4 * j + 3]);
                            if (!AFFINE) { g0 *= rf[2 * gs]; g1 *= rf[2 * gs]; u0 *= rf[2 * gs + 1]; u1 *= rf[2 * gs + 1]; }
                            const float r0 = silu_fast(g0) * u0, r1 = silu_fast(g1) * u1;
                            peak = fmaxf(peak, fmaxf(fabsf(r0), fabsf(r1)));
                            o[j] = pack_f16_sat(r0, r1);
                        }
                        const int col = t.ntile * 64 + (2 * q + gs) * 8 + (lane >> 2);
                        const int pos = (col & ~15) + (int)((p.pos_lut >> (4 * (col & 15))) & 0xf);
                        const int sl0 = c * 64 + 2 * (lane & 3);                 // first of this thread's slots
                        __half* dst = a.act + (size_t)(t.slot0 + sl0) * a.act_stride + pos;
                        const int n_ok = t.rows - sl0;
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            if (8 * j < n_ok) st_global_u16(dst + (size_t)(8 * j) * a.act_stride, o[j]);
                            if (8 * j + 1 < n_ok) st_global_u16(dst + (size_t)(8 * j + 1) * a.act_stride, o[j] >> 16);
                        }
                    }
                }
            } else {
                const int chunks = (t.rows + 31) >> 5;
                const int c_lo = WIDE ? eh * 4 : 0, c_hi = WIDE ? min(chunks, eh * 4 + 4) : chunks;
                if (c_lo >= c_hi) release();
                const int col = t.ntile * 128 + lane128;
                for (int c = c_lo; c < c_hi; ++c) {
                    uint32_t v[32];
                    tmem_ld32(taddr + c * 32, v);
                    if (c == c_hi - 1) release();
                    // the arithmetic first, for all 32 values and without a branch, then the stores under their
                    // row guards
                    float o[32];
                    if (a.row_scale != nullptr) {
                        // a weight per slot: one per lane, handed round by shuffle
                        const int my = c * 32 + lane;
                        const float rs = (my < t.rows ? a.row_scale[t.slot0 + my] : 1.f) * rf[0];
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __uint_as_float(v[i]) * __shfl_sync(0xffffffffu, rs, i);
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = AFFINE ? __uint_as_float(v[i]) : __uint_as_float(v[i]) * rf[0];
                    }
                    const size_t o0 = (size_t)(t.slot0 + c * 32) * a.set.n_in + col;
                    const int n_ok = t.rows - c * 32;
                    if (a.out16 != nullptr && a.out_index != nullptr) {
                        // rows scattered to the positions the caller names (expert parallelism: straight into the
                        // buffer the rows travel back in): one index per lane, handed round by shuffle
                        const int my = c * 32 + lane;
                        const int orow = my < t.rows ? a.out_index[t.slot0 + my] : 0;
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            peak = fmaxf(peak, fmaxf(fabsf(o[i]), fabsf(o[i + 1])));
                            const uint32_t h = pack_f16_sat(o[i], o[i + 1]);
                            const int r0 = __shfl_sync(0xffffffffu, orow, i), r1 = __shfl_sync(0xffffffffu, orow, i + 1);
                            if (i < n_ok) st_global_u16(a.out16 + (size_t)r0 * a.set.n_in + col, h);
                            if (i + 1 < n_ok) st_global_u16(a.out16 + (size_t)r1 * a.set.n_in + col, h >> 16);
                        }
                    } else if (a.out16 != nullptr) {
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            peak = fmaxf(peak, fmaxf(fabsf(o[i]), fabsf(o[i + 1])));
                            const uint32_t h = pack_f16_sat(o[i], o[i + 1]);
                            if (i < n_ok) st_global_u16(a.out16 + o0 + (size_t)i * a.set.n_in, h);
                            if (i + 1 < n_ok) st_global_u16(a.out16 + o0 + (size_t)(i + 1) * a.set.n_in, h >> 16);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (i < n_ok) a.out[o0 + (size_t)i * a.set.n_in] = o[i];
                    }
                }
            }
            // values beyond the fp16 range were clamped: counted (per thread and tile), never silent
            if (peak > 65504.f && a.status != nullptr) atomicAdd(a.status + kStatusSaturations, 1);
            PROF_END(1)
            return true;
        });
        if (warp == 4) { PROF_FLUSH(2) }
    } else if (warp >= 8 && warp < 16) {
        // ── producers ───────────────────────────────────────────────────────
        // two groups of four warps on alternating K steps; a thread owns one weight row of the tile
        const int grp_id = (warp - 8) >> 2;
        const int lane128 = tid - 256 - grp_id * 128;     // tensor-memory lane = (warp % 4) * 32 + lane
        const int qrow = tile_row_of_lane<SWIGLU>(lane128);
        const uint32_t swz = QROW == 32 ? ((uint32_t)qrow >> 2) & 1u : (QROW == 64 ? ((uint32_t)qrow >> 1) & 3u : 0u);
        const uint32_t q_off = Q_OFF + (uint32_t)qrow * QROW;
        const uint32_t t_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16) + kTmemA;
        // TS = false: this row's 128 bytes of the K-major swizzled weight tile
        const uint32_t w_off = (uint32_t)XB + (uint32_t)((lane128 >> 3) * 1024 + (lane128 & 7) * 128);
        Ring r = {0, 0u};
        r.advance(grp_id, stages);
        PROF_DECL
        for_each_tile<SWIGLU, XR, SPLIT>(a, p.nt_r, p.nt_x, [&](const TileInfo& t, int it) -> bool {
            const int ksteps = t.K / kTileK;
            const int sbuf = it & 1;
            const uint32_t srow = (uint32_t)(t.K >> p.lg_group) * (AFFINE ? 2u : 1u);
            const uint32_t s_addr = sc_base + (uint32_t)(sbuf * p.sc_bytes) + (uint32_t)qrow * srow;
            const uint32_t b_addr = s_addr + 128u * srow;
            PROF_BEGIN
            if (!mbar_wait(smem_u32(&bars->sfull[sbuf]), (uint32_t)((it >> 1) & 1), abort_flag)) return false;
            PROF_END(0)
            int r_exp = 0;
            if (FMT == FMT_MXFP8) {
                uint32_t mx = 0;
                for (uint32_t i = 0; i < srow; i += 16) mx = max_byte(lds128(s_addr + i), mx);
                r_exp = (int)hmax_bytes(mx);
            }
            int ks = grp_id;
            for (; ks < ksteps; ks += 2) {
                PROF_BEGIN
                if (!mbar_wait(smem_u32(&bars->qfull[r.s]), r.ph, abort_flag)) return false;
                PROF_END(1)
                PROF_BEGIN
                const uint32_t stage = sbase + (uint32_t)(r.s * p.stage_bytes);
                uint32_t out[32];
                if (AFFINE) {
                    __half2 sc[2], bi[2];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t gi = (uint32_t)(ks * kTileK + h * 32) >> p.lg_group;
                        sc[h] = bf16_to_half2(lds16(s_addr + gi * 2));
                        bi[h] = bf16_to_half2(lds16(b_addr + gi * 2));
                    }
                    if (FMT == FMT_A4) Dequant<FMT_A4>::run(stage + q_off, swz, sc, bi, out);
                    if (FMT == FMT_A8) Dequant<FMT_A8>::run(stage + q_off, swz, sc, bi, out);
                    if (FMT == FMT_A2) Dequant<FMT_A2>::run(stage + q_off, swz, sc, bi, out);
                } else if (FMT == FMT_MXFP8) {
                    const uint32_t s2 = lds16(s_addr + (uint32_t)ks * 2);
                    __half2 mult[2] = {pow2_half2((int)(s2 & 0xffu) - r_exp), pow2_half2((int)(s2 >> 8) - r_exp)};
                    Dequant<FMT_MXFP8>::run(stage + q_off, swz, mult, mult, out);
                } else {
                    Dequant<FMT_NVFP4>::run(stage + q_off, swz, lds32(s_addr + (uint32_t)ks * 4), out);
                }
                if (TS) {
                    tmem_st32(t_lane + (uint32_t)(r.s * 32), out);
                    tc_fence_before();
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const uint32_t dst = stage + w_off + (((uint32_t)j ^ (uint32_t)(lane128 & 7)) << 4);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(out[4 * j]), "r"(out[4 * j + 1]),
                                     "r"(out[4 * j + 2]), "r"(out[4 * j + 3])
                                     : "memory");
                    }
                    fence_async_proxy();                 // generic-proxy writes -> visible to the tensor-core reads
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars->full[r.s]));
                PROF_END(2)
                r.advance(2, stages);
            }
            // the ring position is now `ks` steps into this tile; this group's next step is `grp_id` steps
            // into the next one
            const int delta = ksteps + grp_id - ks;       // -1, 0 or 1
            if (delta > 0) r.advance(delta, stages);
            else if (delta < 0) r.advance(2 * stages + delta, stages);   // one step back: two turns minus one
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars->sempty[sbuf]));   // this warp is done with the tile's scales
            return true;
        });
        if (warp == 8) { PROF_FLUSH(3) }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
    if (tid == 0 && bars->abort && a.status != nullptr) atomicExch(a.status, 3);
}

}  // namespace

namespace {

int fmt_index(const QFormat& f) {
    if (f.mode == IMX_MODE_AFFINE) return f.bits == 4 ? FMT_A4 : (f.bits == 8 ? FMT_A8 : (f.bits == 2 ? FMT_A2 : -1));
    if (f.mode == IMX_MODE_MXFP8) return FMT_MXFP8;
    if (f.mode == IMX_MODE_NVFP4) return FMT_NVFP4;
    return -1;
}

int log2_exact(int v) {
    int l = 0;
    while ((1 << l) < v) ++l;
    return (1 << l) == v ? l : -1;
}

// bytes of one row of scales (K values) and the condition the copy engine puts on it
size_t scale_row(int K, const QFormat& f) { return (size_t)(K / f.group) * (f.mode == IMX_MODE_AFFINE ? 2 : 1); }
bool k_ok(int K, const QFormat& f) {
    if (K % kTileK || K % f.group) return false;
    const size_t sr = scale_row(K, f);
    return sr % 16 == 0 && K / f.group <= 256;
}

// packed codes + scales (+ biases) maps of one stacked quantized matrix [rows, K]
int make_q_maps(const QMat& m, size_t rows, int K, const QFormat& f, int fmt, CUtensorMap* w, CUtensorMap* sc, CUtensorMap* bi) {
    const int qrow = q_row_bytes(fmt);
    const size_t row_bytes = packed_row_bytes(K, f.bits);
    const int swz = qrow == 64 ? 64 : (qrow == 32 ? 32 : 0);
    IMX_TRY(make_tensor_map_2d(m.w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, rows, row_bytes, row_bytes, qrow, 64, false, w, false, swz));
    const int groups = K / f.group;
    if (f.mode == IMX_MODE_AFFINE) {
        IMX_TRY(make_tensor_map_2d(m.scales, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, rows, groups, (size_t)groups * 2, groups, 64, false, sc));
        IMX_TRY(make_tensor_map_2d(m.biases, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, rows, groups, (size_t)groups * 2, groups, 64, false, bi));
    } else {
        IMX_TRY(make_tensor_map_2d(m.scales, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, rows, groups, (size_t)groups, groups, 64, false, sc));
        *bi = *sc;
    }
    return IMX_OK;
}

template <int FMT>
int configure() {
    constexpr int kSmem = 227 * 1024;
    IMX_CHECK_CUDA(cudaFuncSetAttribute(prefill_tc_kernel<true, FMT, true, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
    IMX_CHECK_CUDA(cudaFuncSetAttribute(prefill_tc_kernel<true, FMT, true, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
    IMX_CHECK_CUDA(cudaFuncSetAttribute(prefill_tc_kernel<false, FMT, true, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
    IMX_CHECK_CUDA(cudaFuncSetAttribute(prefill_tc_kernel<false, FMT, true, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
    IMX_CHECK_CUDA(cudaFuncSetAttribute(prefill_tc_kernel<false, FMT, true, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
    IMX_CHECK_CUDA(cudaFuncSetAttribute(prefill_tc_kernel<true, FMT, false, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
    IMX_CHECK_CUDA(cudaFuncSetAttribute(prefill_tc_kernel<false, FMT, false, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
    return IMX_OK;
}

struct Plan {
    TcParams p;
    size_t smem;
    bool wide;
    bool xr;
};

template <int FMT>
int launch_fmt(const GroupedArgs& a, const Plan& gu, const Plan& dn, bool ts, const TcMaps& mgu, const TcMaps& mdn, int sms,
               cudaStream_t stream, cudaEvent_t mid) {
    if (!a.second_only) {
        if (!ts) prefill_tc_kernel<true, FMT, false, false, false><<<sms, kThreadsTc, gu.smem, stream>>>(a, gu.p, mgu);
        else if (gu.wide) prefill_tc_kernel<true, FMT, true, true, false><<<sms, kThreadsTc, gu.smem, stream>>>(a, gu.p, mgu);
        else prefill_tc_kernel<true, FMT, true, false, false><<<sms, kThreadsTc, gu.smem, stream>>>(a, gu.p, mgu);
        IMX_LAUNCHED();
        IMX_CHECK_CUDA(cudaGetLastError());
    }
    if (mid) IMX_CHECK_CUDA(cudaEventRecord(mid, stream));
    if (!ts) prefill_tc_kernel<false, FMT, false, false, false><<<sms, kThreadsTc, dn.smem, stream>>>(a, dn.p, mdn);
    else if (dn.wide) prefill_tc_kernel<false, FMT, true, true, false><<<sms, kThreadsTc, dn.smem, stream>>>(a, dn.p, mdn);
    else if (dn.xr) prefill_tc_kernel<false, FMT, true, false, true><<<sms, kThreadsTc, dn.smem, stream>>>(a, dn.p, mdn);
    else prefill_tc_kernel<false, FMT, true, false, false><<<sms, kThreadsTc, dn.smem, stream>>>(a, dn.p, mdn);
    IMX_LAUNCHED();
    IMX_CHECK_CUDA(cudaGetLastError());
    return IMX_OK;
}

}  // namespace

#ifdef IMX_TC_PROFILE
extern "C" IMX_API int imx_debug_tc_prof(unsigned long long* out32) {
    return cudaMemcpyFromSymbol(out32, g_tc_prof, sizeof(unsigned long long) * 32) == cudaSuccess ? 0 : 2;
}
#endif

bool prefill_tc_supported(const ExpertSet& s, bool second_only) {
    const QFormat& f = s.fmt;
    if (fmt_index(f) < 0) return false;
    if (log2_exact(f.group) < 0 || f.group > 128 || f.group < 16) return false;
    if (f.mode == IMX_MODE_AFFINE && f.group < 32) return false;
    if (s.n_in % 128 || s.n_mid % 64) return false;
    // the second product alone never reduces over n_in (a plain quantized matmul with any number of output rows)
    if ((!second_only && !k_ok(s.n_in, f)) || !k_ok(s.n_mid, f)) return false;
    if (s.has_extra && (s.x_mid % 64 || !k_ok(s.x_mid, f))) return false;
    return true;
}

// variant: 0 = the shipped configuration (tensor-memory operand, 256-slot tiles in both products), 1 =
// tensor-memory operand, 128-slot tiles and streamed activations everywhere, 2 = as 1 with the dequantized
// tile in shared memory (1, 2: cross-checks).
int launch_prefill_tc(const GroupedArgs& a, cudaStream_t stream, cudaEvent_t mid, int variant) {
    IMX_REQUIRE(prefill_tc_supported(a.set, a.second_only != 0), "prefill path: format/shape not supported");
    IMX_REQUIRE((a.row_index == nullptr || a.xs != nullptr || a.second_only) && a.n_slots > 0,
                "prefill path: slot-ordered activation buffer missing");
    if (a.max_units == 0) return IMX_OK;
    const ExpertSet& s = a.set;
    const QFormat& f = s.fmt;
    const int fmt = fmt_index(f);
    const bool ts = variant != 2;
    const int x_mid = s.has_extra ? s.x_mid : s.n_mid;
    const int mid_max = s.n_mid > x_mid ? s.n_mid : x_mid;
    const int mid_min = s.n_mid < x_mid ? s.n_mid : x_mid;

    DeviceInfo di;
    IMX_TRY(current_device(&di));
    if (device_needs_setup(di.ordinal, kSetupPrefillTc)) {   // once per device, outside any stream capture (first call)
        IMX_TRY(configure<FMT_A4>());
        IMX_TRY(configure<FMT_A8>());
        IMX_TRY(configure<FMT_A2>());
        IMX_TRY(configure<FMT_MXFP8>());
        IMX_TRY(configure<FMT_NVFP4>());
        device_mark_setup(di.ordinal, kSetupPrefillTc);
    }

    // Shared memory of a launch: [panel][stages][two scale buffers][control block].  As many stages as fit,
    // at most 8 (the ring of A tiles in tensor memory has 256 columns) and, with a resident panel, at most
    // the shortest reduction's K steps (the ring's back-pressure then also guards the panel).
    const size_t q_tile = 128u * (size_t)q_row_bytes(fmt);
    auto plan = [&](int K_max, int K_min, bool wide, bool xr, Plan* out) -> bool {
        const size_t sc = (size_t)128 * scale_row(K_max, f) * (f.mode == IMX_MODE_AFFINE ? 2 : 1);
        const size_t panel = xr ? (size_t)(K_max / kTileK) * kXBytes : 0;
        const size_t stage = (xr ? 0 : (size_t)kXBytes * (wide ? 2 : 1) + (ts ? 0 : kWBytes)) + q_tile;
        const size_t fixed = panel + 2 * sc + sizeof(Bars) + 1024;
        const size_t room = 227 * 1024;
        if (fixed + 2 * stage > room) return false;
        int st = (int)((room - fixed) / stage);
        if (st > kMaxStages) st = kMaxStages;
        if (xr && st > K_min / kTileK) st = K_min / kTileK;
        if (st < 2) return false;
        out->p = TcParams{};
        out->p.stages = st;
        out->p.stage_bytes = (int)stage;
        out->p.sc_bytes = (int)sc;
        out->p.panel_bytes = (int)panel;
        out->p.lg_group = log2_exact(f.group);
        out->smem = fixed + (size_t)st * stage;
        out->wide = wide;
        out->xr = xr;
        return true;
    };
    Plan gu = {}, dn = {};
    if (!a.second_only && !(variant == 0 && plan(s.n_in, s.n_in, true, false, &gu)))
        IMX_REQUIRE(plan(s.n_in, s.n_in, false, false, &gu), "prefill path: sizes exceed shared memory");
    // second product: 256-slot tiles with streamed activations as well (c3: 276 us against 377 us with 128-slot
    // tiles and the activation panel resident); the resident panel where the wide stages do not fit
    if (!(variant == 0 && (plan(mid_max, mid_min, true, false, &dn) || plan(mid_max, mid_min, false, true, &dn))))
        IMX_REQUIRE(plan(mid_max, mid_min, false, false, &dn), "prefill path: sizes exceed shared memory");
    gu.p.nt_r = s.n_mid / 64;
    gu.p.nt_x = x_mid / 64;
    dn.p.nt_r = dn.p.nt_x = s.n_in / 128;
    // where the first product's epilogue puts output column i of a block of 16: the order the second
    // product's weights are unpacked in
    int order[16];
    expert_block_order(f, order);
    unsigned long long lut = 0;
    for (int pos = 0; pos < 16; ++pos) lut |= (unsigned long long)pos << (4 * order[pos]);
    gu.p.pos_lut = dn.p.pos_lut = lut;

    // activations in sorted-slot order (the `take_axis` of moe.rs:124-127, once for all experts)
    const __half* xsrc = a.in;                     // already slot-ordered when there is no row index
    if (a.row_index != nullptr && !a.second_only) {
        IMX_TRY(launch_gather_rows(a.in, a.row_index, a.n_slots, (size_t)s.n_in * 2, a.xs, stream, a.slots_end_dev, a.slots_resume));
        xsrc = a.xs;
    }
    TcMaps mgu, mdn;
    std::memset(&mgu, 0, sizeof(mgu));
    if (!a.second_only)
    IMX_TRY(make_tensor_map_2d(xsrc, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (size_t)a.n_slots, (size_t)s.n_in, (size_t)s.n_in * 2, kTileK,
                               128, true, &mgu.x));
    IMX_TRY(make_tensor_map_2d(a.act, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (size_t)a.n_slots, (size_t)mid_max, (size_t)a.act_stride * 2,
                               kTileK, 128, true, &mdn.x));
    // routed experts: gate and up rows live in one stacked matrix [E*2I, H]; down in [E*H, I]
    if (!a.second_only) IMX_TRY(make_q_maps(s.gate, (size_t)s.num_experts * 2 * s.n_mid, s.n_in, f, fmt, &mgu.w[0], &mgu.s[0], &mgu.b[0]));
    IMX_TRY(make_q_maps(s.down, (size_t)s.num_experts * s.n_in, s.n_mid, f, fmt, &mdn.w[0], &mdn.s[0], &mdn.b[0]));
    if (s.has_extra) {
        if (!a.second_only) {
            IMX_TRY(make_q_maps(s.x_gate, (size_t)s.x_mid, s.n_in, f, fmt, &mgu.w[1], &mgu.s[1], &mgu.b[1]));
            IMX_TRY(make_q_maps(s.x_up, (size_t)s.x_mid, s.n_in, f, fmt, &mgu.w[2], &mgu.s[2], &mgu.b[2]));
        }
        IMX_TRY(make_q_maps(s.x_down, (size_t)s.n_in, s.x_mid, f, fmt, &mdn.w[1], &mdn.s[1], &mdn.b[1]));
    } else {
        mgu.w[1] = mgu.w[2] = mgu.w[0]; mgu.s[1] = mgu.s[2] = mgu.s[0]; mgu.b[1] = mgu.b[2] = mgu.b[0];
        mdn.w[1] = mdn.w[0]; mdn.s[1] = mdn.s[0]; mdn.b[1] = mdn.b[0];
    }
    mdn.w[2] = mdn.w[1]; mdn.s[2] = mdn.s[1]; mdn.b[2] = mdn.b[1];

    switch (fmt) {
        case FMT_A4: return launch_fmt<FMT_A4>(a, gu, dn, ts, mgu, mdn, di.sms, stream, mid);
        case FMT_A8: return launch_fmt<FMT_A8>(a, gu, dn, ts, mgu, mdn, di.sms, stream, mid);
        case FMT_A2: return launch_fmt<FMT_A2>(a, gu, dn, ts, mgu, mdn, di.sms, stream, mid);
        case FMT_MXFP8: return launch_fmt<FMT_MXFP8>(a, gu, dn, ts, mgu, mdn, di.sms, stream, mid);
        case FMT_NVFP4: return launch_fmt<FMT_NVFP4>(a, gu, dn, ts, mgu, mdn, di.sms, stream, mid);
    }
    set_error("prefill path: unknown format");
    return IMX_ERR_INVALID;
}

}  // namespace imx
