// Decode-regime grouped expert products, tensor-map fed kernels (affine 4-bit,
// group 64).  Same arithmetic as the other decode kernels (exact integer codes
// on the fp16 tensor-core path, fp32 fold with scale and bias per group),
// written for instruction count: a warp gets through its instructions about as
// fast as HBM delivers its stages, and whichever is slower sets the pace.
//
//   * a stage (16 weight rows x 512 codes + their 8 scales and 8 biases per row)
//     arrives with four tiled TMA copies issued by one lane: two 128-byte-wide
//     swizzled boxes of packed codes and one 16-byte-wide box each of scales and
//     biases, all completing on the stage's mbarrier.  Nothing about a stage
//     passes through registers before it is used.
//   * weight row r of a tile sits on MMA row r/2 + 8*(r&1): with the 128-byte
//     swizzle the 8-byte fragment loads of a half-warp then cover all 32 banks.
//   * a 4-bit code becomes an fp16 operand with one AND: left in the low mantissa
//     bits of a half-word whose exponent field is zero it IS the subnormal
//     q * 2^-24 (codes at bits [0,4)) or q * 2^-20 (codes at bits [4,8)).  No
//     offset has to be added and none cancelled.  The two classes are levelled on
//     the activation side: the fp16 activation rows these kernels read hold the
//     values that meet a [4,8) code (odd reduction index) divided by 16 (exact
//     down to 2^-10; Order16::pair_scale_odd).  The fold per group is
//     acc += s*D + b*sum(x) with everything in units of 2^-24, and the epilogue
//     multiplies by 2^24.
//   * sum(x) * 2^-24 per (row, group): for the first product a table written by the
//     router (or by group_sums_kernel); for the second, the first product's
//     epilogue leaves the sum of every 16 columns it writes (per slot), and a warp
//     adds four of them per group into shared memory when it reaches a unit.
//   * activations and table entries of the next 128 codes are loaded while the
//     current 128 are multiplied (register double buffer), across stage
//     boundaries too.
//
// The two products hand out their work differently (measured per warp with
// time stamps on the c2 step: a stage takes 2.0 us +- 25 % under load, so equal
// shares leave the slowest of 2368 warps a fifth behind the mean):
//   * first product: equal contiguous shares of the (unit, tile pair, stage)
//     sequence, a pair cut across warps finished by the warp that owns its first
//     stage (decode_first_kernel).  The warps of a CTA then read the same unit's
//     activation rows -- per stage as many bytes as the weights -- from L1
//     (85 % hits); chunks handed out through a counter balance the warps but
//     scatter the units over the SMs, and the L1 misses cost more than the
//     balance gains (75 against 63 us).
//   * second product: chunks through a counter (decode_second_kernel); its
//     activation rows are a quarter as long, and the launch went from 41 to 38 us.
// Every wait is bounded.
#include <cuda.h>

#include <atomic>
#include <cstring>

#include "decode_common.cuh"

namespace imx {

namespace {

using namespace decode;

constexpr int kStageCodes = 256;               // codes per row per stage, for both tiles of a pair
constexpr int kWBytes = 2 * 16 * 128;          // packed codes of a stage: one box of 16 rows x 128 bytes per tile
constexpr int kSBytes = 4 * 16 * 16;           // scales, biases of tile 0, then of tile 1: 16 rows x 8 groups x 2 bytes
// shared memory of a CTA of `warps` warps with `stages` stages each: codes | scales+biases | barriers (+ slack to
// align the base to 1024 bytes)
constexpr int kMaxSumGroups = 64;              // second product: groups of 64 per SwiGLU row (intermediate <= 4096)
// `sum_groups`: row length of the per-warp table of group sums (0: no table, first product)
constexpr size_t smem_bytes(int warps, int stages, int sum_groups) {
    return (size_t)warps * stages * (kWBytes + kSBytes + 8) + (size_t)warps * 8 * sum_groups * 4 + 1024;
}
constexpr int kSpinLimit = 1 << 20;
constexpr int kFlagSpinLimit = 1 << 22;
constexpr float kUnscale = 16777216.f;         // 2^24: the accumulators are in units of 2^-24
// Per-warp time stamps, compiled in only for timing experiments (-DIMX_DEC_PROFILE).
#ifdef IMX_DEC_PROFILE
__device__ unsigned long long g_dec_prof[2][kFlagWarps][8];
__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define DPROF(i) if (lane == 0) g_dec_prof[kProfWhich][gw][i] = (i) == 0 || (i) == 7 ? gtime() : (unsigned long long)clock64();
#define DPROF_ADD(i, v) if (lane == 0) g_dec_prof[kProfWhich][gw][i] += (unsigned long long)(v);
#define DPROF_SET(i, v) if (lane == 0) g_dec_prof[kProfWhich][gw][i] = (unsigned long long)(v);
#else
#define DPROF(i)
#define DPROF_ADD(i, v)
#define DPROF_SET(i, v)
#endif
std::atomic<int> g_flag_spin_limit{kFlagSpinLimit};
std::atomic<int> g_withhold_flags{0};

// [0] the routed experts' stacked matrix, [1]/[2] the extra expert's matrix for tile 0 / tile 1 of a pair
struct DecodeMaps {
    CUtensorMap w[3];
    CUtensorMap s[3];
    CUtensorMap b[3];
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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
// Tiled TMA copy with an L2 eviction-priority hint.
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar, uint64_t policy) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
                 ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(x), "r"(y), "l"(policy)
                 : "memory");
}
template <int OFF>
__device__ __forceinline__ void lds64(uint32_t addr, uint32_t (&v)[2]) {
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+%3];" : "=r"(v[0]), "=r"(v[1]) : "r"(addr), "n"(OFF));
}
template <int OFF>
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF));
    return v;
}
// first MMA of a chain: accumulator input is zero
// Loads that stay where they are written (ahead of the shared-memory loads and MMAs of the previous
// 128 codes), so that their latency is covered.
__device__ __forceinline__ uint4 ldg128_early(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void mma_f16_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    const float z = 0.f;
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(z));
}

// Unpack of a word of eight 4-bit codes into fp16 subnormals: the nibbles at bits
// [0,4) of each half-word are q * 2^-24 as they stand, those at bits [4,8) are
// q * 2^-20.  MMA m of a 16-code block takes r0 = codes (J, J+4) (reduction
// indices 0..7 of the MMA) and r1 = codes (J+1, J+5) (indices 8..15).
template <int M>
__device__ __forceinline__ void frag2(const uint32_t (&w)[2], uint32_t& r0, uint32_t& r1) {
    const uint32_t v = (M & 1) ? (w[M >> 1] >> 8) : w[M >> 1];
    r0 = v & 0x000f000fu;
    r1 = v & 0x00f000f0u;
}

// Sum of every group of 64 values of a row of fp16 activations, in units of 2^-24:
// out[slot, j] = 2^-24 * sum(x[row(slot), 64 j .. 64 j + 63]), fixed order, fp32.  The rows are in the
// expert kernels' layout: pairs 1 and 3 of every 8 stored values hold x / 16.
__global__ void group_sums_kernel(const __half* __restrict__ in, const int32_t* __restrict__ row_index, int n_slots,
                                  int groups, int ld, float* __restrict__ out, const int32_t* __restrict__ n_rows_dev) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (n_rows_dev != nullptr ? min(n_slots, *n_rows_dev) : n_slots) * groups) return;
    const int slot = idx / groups, j = idx - slot * groups;
    const int row = row_index ? row_index[slot] : slot;
    const uint4* p = reinterpret_cast<const uint4*>(in + (size_t)row * ld + (size_t)j * 64);
    float lo = 0.f, hi = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint4 v = __ldg(p + i);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
            if (e & 1) hi += f.x + f.y;
            else lo += f.x + f.y;
        }
    }
    out[idx] = (lo + 16.f * hi) * 5.9604644775390625e-8f;   // 2^-24
}

// Position in the launch's stage sequence: routed units first, then the extra expert's units; within a
// unit tile pair after tile pair, within a pair stage after stage.
struct Cursor {
    int unit, pair, st, extra;
};


// ── first product: equal contiguous shares ──────────────────────────────────
// The (unit, tile pair, stage) sequence of the launch is split into contiguous ranges, one per warp; a pair cut
// across warps is finished by the warp that owns its first stage, the others hand their fp32 partial sums over
// through the workspace.  Neighbouring warps of a CTA then work on the same unit, whose activation rows (as much
// data per stage as the weights) stay in L1: handing the work out in chunks, as the second product does, costs
// this kernel more in L1 misses than it gains in balance.  Every wait is bounded.
template <int kWarps, int kStages>
__global__ void __launch_bounds__(kWarps * 32, 1)
decode_first_kernel(const GroupedArgs a, const int ppu_r, const int ppu_x, const int st_r, const int st_x,
                   const int flag_base, const int sum_groups, const int flag_spin_limit, const int withhold_flags,
                   const __grid_constant__ DecodeMaps maps) {
    constexpr int kSmemW = kWarps * kStages * kWBytes, kSmemS = kWarps * kStages * kSBytes;
    extern __shared__ unsigned char smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);   // known to be warp-uniform
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t wbuf = sbase + (uint32_t)warp * (kStages * kWBytes);
    const uint32_t sbuf = sbase + kSmemW + (uint32_t)warp * (kStages * kSBytes);
    const uint32_t bars = sbase + kSmemW + kSmemS + (uint32_t)warp * (kStages * 8);

    const int n_r = a.n_units[1];
    const int stages_r = n_r * ppu_r * st_r;
    const int total = stages_r + (a.n_units[0] - n_r) * ppu_x * st_x;

    const int gw = blockIdx.x * kWarps + warp;
    const int nw = gridDim.x * kWarps;
    // Equal shares of the sequence, with a stage of the extra expert counted as 5/4 of a routed one: its weights
    // are read by every one of its units at about the same time, and those stages take a fifth longer.
    const long long weighted = 4ll * stages_r + 5ll * (total - stages_r);
    auto range_lo = [&](int w) {
        const long long u = (long long)w * weighted / nw;
        return u <= 4ll * stages_r ? (int)(u / 4) : stages_r + (int)((u - 4ll * stages_r) / 5);
    };
    const int sig_lo = range_lo(gw), sig_hi = range_lo(gw + 1);
    if (sig_lo >= sig_hi) return;
#ifdef IMX_DEC_PROFILE
    constexpr int kProfWhich = 1;
#endif
    DPROF(0) DPROF(1) DPROF_SET(5, 0) DPROF_SET(6, sig_hi - sig_lo)
    int32_t* flags = a.sched + flag_base;
    float* my_slot = a.partials + (size_t)gw * 256;

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kStages; ++s) mbar_init(bars + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();

    const ExpertSet& S = a.set;

    // where the range starts (the only divisions of the kernel); both cursors advance stage by stage from here
    Cursor start;
    {
        int local = sig_lo, ppu = ppu_r, st = st_r, unit0 = 0;
        start.extra = 0;
        if (sig_lo >= stages_r) {
            local = sig_lo - stages_r;
            ppu = ppu_x;
            st = st_x;
            unit0 = n_r;
            start.extra = 1;
        }
        const int task = local / st;
        start.st = local - task * st;
        start.unit = unit0 + task / ppu;
        start.pair = task - (task / ppu) * ppu;
    }
    // one stage forward; true when a new tile pair begins
    auto advance = [&](Cursor& c) -> bool {
        if (++c.st < (c.extra ? st_x : st_r)) return false;
        c.st = 0;
        if (++c.pair == (c.extra ? ppu_x : ppu_r)) {
            c.pair = 0;
            if (++c.unit == n_r) c.extra = 1;
        }
        return true;
    };

    // ── fetch side (warp-uniform; lane 0 issues the copies) ─────────────────
    Cursor fc = start;
    int f_sigma = sig_lo, f_unit = -1, f_expert = 0;
    int f_map0 = 0, f_map1 = 0, f_row0 = 0, f_row1 = 0;
    bool f_first = true;                // the first stage of the range fetches scales whatever its parity
    auto fetch_rows = [&]() {           // rows of the pair's two tiles in their tensor maps
        if (fc.unit != f_unit) {
            f_unit = fc.unit;
            f_expert = a.units[fc.unit].expert;
        }
        if (fc.extra) {
            f_map0 = 1;
            f_map1 = 2;
            f_row0 = f_row1 = fc.pair * 16;
        } else {
            f_map0 = f_map1 = 0;
            f_row0 = f_expert * 2 * S.n_mid + fc.pair * 16;
            f_row1 = f_row0 + S.n_mid;
        }
    };
    fetch_rows();
    int n_fetch = 0, n_sfetch = 0;
    auto issue = [&]() {
        const bool with_scales = !(fc.st & 1) || f_first;   // a 16-byte row of scales serves two stages
        if (lane == 0) {
            const int slot = n_fetch % kStages;
            const uint32_t bar = bars + 8 * slot;
            const uint32_t wdst = wbuf + slot * kWBytes;
            mbar_expect_tx(bar, with_scales ? kWBytes + kSBytes : kWBytes);
            // weights, scales and biases are read once per step: first in line for eviction, so that the
            // stream does not push the activations, sums and hand-off slots out of L2 (8 % of the c2 step)
            uint64_t policy;
            asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
            tma_load_2d_hint(wdst, &maps.w[f_map0], fc.st * 128, f_row0, bar, policy);
            tma_load_2d_hint(wdst + 2048, &maps.w[f_map1], fc.st * 128, f_row1, bar, policy);
            if (with_scales) {
                const uint32_t sdst = sbuf + (n_sfetch % kStages) * kSBytes;
                const int xs = (fc.st >> 1) * 8;
                tma_load_2d_hint(sdst, &maps.s[f_map0], xs, f_row0, bar, policy);
                tma_load_2d_hint(sdst + 256, &maps.b[f_map0], xs, f_row0, bar, policy);
                tma_load_2d_hint(sdst + 512, &maps.s[f_map1], xs, f_row1, bar, policy);
                tma_load_2d_hint(sdst + 768, &maps.b[f_map1], xs, f_row1, bar, policy);
            }
        }
        if (with_scales) ++n_sfetch;
        f_first = false;
        ++n_fetch;
        ++f_sigma;
        if (advance(fc) && f_sigma < sig_hi) fetch_rows();
    };

    // ── compute side ────────────────────────────────────────────────────────
    Cursor cc = start;
    int c_sigma = sig_lo;
    int c_st_lo = start.st;             // stage of its pair at which the current piece began
    int c_unit = -1, c_rows = 0, c_slot0 = 0;
    const __half* c_act = nullptr;      // this lane's activation row (slot g of the unit, clamped to a valid slot)
    const float* c_sum_a = nullptr;     // group sums of slots 2t and 2t+1 (clamped likewise)
    const float* c_sum_b = nullptr;
    auto setup_unit = [&]() {
        c_unit = cc.unit;
        const WorkUnit u = a.units[cc.unit];
        c_rows = u.rows;
        c_slot0 = u.slot0;
        const int last = u.rows - 1;
        const int sl = u.slot0 + (g < last ? g : last);
        const int sa = u.slot0 + (2 * t < last ? 2 * t : last), sb = u.slot0 + (2 * t + 1 < last ? 2 * t + 1 : last);
        // rows of `in` (and of its table of group sums) behind the slots
        const int row = a.row_index ? a.row_index[sl] : sl;
        const int ra = a.row_index ? a.row_index[sa] : sa, rb = a.row_index ? a.row_index[sb] : sb;
        c_act = a.in + (size_t)row * S.n_in + t * 16;
        c_sum_a = a.gsum_x + (size_t)ra * sum_groups;
        c_sum_b = a.gsum_x + (size_t)rb * sum_groups;
    };
    // the first copies leave before the unit's set-up, which then runs under their latency
#pragma unroll
    for (int s = 0; s < kStages - 1; ++s)
        if (f_sigma < sig_hi) issue();
    setup_unit();
    float acc[2][4];
#pragma unroll
    for (int T = 0; T < 2; ++T)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[T][i] = 0.f;

    // Finishes the piece that ends with the stage just computed (stage cc.st of pair cc.pair).
    auto finish_piece = [&]() -> bool {
        const int st_n = cc.extra ? st_x : st_r;
        if (c_st_lo > 0) {
            // not the owner: hand the partial sums to the warp that owns the pair's first stage
#pragma unroll
            for (int T = 0; T < 2; ++T)
#pragma unroll
                for (int i = 0; i < 4; ++i) my_slot[(T * 4 + i) * 32 + lane] = acc[T][i];
            __threadfence();
            __syncwarp();
            if (lane == 0 && !withhold_flags) *reinterpret_cast<volatile int32_t*>(flags + gw) = 1;
        } else {
            if (cc.st + 1 < st_n) {
                // owner of a pair that was cut: add the partials of the following warps, in warp order
                const int sigma_end = c_sigma - (cc.st + 1) + st_n;   // one past the pair's last stage
                int covered = sig_hi;
                for (int w = gw + 1; covered < sigma_end && w < nw; ++w) {
                    if (range_lo(w + 1) == range_lo(w)) continue;   // a warp without work raises no flag
                    int ok = 1;
                    if (lane == 0) {
                        int spin = 0;
                        while (*reinterpret_cast<volatile int32_t*>(flags + w) == 0) {
                            if (++spin > flag_spin_limit) {
                                ok = 0;
                                break;
                            }
                            __nanosleep(64);
                        }
                    }
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) {
                        if (lane == 0 && a.status != nullptr) atomicExch(a.status, 2);
                        return false;
                    }
                    __threadfence();
                    const float* slot = a.partials + (size_t)w * 256;
#pragma unroll
                    for (int T = 0; T < 2; ++T)
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            acc[T][i] += *reinterpret_cast<const volatile float*>(slot + (T * 4 + i) * 32 + lane);
                    covered = range_lo(w + 1);
                }
            }
            // accumulator i of a tile: weight row 2g + (i >> 1) of the tile, slot 2t + (i & 1) of the unit
            {
                float sum_a = 0.f, sum_b = 0.f;                        // over the pair's 16 columns: slot 2t, slot 2t+1
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int slot_l = 2 * t + (i & 1);
                    const int row = cc.pair * 16 + 2 * g + (i >> 1);
                    float v = silu_f(acc[0][i] * kUnscale) * (acc[1][i] * kUnscale);
                    if (row & 1) v *= 0.0625f;                                 // meets a [4,8) code in the second product
                    const __half h = f32_to_f16_sat(v, slot_l < c_rows ? a.status : nullptr);
                    const float back = __half2float(h) * ((row & 1) ? 16.f : 1.f);
                    if (i & 1) sum_b += back;
                    else sum_a += back;
                    if (slot_l < c_rows) {
                        const int col = (row & ~15) + permuted_pos<4>(row & 15);   // the order the second product reads
                        a.act[(size_t)(c_slot0 + slot_l) * a.act_stride + col] = h;
                    }
                }
                // what the second product needs of these columns besides their values: their sum per slot
#pragma unroll
                for (int d = 4; d < 32; d <<= 1) {
                    sum_a += __shfl_xor_sync(0xffffffffu, sum_a, d);
                    sum_b += __shfl_xor_sync(0xffffffffu, sum_b, d);
                }
                if (g == 0) {
                    float* ps = a.psum + (size_t)(c_slot0 + 2 * t) * (a.act_stride >> 4) + cc.pair;
                    if (2 * t < c_rows) ps[0] = sum_a;
                    if (2 * t + 1 < c_rows) ps[a.act_stride >> 4] = sum_b;
                }
            }
        }
#pragma unroll
        for (int T = 0; T < 2; ++T)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[T][i] = 0.f;
        return true;
    };

    // lane constants of the swizzled fragment loads: row 2g of a box, 8 bytes at (t & 1) * 8 of the
    // 16-byte piece ((t >> 1) ^ row) -- the row below it is the same address ^ 144
    const uint32_t lane_w = (uint32_t)g * 256u + (uint32_t)(t & 1) * 8u + ((((uint32_t)t >> 1) ^ ((2u * g) & 7u)) << 4);
    const uint32_t lane_s = (uint32_t)g * 32u;

    int n_comp = 0, n_scomp = 0;
    uint32_t c_sslot = 0;                                // shared-memory offset of the scales the stage reads
    bool c_first = true;
    uint32_t bf[2][8];                                   // activations of 64 codes: [2 m + r] for MMA m
    float sxa[4], sxb[4];                                // group sums of the stage's 4 groups: slot 2t, slot 2t+1
    // activations of step j (64 codes) of the stage the compute cursor is at
    auto load_step = [&](int buf, int j) {
        const uint4* p = reinterpret_cast<const uint4*>(c_act + (size_t)cc.st * kStageCodes) + j * 8;
        const uint4 v0 = ldg128_early(p), v1 = ldg128_early(p + 1);
        bf[buf][0] = v0.x; bf[buf][1] = v0.y; bf[buf][2] = v0.z; bf[buf][3] = v0.w;
        bf[buf][4] = v1.x; bf[buf][5] = v1.y; bf[buf][6] = v1.z; bf[buf][7] = v1.w;
    };
    auto load_sums = [&]() {
        uint4 va, vb;
        va = ldg128_early(reinterpret_cast<const uint4*>(c_sum_a + cc.st * 4));
        vb = ldg128_early(reinterpret_cast<const uint4*>(c_sum_b + cc.st * 4));
        sxa[0] = __uint_as_float(va.x); sxa[1] = __uint_as_float(va.y); sxa[2] = __uint_as_float(va.z); sxa[3] = __uint_as_float(va.w);
        sxb[0] = __uint_as_float(vb.x); sxb[1] = __uint_as_float(vb.y); sxb[2] = __uint_as_float(vb.z); sxb[3] = __uint_as_float(vb.w);
    };
    load_sums();
    load_step(0, 0);
    DPROF(2)
#pragma unroll 1
    while (c_sigma < sig_hi) {
        if (f_sigma < sig_hi) issue();                   // refills the slot that was consumed last

        const int slot = n_comp % kStages;
        if (!(cc.st & 1) || c_first) {
            c_sslot = (uint32_t)(n_scomp % kStages) * kSBytes;
            ++n_scomp;
        }
        c_first = false;
        {
            const uint32_t bar = bars + 8 * slot;
            const uint32_t parity = (uint32_t)(n_comp / kStages) & 1u;
            int spin = 0;
            while (!mbar_try_wait(bar, parity)) {
                if (++spin > kSpinLimit) {
                    if (a.status != nullptr) atomicExch(a.status, 1);
                    return;
                }
            }
        }
#ifdef IMX_DEC_PROFILE
        if (n_comp == 0) { DPROF(3) }
#endif
        const uint32_t wst = wbuf + (uint32_t)slot * kWBytes + lane_w;
        const uint32_t sst = sbuf + c_sslot + lane_s + (uint32_t)(cc.st & 1) * 8u;   // groups 4 (st & 1) .. + 3 of the row
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int cur = j & 1;
            if (j < 3) load_step(cur ^ 1, j + 1);
            const uint32_t alo = wst ^ (uint32_t)(j * 32), ahi = alo ^ 144u;
            const float xa = sxa[j], xb = sxb[j];
#pragma unroll
            for (int T = 0; T < 2; ++T) {
                uint32_t wlo[2], whi[2];
                if (T == 0) { lds64<0>(alo, wlo); lds64<0>(ahi, whi); }
                else { lds64<2048>(alo, wlo); lds64<2048>(ahi, whi); }
                // scales / biases of groups (j & ~1), (j | 1) for weight rows 2g (lo) and 2g+1 (hi) of tile T
                uint32_t sc_lo, sc_hi, bi_lo, bi_hi;
                if (T == 0 && j < 2) { sc_lo = lds32<0>(sst); sc_hi = lds32<16>(sst); bi_lo = lds32<256>(sst); bi_hi = lds32<272>(sst); }
                if (T == 0 && j >= 2) { sc_lo = lds32<4>(sst); sc_hi = lds32<20>(sst); bi_lo = lds32<260>(sst); bi_hi = lds32<276>(sst); }
                if (T == 1 && j < 2) { sc_lo = lds32<512>(sst); sc_hi = lds32<528>(sst); bi_lo = lds32<768>(sst); bi_hi = lds32<784>(sst); }
                if (T == 1 && j >= 2) { sc_lo = lds32<516>(sst); sc_hi = lds32<532>(sst); bi_lo = lds32<772>(sst); bi_hi = lds32<788>(sst); }
                const uint32_t* b = bf[cur];
                float d[4];
                uint32_t a0, a1, a2, a3;
                frag2<0>(wlo, a0, a2); frag2<0>(whi, a1, a3);
                mma_f16_z(d, a0, a1, a2, a3, b[0], b[1]);
                frag2<1>(wlo, a0, a2); frag2<1>(whi, a1, a3);
                mma_f16(d, a0, a1, a2, a3, b[2], b[3]);
                frag2<2>(wlo, a0, a2); frag2<2>(whi, a1, a3);
                mma_f16(d, a0, a1, a2, a3, b[4], b[5]);
                frag2<3>(wlo, a0, a2); frag2<3>(whi, a1, a3);
                mma_f16(d, a0, a1, a2, a3, b[6], b[7]);
                // d = 2^-24 * sum of q * x over the group; fold with the group's scale and bias
                const float s_lo = __uint_as_float((j & 1) ? (sc_lo & 0xffff0000u) : (sc_lo << 16));
                const float s_hi = __uint_as_float((j & 1) ? (sc_hi & 0xffff0000u) : (sc_hi << 16));
                const float b_lo = __uint_as_float((j & 1) ? (bi_lo & 0xffff0000u) : (bi_lo << 16));
                const float b_hi = __uint_as_float((j & 1) ? (bi_hi & 0xffff0000u) : (bi_hi << 16));
                acc[T][0] = fmaf(s_lo, d[0], fmaf(b_lo, xa, acc[T][0]));
                acc[T][1] = fmaf(s_lo, d[1], fmaf(b_lo, xb, acc[T][1]));
                acc[T][2] = fmaf(s_hi, d[2], fmaf(b_hi, xa, acc[T][2]));
                acc[T][3] = fmaf(s_hi, d[3], fmaf(b_hi, xb, acc[T][3]));
            }
        }
        __syncwarp();          // every lane is done reading this slot before it is refilled
        ++n_comp;
        ++c_sigma;
        const bool pair_done = cc.st + 1 == (cc.extra ? st_x : st_r);
        if (pair_done || c_sigma == sig_hi) {
            if (!finish_piece()) return;
            c_st_lo = 0;       // every piece after the first starts with its pair
        }
        advance(cc);
        if (c_sigma < sig_hi) {
            if (cc.unit != c_unit) setup_unit();
            load_sums();       // first 64 codes and the sums of the next stage
            load_step(0, 0);
        }
    }
    DPROF(4) DPROF(7)
}

// ── second product: chunks handed out through a counter ─────────────────────
__device__ __forceinline__ WorkUnit load_unit(const WorkUnit* u) {
    const int4 v = __ldg(reinterpret_cast<const int4*>(u));
    WorkUnit w;
    w.expert = v.x;
    w.slot0 = v.y;
    w.rows = v.z;
    w.pad = v.w;
    return w;
}

// What a launch needs besides the arguments of the product.
struct DecodeParams {
    int ppu_r, ppu_x;        // tile pairs per unit: routed experts, extra expert
    int st_r, st_x;          // stages per tile pair
    int pairs_a;             // coarse chunks: this many whole tile pairs of a routed unit each (divides ppu_r)
    int chunk;               // fine chunks: this many stages of one tile pair (divides st_r)
    int fine_pairs;          // the last so many tile pairs of the routed units go out as fine chunks
    int sum_groups;          // row length of the table of group sums (first product: the router's; second: the warp's)
    int ctr;                 // word of `sched` that hands out this launch's chunks
    int cut;                 // chunks per pair the hand-off buffers are laid out for (row length of pair_partials)
    int spin_limit;          // bound of the wait for a stage's copies
};

// One chunk of a launch's work: whole tile pairs of one unit, or part of the reduction of one pair.
struct Chunk {
    int id;                  // position in the launch's chunk order
    int unit, pair;          // unit and (first) tile pair of the unit
    int pairs;               // whole pairs in the chunk (parts == 1)
    int sub, parts;          // which part of the pair's reduction, of how many
    int extra;
    int slot;                // parts > 1: the pair's hand-off slot
};

template <int kWarps, int kStages>
__global__ void __launch_bounds__(kWarps * 32, 1)
decode_second_kernel(const GroupedArgs a, const DecodeParams p, const __grid_constant__ DecodeMaps maps) {
    constexpr int kSmemW = kWarps * kStages * kWBytes, kSmemS = kWarps * kStages * kSBytes;
    extern __shared__ unsigned char smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);   // known to be warp-uniform
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t wbuf = sbase + (uint32_t)warp * (kStages * kWBytes);
    const uint32_t sbuf = sbase + kSmemW + (uint32_t)warp * (kStages * kSBytes);
    const uint32_t bars = sbase + kSmemW + kSmemS + (uint32_t)warp * (kStages * 8);
    // group sums of the unit's SwiGLU rows, [8 slots][sum_groups]
    const uint32_t sums = sbase + kSmemW + kSmemS + kWarps * kStages * 8 + (uint32_t)warp * (uint32_t)(8 * p.sum_groups * 4);

    // The launch's work goes out in chunks through a counter: warp w starts with chunk w, every further one is
    // the counter's next.  (Warps drift apart -- the stream is bound by HBM and a stage's latency varies by a
    // quarter -- so equal static shares leave the slowest warp a fifth behind the mean.)  Order: the extra
    // expert's tile pairs (the slowest per stage), then the routed units' pairs, coarse chunks of whole pairs
    // first and, for the end of the launch, fine chunks of a few stages, so that all warps finish within a
    // few stages of one another.  A pair cut into fine chunks is put together by whichever of them is last.
    const int n_r = a.n_units[1], n_x = a.n_units[0] - n_r;
    const int C = p.chunk;
    const int parts_b = p.st_r / C;
    const int pairs_r = n_r * p.ppu_r;
    int fine = p.fine_pairs < pairs_r ? p.fine_pairs : pairs_r;
    const int chunks_a = (pairs_r - fine) / p.pairs_a;
    fine = pairs_r - chunks_a * p.pairs_a;
    const int chunks_x = n_x * p.ppu_x;
    const int first_b = chunks_x + chunks_a;
    const int n_chunks = first_b + fine * parts_b;
    const int gw = blockIdx.x * kWarps + warp;
    const int nw = gridDim.x * kWarps;
    if (gw >= n_chunks) return;
#ifdef IMX_DEC_PROFILE
    constexpr int kProfWhich = 0;
#endif
    DPROF(0) DPROF(1) DPROF_SET(5, 0) DPROF_SET(6, 0)
    int32_t* ctr = a.sched + p.ctr;

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kStages; ++s) mbar_init(bars + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();

    const ExpertSet& S = a.set;

    auto decode_chunk = [&](int id) -> Chunk {
        Chunk k;
        k.id = id;
        k.extra = 0;
        k.pairs = 1;
        k.sub = 0;
        k.parts = 1;
        k.slot = 0;
        int q;                                   // pair among the routed units' pairs
        if (id < chunks_x) {
            const int u = id / p.ppu_x;
            k.extra = 1;
            k.pair = id - u * p.ppu_x;
            k.unit = n_r + u;
            return k;
        } else if (id < first_b) {
            q = (id - chunks_x) * p.pairs_a;
            k.pairs = p.pairs_a;
        } else {
            const int l = id - first_b;
            k.slot = l / parts_b;
            k.sub = l - k.slot * parts_b;
            k.parts = parts_b;
            q = chunks_a * p.pairs_a + k.slot;
        }
        k.unit = q / p.ppu_r;
        k.pair = q - k.unit * p.ppu_r;
        return k;
    };

    // ── fetch side (warp-uniform; lane 0 issues the copies) ─────────────────
    Chunk fk = decode_chunk(gw);
    WorkUnit f_unit = load_unit(a.units + fk.unit);
    int f_pair = 0, f_st = 0, f_st_end = 0, f_left = 0;   // pair and stage the next copies are for; end of the pair's part; stages left in the chunk
    auto fetch_enter = [&]() {          // the fetch side enters chunk fk
        const int st = fk.extra ? p.st_x : p.st_r;
        f_pair = fk.pair;
        f_st = fk.parts > 1 ? fk.sub * C : 0;
        f_st_end = fk.parts > 1 ? f_st + C : st;
        f_left = fk.parts > 1 ? C : fk.pairs * st;
    };
    fetch_enter();
    bool f_more = true;                 // chunks may be left
    int f_map0 = 0, f_map1 = 0, f_row0 = 0, f_row1 = 0;
    int ticket = 0;                     // lane 0: the counter's answer for the chunk after fk (asked for ahead of its use)
    auto ask = [&]() {
        if (lane == 0) ticket = atomicAdd(ctr, 1);
    };
    auto fetch_rows = [&]() {           // rows of the pair's two tiles in their tensor maps
        f_map0 = f_map1 = fk.extra ? 1 : 0;
        f_row0 = (fk.extra ? 0 : f_unit.expert * S.n_in) + f_pair * 32;
        f_row1 = f_row0 + 16;
    };
    int n_fetch = 0, n_sfetch = 0;
    auto issue = [&]() {
        const bool with_scales = !(f_st & 1);               // a 16-byte row of scales serves two stages; parts start even
        if (lane == 0) {
            const int slot = n_fetch % kStages;
            const uint32_t bar = bars + 8 * slot;
            const uint32_t wdst = wbuf + slot * kWBytes;
            mbar_expect_tx(bar, with_scales ? kWBytes + kSBytes : kWBytes);
            // The routed experts' weights, scales and biases are read once per step: first in line for
            // eviction, so that the stream does not push the activations, sums and hand-off slots out of L2
            // (8 % of the c2 step).  The extra expert's are read again by every one of its units: kept.
            uint64_t policy;
            if (fk.extra) asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
            else asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
            tma_load_2d_hint(wdst, &maps.w[f_map0], f_st * 128, f_row0, bar, policy);
            tma_load_2d_hint(wdst + 2048, &maps.w[f_map1], f_st * 128, f_row1, bar, policy);
            if (with_scales) {
                const uint32_t sdst = sbuf + (n_sfetch % kStages) * kSBytes;
                const int xs = (f_st >> 1) * 8;
                tma_load_2d_hint(sdst, &maps.s[f_map0], xs, f_row0, bar, policy);
                tma_load_2d_hint(sdst + 256, &maps.b[f_map0], xs, f_row0, bar, policy);
                tma_load_2d_hint(sdst + 512, &maps.s[f_map1], xs, f_row1, bar, policy);
                tma_load_2d_hint(sdst + 768, &maps.b[f_map1], xs, f_row1, bar, policy);
            }
        }
        if (with_scales) ++n_sfetch;
        ++n_fetch;
        --f_left;
        if (++f_st == f_st_end && f_left > 0) {             // on to the chunk's next pair
            ++f_pair;
            f_st = 0;
            fetch_rows();
        }
    };
    // the fetch side moves on to the counter's next chunk; false when the launch has none left
    auto fetch_next_chunk = [&]() -> bool {
        const int id = nw + __shfl_sync(0xffffffffu, ticket, 0);
        if (id >= n_chunks) return false;
        fk = decode_chunk(id);
        f_unit = load_unit(a.units + fk.unit);
        fetch_enter();
        fetch_rows();
        ask();
        return true;
    };

    // ── compute side ────────────────────────────────────────────────────────
    Chunk ck = fk;
    WorkUnit c_unit = f_unit;
    int c_pair = f_pair, c_st = f_st, c_st_end = f_st_end;   // pair and stage being computed; end of the pair's part
    int c_pairs_left = ck.pairs;
    int c_setup_unit = -1;
    const __half* c_act = nullptr;      // this lane's activation row (slot g of the unit, clamped to a valid slot)
    uint32_t c_sums_a = 0, c_sums_b = 0; // group sums of slots 2t and 2t+1 (clamped likewise) in this warp's shared-memory table
    float c_rs0 = 1.f, c_rs1 = 1.f;     // output scale of slots 2t, 2t+1
    auto setup_unit = [&]() {
        c_setup_unit = ck.unit;
        const WorkUnit& u = c_unit;
        const int last = u.rows - 1;
        const int sl = u.slot0 + (g < last ? g : last);
        const int sa = u.slot0 + (2 * t < last ? 2 * t : last), sb = u.slot0 + (2 * t + 1 < last ? 2 * t + 1 : last);
        {
            c_act = a.act + (size_t)sl * a.act_stride + t * 16;
            if (a.row_scale != nullptr) {
                c_rs0 = a.row_scale[sa];
                c_rs1 = a.row_scale[sb];
            }
            // Group sums of the unit's rows, in units of 2^-24, into the warp's table, from the sums of every
            // 16 columns the first product left (a group of 64 = four of them, added in column order): lane L
            // takes slot L / 4 and every fourth group from L % 4.
            const int groups = (ck.extra ? S.x_mid : S.n_mid) >> 6;
            __syncwarp();
            if (g < u.rows) {
                const float* row = a.psum + (size_t)(u.slot0 + g) * (a.act_stride >> 4);
                for (int grp = t; grp < groups; grp += 4) {
                    const float4 q = *reinterpret_cast<const float4*>(row + grp * 4);
                    const float v = (((q.x + q.y) + q.z) + q.w) * 5.9604644775390625e-8f;   // 2^-24
                    asm volatile("st.shared.f32 [%0], %1;" ::"r"(sums + (uint32_t)(g * p.sum_groups + grp) * 4u), "f"(v) : "memory");
                }
            }
            __syncwarp();
            c_sums_a = sums + (uint32_t)((sa - u.slot0) * p.sum_groups) * 4u;
            c_sums_b = sums + (uint32_t)((sb - u.slot0) * p.sum_groups) * 4u;
        }
    };
    // the first copies leave before the unit's set-up, which then runs under their latency
    fetch_rows();
    ask();
#pragma unroll
    for (int s = 0; s < kStages - 1; ++s)
        if (f_left > 0) issue();
    setup_unit();
    float acc[2][4];
#pragma unroll
    for (int T = 0; T < 2; ++T)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[T][i] = 0.f;

    // The accumulators of a pair (or of the chunk's part of it) are complete: with the whole reduction in one
    // chunk they are the result; else the chunk leaves them in the pair's hand-off slot and the chunk of the
    // pair that arrives last adds all of them up, in the order of the parts whoever it is.  Nobody waits.
    auto finish_pair = [&]() {
        const int cut = ck.parts;
        if (cut > 1) {
            float* slots = a.pair_partials + (size_t)ck.slot * p.cut * 256;
            float* mine = slots + ck.sub * 256;
#pragma unroll
            for (int T = 0; T < 2; ++T)
#pragma unroll
                for (int i = 0; i < 4; ++i) __stcg(mine + (T * 4 + i) * 32 + lane, acc[T][i]);
            __threadfence();
            __syncwarp();
            int arrived = 0;
            if (lane == 0) arrived = atomicAdd(a.pair_count + ck.slot, 1);
            arrived = __shfl_sync(0xffffffffu, arrived, 0);
            if (arrived != cut - 1) return;
            __threadfence();
            if (lane == 0) a.pair_count[ck.slot] = 0;                  // as the next launch expects it
#pragma unroll
            for (int T = 0; T < 2; ++T)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[T][i] = 0.f;
            for (int s = 0; s < cut; ++s)
#pragma unroll
                for (int T = 0; T < 2; ++T)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[T][i] += __ldcg(slots + s * 256 + (T * 4 + i) * 32 + lane);
        }
        // accumulator i of a tile: weight row 2g + (i >> 1) of the tile, slot 2t + (i & 1) of the unit
        {
#pragma unroll
            for (int T = 0; T < 2; ++T)
#pragma unroll
                for (int sl = 0; sl < 2; ++sl) {
                    // rows 2g and 2g+1 of the tile are neighbours in the output row of slot 2t + sl
                    const int slot_l = 2 * t + sl;
                    const int row = c_pair * 32 + T * 16 + 2 * g;
                    const float sc = kUnscale * (sl ? c_rs1 : c_rs0);
                    if (slot_l < c_unit.rows)
                        *reinterpret_cast<float2*>(a.out + (size_t)(c_unit.slot0 + slot_l) * S.n_in + row) =
                            make_float2(acc[T][sl] * sc, acc[T][2 + sl] * sc);
                }
        }
    };

    // lane constants of the swizzled fragment loads: row 2g of a box, 8 bytes at (t & 1) * 8 of the
    // 16-byte piece ((t >> 1) ^ row) -- the row below it is the same address ^ 144
    const uint32_t lane_w = (uint32_t)g * 256u + (uint32_t)(t & 1) * 8u + ((((uint32_t)t >> 1) ^ ((2u * g) & 7u)) << 4);
    const uint32_t lane_s = (uint32_t)g * 32u;

    int n_comp = 0, n_scomp = 0;
    uint32_t c_sslot = 0;                                // shared-memory offset of the scales the stage reads
    uint32_t bf[2][8];                                   // activations of 64 codes: [2 m + r] for MMA m
    float sxa[4], sxb[4];                                // group sums of the stage's 4 groups: slot 2t, slot 2t+1
    // activations of step j (64 codes) of the stage the compute side is at
    auto load_step = [&](int buf, int j) {
        const uint4* q = reinterpret_cast<const uint4*>(c_act + (size_t)c_st * kStageCodes) + j * 8;
        const uint4 v0 = ldg128_early(q), v1 = ldg128_early(q + 1);
        bf[buf][0] = v0.x; bf[buf][1] = v0.y; bf[buf][2] = v0.z; bf[buf][3] = v0.w;
        bf[buf][4] = v1.x; bf[buf][5] = v1.y; bf[buf][6] = v1.z; bf[buf][7] = v1.w;
    };
    auto load_sums = [&]() {
        uint4 va, vb;
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(va.x), "=r"(va.y), "=r"(va.z), "=r"(va.w) : "r"(c_sums_a + (uint32_t)c_st * 16u));
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(vb.x), "=r"(vb.y), "=r"(vb.z), "=r"(vb.w) : "r"(c_sums_b + (uint32_t)c_st * 16u));
        sxa[0] = __uint_as_float(va.x); sxa[1] = __uint_as_float(va.y); sxa[2] = __uint_as_float(va.z); sxa[3] = __uint_as_float(va.w);
        sxb[0] = __uint_as_float(vb.x); sxb[1] = __uint_as_float(vb.y); sxb[2] = __uint_as_float(vb.z); sxb[3] = __uint_as_float(vb.w);
    };
    load_sums();
    load_step(0, 0);
    DPROF(2)
#pragma unroll 1
    while (true) {
        // refill the slot that was consumed last; past the end of a chunk the copies are the next chunk's
        if (f_left == 0 && f_more) f_more = fetch_next_chunk();
        if (f_left > 0) issue();

        const int slot = n_comp % kStages;
        if (!(c_st & 1)) {
            c_sslot = (uint32_t)(n_scomp % kStages) * kSBytes;
            ++n_scomp;
        }
        {
            const uint32_t bar = bars + 8 * slot;
            const uint32_t parity = (uint32_t)(n_comp / kStages) & 1u;
            int spin = 0;
            while (!mbar_try_wait(bar, parity)) {
                if (++spin > p.spin_limit) {
                    if (a.status != nullptr) atomicExch(a.status, 1);
                    return;
                }
            }
        }
#ifdef IMX_DEC_PROFILE
        if (n_comp == 0) { DPROF(3) }
#endif
        const uint32_t wst = wbuf + (uint32_t)slot * kWBytes + lane_w;
        const uint32_t sst = sbuf + c_sslot + lane_s + (uint32_t)(c_st & 1) * 8u;   // groups 4 (st & 1) .. + 3 of the row
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int cur = j & 1;
            if (j < 3) load_step(cur ^ 1, j + 1);
            const uint32_t alo = wst ^ (uint32_t)(j * 32), ahi = alo ^ 144u;
            const float xa = sxa[j], xb = sxb[j];
#pragma unroll
            for (int T = 0; T < 2; ++T) {
                uint32_t wlo[2], whi[2];
                if (T == 0) { lds64<0>(alo, wlo); lds64<0>(ahi, whi); }
                else { lds64<2048>(alo, wlo); lds64<2048>(ahi, whi); }
                // scales / biases of groups (j & ~1), (j | 1) for weight rows 2g (lo) and 2g+1 (hi) of tile T
                uint32_t sc_lo, sc_hi, bi_lo, bi_hi;
                if (T == 0 && j < 2) { sc_lo = lds32<0>(sst); sc_hi = lds32<16>(sst); bi_lo = lds32<256>(sst); bi_hi = lds32<272>(sst); }
                if (T == 0 && j >= 2) { sc_lo = lds32<4>(sst); sc_hi = lds32<20>(sst); bi_lo = lds32<260>(sst); bi_hi = lds32<276>(sst); }
                if (T == 1 && j < 2) { sc_lo = lds32<512>(sst); sc_hi = lds32<528>(sst); bi_lo = lds32<768>(sst); bi_hi = lds32<784>(sst); }
                if (T == 1 && j >= 2) { sc_lo = lds32<516>(sst); sc_hi = lds32<532>(sst); bi_lo = lds32<772>(sst); bi_hi = lds32<788>(sst); }
                const uint32_t* b = bf[cur];
                float d[4];
                uint32_t a0, a1, a2, a3;
                frag2<0>(wlo, a0, a2); frag2<0>(whi, a1, a3);
                mma_f16_z(d, a0, a1, a2, a3, b[0], b[1]);
                frag2<1>(wlo, a0, a2); frag2<1>(whi, a1, a3);
                mma_f16(d, a0, a1, a2, a3, b[2], b[3]);
                frag2<2>(wlo, a0, a2); frag2<2>(whi, a1, a3);
                mma_f16(d, a0, a1, a2, a3, b[4], b[5]);
                frag2<3>(wlo, a0, a2); frag2<3>(whi, a1, a3);
                mma_f16(d, a0, a1, a2, a3, b[6], b[7]);
                // d = 2^-24 * sum of q * x over the group; fold with the group's scale and bias
                const float s_lo = __uint_as_float((j & 1) ? (sc_lo & 0xffff0000u) : (sc_lo << 16));
                const float s_hi = __uint_as_float((j & 1) ? (sc_hi & 0xffff0000u) : (sc_hi << 16));
                const float b_lo = __uint_as_float((j & 1) ? (bi_lo & 0xffff0000u) : (bi_lo << 16));
                const float b_hi = __uint_as_float((j & 1) ? (bi_hi & 0xffff0000u) : (bi_hi << 16));
                acc[T][0] = fmaf(s_lo, d[0], fmaf(b_lo, xa, acc[T][0]));
                acc[T][1] = fmaf(s_lo, d[1], fmaf(b_lo, xb, acc[T][1]));
                acc[T][2] = fmaf(s_hi, d[2], fmaf(b_hi, xa, acc[T][2]));
                acc[T][3] = fmaf(s_hi, d[3], fmaf(b_hi, xb, acc[T][3]));
            }
        }
        __syncwarp();          // every lane is done reading this slot before it is refilled
        ++n_comp;
        DPROF_ADD(6, 1)
        if (++c_st == c_st_end) {
            finish_pair();
#pragma unroll
            for (int T = 0; T < 2; ++T)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[T][i] = 0.f;
            if (--c_pairs_left > 0) {                        // the chunk's next pair
                ++c_pair;
                c_st = 0;
            } else {
                if (fk.id == ck.id) break;                   // the fetch side found no further chunk
                ck = fk;                                     // the chunk whose first stage is on its way
                c_unit = f_unit;
                c_pair = ck.pair;
                c_st = ck.parts > 1 ? ck.sub * C : 0;
                c_st_end = ck.parts > 1 ? c_st + C : (ck.extra ? p.st_x : p.st_r);
                c_pairs_left = ck.pairs;
                if (ck.unit != c_setup_unit) setup_unit();
            }
        }
        load_sums();           // first 64 codes and the sums of the next stage
        load_step(0, 0);
    }
    DPROF(4) DPROF(7)
}

}  // namespace

#ifdef IMX_DEC_PROFILE
extern "C" IMX_API int imx_debug_dec_prof(unsigned long long* out, int which) {
    return cudaMemcpyFromSymbol(out, g_dec_prof, sizeof(unsigned long long) * kFlagWarps * 8,
                                sizeof(unsigned long long) * kFlagWarps * 8 * (which ? 1 : 0)) == cudaSuccess ? 0 : 2;
}
#endif

// Test hook (include/ironmlx_b200_testing.h): a short limit on the first product's hand-off wait and flags that
// are never raised make the wait run out, so that the path from an expired wait to the status word can be
// exercised without hanging or faulting anything.
void testing_decode_handoff(int spin_limit, int withhold) {
    g_flag_spin_limit.store(spin_limit > 0 ? spin_limit : kFlagSpinLimit);
    g_withhold_flags.store(withhold ? 1 : 0);
}

bool decode_tmap_supported(const ExpertSet& s) {
    const QFormat& f = s.fmt;
    if (f.mode != IMX_MODE_AFFINE || f.bits != 4 || f.group != 64) return false;
    if (s.n_in % 512 || s.n_mid % 512) return false;
    if (s.has_extra && s.x_mid % 512) return false;
    if (s.n_mid > 64 * kMaxSumGroups || (s.has_extra && s.x_mid > 64 * kMaxSumGroups)) return false;
    return true;
}

// Stages per fine chunk of a reduction of `stages` stages (even): four where they divide it, at most four
// chunks per tile pair.
static int chunk_stages(int stages) {
    int c = stages % 4 == 0 ? 4 : 2;
    while (stages / c > 4 && stages % (2 * c) == 0) c *= 2;
    return c;
}

TmapRoom decode_tmap_room(int n_in, int n_mid, int x_mid) {
    TmapRoom r = {0, 1};
    if (n_in <= 0 || n_mid <= 0 || n_in % 512 || n_mid % 512 || (x_mid > 0 && x_mid % 512)) return r;
    const int st_gu = n_in / kStageCodes, st_dn = n_mid / kStageCodes;
    const int cut_gu = st_gu / chunk_stages(st_gu), cut_dn = st_dn / chunk_stages(st_dn);
    r.cut = cut_gu > cut_dn ? cut_gu : cut_dn;
    r.pair_slots = r.cut > 1 ? kTmapFinePairs : 0;
    return r;
}

namespace {

int make_maps(const QMat& m, size_t rows, int K, CUtensorMap* w, CUtensorMap* sc, CUtensorMap* bi) {
    const size_t groups = (size_t)K / 64;
    IMX_TRY(make_tensor_map_2d(m.w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, rows, (size_t)K / 2, (size_t)K / 2, 128, 16, true, w));
    IMX_TRY(make_tensor_map_2d(m.scales, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, rows, groups, groups * 2, 8, 16, false, sc));
    IMX_TRY(make_tensor_map_2d(m.biases, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, rows, groups, groups * 2, 8, 16, false, bi));
    return IMX_OK;
}

template <int kWarps, int kStages>
int launch_with(const GroupedArgs& a, const DecodeMaps& gu, const DecodeMaps& dn, const DeviceInfo& di, cudaStream_t stream,
                cudaEvent_t mid) {
    const ExpertSet& s = a.set;
    const int sms = di.sms;
    if (device_needs_setup(di.ordinal, kSetupDecodeTmap)) {      // once per device, outside any stream capture
        constexpr int most = (int)smem_bytes(kWarps, kStages, kMaxSumGroups);
        IMX_CHECK_CUDA(cudaFuncSetAttribute(decode_first_kernel<kWarps, kStages>, cudaFuncAttributeMaxDynamicSharedMemorySize, most));
        IMX_CHECK_CUDA(cudaFuncSetAttribute(decode_second_kernel<kWarps, kStages>, cudaFuncAttributeMaxDynamicSharedMemorySize, most));
        device_mark_setup(di.ordinal, kSetupDecodeTmap);
    }
    const int grid = sms;
    const int x_mid = s.has_extra ? s.x_mid : s.n_mid;
    const int mid_max = s.n_mid > x_mid ? s.n_mid : x_mid;
    const int g_in = s.n_in / 64, g_mid = mid_max / 64;
    // shared memory: the rings, plus (second product) a table of group sums as wide as the rows need, so that
    // what is not used stays with the L1 cache
    const size_t smem_gu = smem_bytes(kWarps, kStages, 0), smem_dn = smem_bytes(kWarps, kStages, g_mid);
    // Second product's chunks: whole tile pairs first; the last two or so chunks of every warp a few stages
    // each, where the hand-off buffers have room for their pairs (else single whole pairs).
    const int st_dn_r = s.n_mid / kStageCodes, st_dn_x = x_mid / kStageCodes, ppu_dn = s.n_in / 32;
    const int nw = grid * kWarps;
    const bool room = a.pair_count != nullptr && a.pair_partials != nullptr && a.pair_slots > 0;
    DecodeParams pd = {};
    pd.ppu_r = pd.ppu_x = ppu_dn;
    pd.st_r = st_dn_r;
    pd.st_x = st_dn_x;
    pd.pairs_a = st_dn_r <= 4 && ppu_dn % 2 == 0 ? 2 : 1;       // short reductions: two pairs per coarse chunk
    pd.chunk = chunk_stages(st_dn_r);
    int parts = st_dn_r / pd.chunk;
    if (parts > 1 && !(room && parts <= a.pair_cut)) {
        pd.chunk = st_dn_r;
        parts = 1;
    }
    pd.fine_pairs = 2 * nw / parts;
    if (parts > 1 && pd.fine_pairs > a.pair_slots) pd.fine_pairs = a.pair_slots;
    pd.cut = a.pair_cut > 0 ? a.pair_cut : 1;
    pd.sum_groups = g_mid;
    pd.ctr = 3;
    pd.spin_limit = kSpinLimit;
    if (!a.second_only) {
        if (!a.gsum_x_ready) {
            // first product: group sums of the input rows (unless the router wrote them)
            const int n = a.n_in_rows * g_in;
            group_sums_kernel<<<(n + 255) / 256, 256, 0, stream>>>(a.in, nullptr, a.n_in_rows, g_in, s.n_in, a.gsum_x,
                                                                 a.n_rows_dev); IMX_LAUNCHED();
            IMX_CHECK_CUDA(cudaGetLastError());
        }
        int grid_gu = grid;
        if (grid_gu * kWarps > kFlagWarps) grid_gu = kFlagWarps / kWarps;
        decode_first_kernel<kWarps, kStages><<<grid_gu, kWarps * 32, smem_gu, stream>>>(
            a, s.n_mid / 16, x_mid / 16, s.n_in / kStageCodes, s.n_in / kStageCodes, 8, g_in, g_flag_spin_limit.load(),
            g_withhold_flags.load(), gu); IMX_LAUNCHED();
        IMX_CHECK_CUDA(cudaGetLastError());
    }
    if (mid) IMX_CHECK_CUDA(cudaEventRecord(mid, stream));
    // second product: the group sums of a unit's SwiGLU rows come from the sums of 16 the first product left
    decode_second_kernel<kWarps, kStages><<<grid, kWarps * 32, smem_dn, stream>>>(a, pd, dn); IMX_LAUNCHED();
    IMX_CHECK_CUDA(cudaGetLastError());
    return IMX_OK;
}

}  // namespace

int launch_decode_tmap(const GroupedArgs& a, cudaStream_t stream, cudaEvent_t mid) {
    IMX_REQUIRE(decode_tmap_supported(a.set), "decode (tensor-map) path: format/shape not supported");
    IMX_REQUIRE(a.psum != nullptr && a.partials != nullptr && a.sched != nullptr && (a.gsum_x != nullptr || a.second_only) && a.n_slots > 0 &&
                    (a.n_in_rows > 0 || a.second_only),
                "decode (tensor-map) path: workspace buffers missing");
    if (a.max_units == 0) return IMX_OK;
    const ExpertSet& s = a.set;
    DeviceInfo di;
    IMX_TRY(current_device(&di));
    DecodeMaps gu, dn;
    if (!a.second_only) IMX_TRY(make_maps(s.gate, (size_t)s.num_experts * 2 * s.n_mid, s.n_in, &gu.w[0], &gu.s[0], &gu.b[0]));
    else std::memset(&gu, 0, sizeof(gu));
    IMX_TRY(make_maps(s.down, (size_t)s.num_experts * s.n_in, s.n_mid, &dn.w[0], &dn.s[0], &dn.b[0]));
    if (s.has_extra) {
        if (!a.second_only) {
            IMX_TRY(make_maps(s.x_gate, (size_t)s.x_mid, s.n_in, &gu.w[1], &gu.s[1], &gu.b[1]));
            IMX_TRY(make_maps(s.x_up, (size_t)s.x_mid, s.n_in, &gu.w[2], &gu.s[2], &gu.b[2]));
        }
        IMX_TRY(make_maps(s.x_down, (size_t)s.n_in, s.x_mid, &dn.w[1], &dn.s[1], &dn.b[1]));
    } else {
        gu.w[1] = gu.w[2] = gu.w[0]; gu.s[1] = gu.s[2] = gu.s[0]; gu.b[1] = gu.b[2] = gu.b[0];
        dn.w[1] = dn.w[0]; dn.s[1] = dn.s[0]; dn.b[1] = dn.b[0];
    }
    dn.w[2] = dn.w[1]; dn.s[2] = dn.s[1]; dn.b[2] = dn.b[1];
    // 16 warps x 2 stages: measured best on B200 against 12 x 3, 14 x 3 and 20 x 2 (which spills at 96 registers)
    return launch_with<16, 2>(a, gu, dn, di, stream, mid);
}

}  // namespace imx
