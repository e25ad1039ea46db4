// Decode-regime grouped expert products, TMA-pipelined stream-K variant
// (affine 4-bit, group 64/128).  Same arithmetic as decode_mma.cu (exact
// integer codes on the fp16 tensor-core path, one all-ones MMA per 16 codes
// for the group sums, fold with scale and bias per group in fp32); what
// differs is how the bytes move and how the work is cut:
//
//   * the packed weights reach the SM through the copy engine: every warp owns
//     a ring of kStages shared-memory stages; a stage holds 512 codes (256
//     bytes) of each of the 16 rows of ONE tile (stages alternate between the
//     pair's two tiles); lanes 0..15 each issue one bulk copy
//     (cp.async.bulk global -> shared) for their row, all completing on the
//     stage's mbarrier; fragments are then read with conflict-free 8-byte
//     shared loads (row stride 288 bytes).  256-byte pieces matter: measured on
//     B200, the same ring fed with 128-byte pieces at 1 KB stride tops out at
//     66 % of the copy bandwidth, with 256-byte pieces at 98 %.  Nothing is
//     staged in registers, so 16 warps fit on an SM and hide each other's
//     latencies.
//   * stream-K over stages: the (work unit, tile pair, stage) sequence of the
//     whole launch is cut into equal contiguous ranges, one per warp, so every
//     warp moves the same number of bytes whatever the unit count.  A tile
//     pair cut across warps is finished by the warp that owns its FIRST stage
//     (which reaches it at the end of its range); the other warps reach their
//     piece at the start of theirs, write their fp32 partial sums to a slot in
//     the workspace and raise a flag.  Partials are added in warp order, so the
//     result is deterministic for a given unit count.
//
// Every wait (mbarrier, hand-off flag) is bounded: on expiry the warp records
// a status in the workspace status word and leaves.
#include <utility>

#include "decode_common.cuh"

namespace imx {

namespace {

using namespace decode;

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 2;
constexpr int kStageCodes = 512;               // codes per row per stage
constexpr int kRowPayload = kStageCodes / 2;   // 256 bytes of 4-bit codes: pieces this int keep HBM pages busy
constexpr int kRowStride = 288;                // shared-memory bytes between rows (bank-conflict-free)
constexpr int kStageBytes = 16 * kRowStride;   // 4608: one 16-row tile
constexpr int kPlanCodes = 256;                // a tile pair advances 256 codes per stage (two stages per 512)
constexpr int kWarpBytes = kStages * kStageBytes + 64;
constexpr int kSpinLimit = 1 << 20;
constexpr int kFlagSpinLimit = 1 << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
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
// first MMA of a chain: accumulator input is zero, outputs are fresh registers
__device__ __forceinline__ void mma_f16_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    const float z = 0.f;
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(z));
}

// Two-offset unpack of a word of eight 4-bit codes: the nibbles at bits [0,4)
// of each half-word become 1024+q (planted in an fp16 whose ulp is 1), those at
// bits [4,8) become 64+q (ulp 1/16 with the code sitting four bits up), so a
// word costs one shift and four logic ops.  MMA m of a 16-code block takes
// r0 = codes (J, J+4) with offset 1024 and r1 = codes (J+1, J+5) with offset 64.
template <int M>
__device__ __forceinline__ void frag2(const uint32_t* w, uint32_t& r0, uint32_t& r1) {
    const uint32_t v = (M & 1) ? (w[M >> 1] >> 8) : w[M >> 1];
    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(r0) : "r"(v));
    asm("lop3.b32 %0, %1, 0x00f000f0, 0x54005400, 0xea;" : "=r"(r1) : "r"(v));
}

// Shape of the launch's work: two classes of units (routed experts, then the
// extra expert), each with its own tile pairs per unit and stages per pair.
struct Plan {
    int n_r, n_x;        // units
    int ppu_r, ppu_x;    // tile pairs per unit
    int st_r, st_x;      // stages (256 codes) per pair
    int stages_r;        // n_r * ppu_r * st_r (launches stay far below 2^31 stages)
    int total;          // all stages
};

// One piece of work: stages [st_lo, st_hi) of one tile pair.
struct Piece {
    int unit, pair, extra;
    int st_lo, st_hi, st_n;
    int sigma_end;      // global stage index one past the pair's last stage
};

__device__ __forceinline__ Piece piece_at(const Plan& p, int sigma, int sigma_hi) {
    Piece q;
    int local = sigma;
    int ppu = p.ppu_r, st = p.st_r, unit0 = 0;
    q.extra = 0;
    if (sigma >= p.stages_r) {
        local = sigma - p.stages_r;
        ppu = p.ppu_x;
        st = p.st_x;
        unit0 = p.n_r;
        q.extra = 1;
    }
    const int task = local / st;
    q.st_lo = (int)(local - task * st);
    q.st_n = st;
    q.unit = unit0 + (int)(task / ppu);
    q.pair = (int)(task - (task / ppu) * ppu);
    q.sigma_end = sigma - q.st_lo + st;
    const int end = q.sigma_end < sigma_hi ? q.sigma_end : sigma_hi;
    q.st_hi = q.st_lo + (int)(end - sigma);
    return q;
}

// Pointers of one tile pair.
struct PairPtrs {
    QMat m[2];
    int row0[2];
    int K;
    WorkUnit u;
};

template <bool SWIGLU>
__device__ __forceinline__ PairPtrs pair_ptrs(const GroupedArgs& a, const Piece& q) {
    const ExpertSet& S = a.set;
    PairPtrs r;
    r.u = a.units[q.unit];
    const bool extra = q.extra != 0;
    r.K = SWIGLU ? S.n_in : (extra ? S.x_mid : S.n_mid);
    r.row0[0] = SWIGLU ? q.pair * 16 : q.pair * 32;
    r.row0[1] = SWIGLU ? q.pair * 16 : q.pair * 32 + 16;
    if (SWIGLU) {
        r.m[0] = extra ? S.x_gate : S.gate;
        r.m[1] = extra ? S.x_up : S.up;
        if (!extra) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                r.m[i].w += (size_t)r.u.expert * S.gu_stride_w;
                r.m[i].scales += (size_t)r.u.expert * S.gu_stride_s;
                r.m[i].biases += (size_t)r.u.expert * S.gu_stride_s;
            }
        }
    } else {
        r.m[0] = extra ? S.x_down : S.down;
        if (!extra) {
            r.m[0].w += (size_t)r.u.expert * S.dn_stride_w;
            r.m[0].scales += (size_t)r.u.expert * S.dn_stride_s;
            r.m[0].biases += (size_t)r.u.expert * S.dn_stride_s;
        }
        r.m[1] = r.m[0];
    }
    return r;
}

// Fetch-side view of a piece.
struct FetchCtx {
    const uint8_t* wrow[2];     // packed weight row (lane & 15) of tile 0 / tile 1
    const uint8_t* s[2][2];     // scale rows g and g+8 of both tiles; biases at +bias_off
    ptrdiff_t bias_off[2];
    int st, st_hi;              // stage s = (512-code chunk s>>1, tile s&1)
};

// Compute-side view of a piece.
struct CompCtx {
    const __half* act_in;
    int rows, slot0, row0[2];
    float gs[2];
    int st, st_lo, st_hi, st_n;
    int sigma_end;
};

template <bool SWIGLU, bool G128>
__global__ void __launch_bounds__(kThreads, 1)
decode_tma_kernel(const GroupedArgs a, const int ppu_r, const int ppu_x, const int st_r, const int st_x,
                  const int flag_base) {
    constexpr bool g128 = G128;
    extern __shared__ __align__(128) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t wbuf = smem_u32(smem + (size_t)warp * kWarpBytes);
    const uint32_t bars = wbuf + kStages * kStageBytes;

    Plan plan;
    plan.n_r = a.n_units[1];
    plan.n_x = a.n_units[0] - plan.n_r;
    plan.ppu_r = ppu_r; plan.ppu_x = ppu_x; plan.st_r = st_r; plan.st_x = st_x;
    plan.stages_r = (int)plan.n_r * ppu_r * st_r;
    plan.total = plan.stages_r + (int)plan.n_x * ppu_x * st_x;

    const int gw = blockIdx.x * kWarps + warp;
    const int nw = gridDim.x * kWarps;
    auto range_lo = [&](int w) { return (int)((long long)w * plan.total / nw); };
    const int sig_lo = range_lo(gw), sig_hi = range_lo(gw + 1);
    if (sig_lo >= sig_hi) return;
    int32_t* flags = a.sched + flag_base;
    float* my_slot = a.partials + (size_t)gw * 256;

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kStages; ++s) mbar_init(bars + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();

    const size_t scale_step = g128 ? 8 : 16;           // bytes of scales per row per 512-code chunk

    // ── fetch cursor ────────────────────────────────────────────────────────
    int f_sigma = sig_lo;
    FetchCtx fc;
    auto setup_fetch = [&]() {
        const Piece q = piece_at(plan, f_sigma, sig_hi);
        const PairPtrs pp = pair_ptrs<SWIGLU>(a, q);
        const size_t row_w = (size_t)pp.K / 2;
        const size_t row_s = (size_t)(pp.K / (g128 ? 128 : 64)) * 2;
#pragma unroll
        for (int TT = 0; TT < 2; ++TT) {
            fc.wrow[TT] = pp.m[TT].w + (size_t)(pp.row0[TT] + (lane & 15)) * row_w;
            fc.bias_off[TT] = pp.m[TT].biases - pp.m[TT].scales;
#pragma unroll
            for (int h = 0; h < 2; ++h) fc.s[TT][h] = pp.m[TT].scales + (size_t)(pp.row0[TT] + g + 8 * h) * row_s;
        }
        fc.st = q.st_lo;
        fc.st_hi = q.st_hi;
    };
    setup_fetch();
    uint32_t sc_n[2][4], bi_n[2][4];                   // scales/biases (rows g, g+8) of the stage being fetched
    int n_fetch = 0;
    auto issue = [&]() {
        const int slot = n_fetch % kStages;
        const uint32_t bar = bars + 8 * slot;
        const int T = fc.st & 1, chunk = fc.st >> 1;
        if (lane == 0) mbar_expect_tx(bar, 16 * kRowPayload);
        __syncwarp();
        if (lane < 16)
            bulk_g2s(wbuf + slot * kStageBytes + lane * kRowStride, (T ? fc.wrow[1] : fc.wrow[0]) + (size_t)chunk * kRowPayload,
                     kRowPayload, bar);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint8_t* sp = (T ? fc.s[1][h] : fc.s[0][h]) + (size_t)chunk * scale_step;
            const ptrdiff_t bo = T ? fc.bias_off[1] : fc.bias_off[0];
            if (g128) {
                const uint2 sv = __ldg(reinterpret_cast<const uint2*>(sp));
                const uint2 bv = __ldg(reinterpret_cast<const uint2*>(sp + bo));
                sc_n[h][0] = sv.x; sc_n[h][1] = sv.y; sc_n[h][2] = 0; sc_n[h][3] = 0;
                bi_n[h][0] = bv.x; bi_n[h][1] = bv.y; bi_n[h][2] = 0; bi_n[h][3] = 0;
            } else {
                const uint4 sv = __ldg(reinterpret_cast<const uint4*>(sp));
                const uint4 bv = __ldg(reinterpret_cast<const uint4*>(sp + bo));
                sc_n[h][0] = sv.x; sc_n[h][1] = sv.y; sc_n[h][2] = sv.z; sc_n[h][3] = sv.w;
                bi_n[h][0] = bv.x; bi_n[h][1] = bv.y; bi_n[h][2] = bv.z; bi_n[h][3] = bv.w;
            }
        }
        ++n_fetch;
        ++fc.st;
        ++f_sigma;
        if (fc.st >= fc.st_hi && f_sigma < sig_hi) setup_fetch();
    };

    // ── compute cursor ──────────────────────────────────────────────────────
    int c_sigma = sig_lo;
    CompCtx cc;
    auto setup_comp = [&]() {
        const Piece q = piece_at(plan, c_sigma, sig_hi);
        const PairPtrs pp = pair_ptrs<SWIGLU>(a, q);
        cc.rows = pp.u.rows;
        cc.slot0 = pp.u.slot0;
        cc.row0[0] = pp.row0[0];
        cc.row0[1] = pp.row0[1];
        cc.gs[0] = pp.m[0].global_scale;
        cc.gs[1] = pp.m[1].global_scale;
        cc.st = cc.st_lo = q.st_lo;
        cc.st_hi = q.st_hi;
        cc.st_n = q.st_n;
        cc.sigma_end = q.sigma_end;
        cc.act_in = nullptr;
        if (g < pp.u.rows) {
            const int slot = pp.u.slot0 + g;
            if (SWIGLU) {
                const int row = a.row_index ? a.row_index[slot] : slot;
                cc.act_in = a.in + (size_t)row * a.set.n_in + t * 16;
            } else {
                cc.act_in = a.act + (size_t)slot * a.act_stride + t * 16;
            }
        }
    };
    setup_comp();
    float acc[2][4];
#pragma unroll
    for (int T = 0; T < 2; ++T)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[T][i] = 0.f;

    // Finishes the piece whose stages were just computed.
    auto finish_piece = [&]() -> bool {
        if (cc.st_lo > 0) {
            // not the owner: hand the partial sums to the warp that owns the pair's first stage
#pragma unroll
            for (int T = 0; T < 2; ++T)
#pragma unroll
                for (int i = 0; i < 4; ++i) my_slot[(T * 4 + i) * 32 + lane] = acc[T][i];
            __threadfence();
            __syncwarp();
            if (lane == 0) *reinterpret_cast<volatile int32_t*>(flags + gw) = 1;
        } else {
            // owner: add the partials of the following warps (if the pair was cut), then write out
            if (cc.st_hi < cc.st_n) {
                int covered = sig_hi;                          // this warp covered the pair up to its range end
                for (int w = gw + 1; covered < cc.sigma_end && w < nw; ++w) {
                    if (range_lo(w + 1) == range_lo(w)) continue;   // a warp without work raises no flag
                    int ok = 1;
                    if (lane == 0) {
                        int spin = 0;
                        while (*reinterpret_cast<volatile int32_t*>(flags + w) == 0) {
                            if (++spin > kFlagSpinLimit) {
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
            TaskCtx tc;
            tc.rows = cc.rows;
            tc.slot0 = cc.slot0;
            tc.row0[0] = cc.row0[0];
            tc.row0[1] = cc.row0[1];
            tc.valid = 1;
            tc.gs[0] = cc.gs[0];
            tc.gs[1] = cc.gs[1];
            epilogue<4, SWIGLU>(a, tc, acc, g, t);
        }
#pragma unroll
        for (int T = 0; T < 2; ++T)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[T][i] = 0.f;
        return true;
    };

    issue();                                             // stage 0 of this warp's range
    int n_comp = 0;
    float xsc[8][2];                                     // group sums of x over the current 512-code chunk (slots 2t, 2t+1)
    float xoc[8][2];                                     // the matching offset sums / 64
    bool xs_ready = false;
#pragma unroll 1
    while (c_sigma < sig_hi) {
        // scales fetched with this stage become current; then start the next stage
        uint32_t sc[2][4], bi[2][4];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                sc[h][j] = sc_n[h][j];
                bi[h][j] = bi_n[h][j];
            }
        if (f_sigma < sig_hi) issue();

        const int slot = n_comp % kStages;
        const int T = cc.st & 1, chunk = cc.st >> 1;
        const bool need_xs = (T == 0) || !xs_ready;      // tile 1 reuses the sums tile 0 computed for this chunk
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
        const uint32_t wst = wbuf + slot * kStageBytes + (uint32_t)g * kRowStride + (uint32_t)t * 8;
        constexpr uint32_t ONES = 0x3c003c00u;           // fp16 (1, 1)
        constexpr uint32_t C16 = 0x4c004c00u;            // fp16 (16, 16)
        float acc_t[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            // activations of this iteration: 2 steps x 32 bytes of this lane's slot
            uint32_t bf[2][8];
            if (cc.act_in != nullptr) {
                const uint4* p = reinterpret_cast<const uint4*>(cc.act_in + (size_t)chunk * kStageCodes + i * 128);
#pragma unroll
                for (int s = 0; s < 2; ++s) {
                    const uint4 v0 = __ldg(p + s * 8), v1 = __ldg(p + s * 8 + 1);
                    bf[s][0] = v0.x; bf[s][1] = v0.y; bf[s][2] = v0.z; bf[s][3] = v0.w;
                    bf[s][4] = v1.x; bf[s][5] = v1.y; bf[s][6] = v1.z; bf[s][7] = v1.w;
                }
            } else {
#pragma unroll
                for (int s = 0; s < 2; ++s)
#pragma unroll
                    for (int j = 0; j < 8; ++j) bf[s][j] = 0u;
            }
#pragma unroll
            for (int s = 0; s < 2; ++s) {
                const int j = i * 2 + s;                       // step (64 codes) within the chunk
                if (need_xs) {
                    // rows 0..7 of the constant operand are ones (sum of x), rows 8..15 hold
                    // 16 on the offset-1024 positions and 1 on the offset-64 ones (offset sum / 64)
                    float xs[4];
                    mma_f16_z(xs, ONES, C16, ONES, ONES, bf[s][0], bf[s][1]);
#pragma unroll
                    for (int m = 1; m < 4; ++m) mma_f16(xs, ONES, C16, ONES, ONES, bf[s][2 * m], bf[s][2 * m + 1]);
                    xsc[j][0] = xs[0];
                    xsc[j][1] = xs[1];
                    xoc[j][0] = xs[2];
                    xoc[j][1] = xs[3];
                }
                uint32_t wlo[2], whi[2];
                const uint32_t addr = wst + (uint32_t)(i * 64 + s * 32);
                asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(wlo[0]), "=r"(wlo[1]) : "r"(addr));
                asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(whi[0]), "=r"(whi[1]) : "r"(addr + 8 * kRowStride));
                float d[4];
                uint32_t a0, a1, a2, a3;
                frag2<0>(wlo, a0, a2); frag2<0>(whi, a1, a3);
                mma_f16_z(d, a0, a1, a2, a3, bf[s][0], bf[s][1]);
                frag2<1>(wlo, a0, a2); frag2<1>(whi, a1, a3);
                mma_f16(d, a0, a1, a2, a3, bf[s][2], bf[s][3]);
                frag2<2>(wlo, a0, a2); frag2<2>(whi, a1, a3);
                mma_f16(d, a0, a1, a2, a3, bf[s][4], bf[s][5]);
                frag2<3>(wlo, a0, a2); frag2<3>(whi, a1, a3);
                mma_f16(d, a0, a1, a2, a3, bf[s][6], bf[s][7]);
                // group of this step: 64-code groups -> j, 128-code groups -> j/2
                const int word = G128 ? (j >> 2) : (j >> 1);
                const bool hi_half = G128 ? ((j >> 1) & 1) != 0 : (j & 1) != 0;
                auto pick = [&](uint32_t v) { return __uint_as_float(hi_half ? (v & 0xffff0000u) : (v << 16)); };
                const float s_lo = pick(sc[0][word]), s_hi = pick(sc[1][word]);
                const float b_lo = pick(bi[0][word]), b_hi = pick(bi[1][word]);
                const float o_lo = -64.f * s_lo, o_hi = -64.f * s_hi;     // times the offset sum / 64
                acc_t[0] = fmaf(s_lo, d[0], fmaf(o_lo, xoc[j][0], fmaf(b_lo, xsc[j][0], acc_t[0])));
                acc_t[1] = fmaf(s_lo, d[1], fmaf(o_lo, xoc[j][1], fmaf(b_lo, xsc[j][1], acc_t[1])));
                acc_t[2] = fmaf(s_hi, d[2], fmaf(o_hi, xoc[j][0], fmaf(b_hi, xsc[j][0], acc_t[2])));
                acc_t[3] = fmaf(s_hi, d[3], fmaf(o_hi, xoc[j][1], fmaf(b_hi, xsc[j][1], acc_t[3])));
            }
        }
        if (T == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[0][i] += acc_t[i];
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[1][i] += acc_t[i];
        }
        xs_ready = (T == 0);                             // valid for the tile-1 stage of the same chunk only
        __syncwarp();          // every lane is done reading this slot before it is refilled
        ++n_comp;
        ++cc.st;
        ++c_sigma;
        if (cc.st >= cc.st_hi) {
            xs_ready = false;
            if (!finish_piece()) return;
            if (c_sigma < sig_hi) setup_comp();
        }
    }
}

}  // namespace

bool decode_tma_supported(const ExpertSet& s) {
    const QFormat& f = s.fmt;
    if (f.mode != IMX_MODE_AFFINE || f.bits != 4) return false;
    if (f.group != 64 && f.group != 128) return false;
    if (s.n_in % kStageCodes || s.n_mid % kStageCodes) return false;
    if (s.has_extra && s.x_mid % kStageCodes) return false;
    return true;
}

int launch_decode_tma(const GroupedArgs& a, cudaStream_t stream, cudaEvent_t mid) {
    IMX_REQUIRE(decode_tma_supported(a.set), "decode (TMA) path: format/shape not supported");
    IMX_REQUIRE(a.partials != nullptr && a.sched != nullptr, "decode (TMA) path: hand-off buffers missing");
    if (a.max_units == 0) return IMX_OK;
    const ExpertSet& s = a.set;
    static int sms = 0;
    const size_t smem = (size_t)kWarpBytes * kWarps;
    if (sms == 0) {
        int dev = 0, v = 0;
        IMX_CHECK_CUDA(cudaGetDevice(&dev));
        IMX_CHECK_CUDA(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev));
        IMX_CHECK_CUDA(cudaFuncSetAttribute(decode_tma_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        IMX_CHECK_CUDA(cudaFuncSetAttribute(decode_tma_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        IMX_CHECK_CUDA(cudaFuncSetAttribute(decode_tma_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        IMX_CHECK_CUDA(cudaFuncSetAttribute(decode_tma_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        sms = v;
    }
    int grid = sms;
    if (grid * kWarps > kFlagWarps) grid = kFlagWarps / kWarps;
    const bool g128 = s.fmt.group == 128;
    const int x_mid = s.has_extra ? s.x_mid : s.n_mid;
    auto k_gu = g128 ? decode_tma_kernel<true, true> : decode_tma_kernel<true, false>;
    auto k_dn = g128 ? decode_tma_kernel<false, true> : decode_tma_kernel<false, false>;
    k_gu<<<grid, kThreads, smem, stream>>>(a, s.n_mid / 16, x_mid / 16, s.n_in / kPlanCodes, s.n_in / kPlanCodes, 8);
    IMX_CHECK_CUDA(cudaGetLastError());
    if (mid) IMX_CHECK_CUDA(cudaEventRecord(mid, stream));
    k_dn<<<grid, kThreads, smem, stream>>>(a, s.n_in / 32, s.n_in / 32, s.n_mid / kPlanCodes, x_mid / kPlanCodes,
                                           8 + kFlagWarps);
    IMX_CHECK_CUDA(cudaGetLastError());
    return IMX_OK;
}

}  // namespace imx
