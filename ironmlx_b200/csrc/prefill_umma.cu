// Prefill-regime grouped expert products on the 5th-generation tensor cores:
// tcgen05.mma (kind::f16, fp16 x fp16 -> fp32) with the accumulator in tensor
// memory, for affine 4-bit weights (group 64/128).
//
//   first product   act[slot, :] = silu(x W_gate^T) * (x W_up^T)       (moe.rs:26-30)
//   second product  out[slot, :] = row_scale[slot] * (act W_down^T)    (moe.rs:31, 155-161)
//
// Tile = 128 sorted slots of one expert (the M side, one TMEM lane per slot) x
// 128 output columns (first product: 64 gate rows + the matching 64 up rows,
// so SwiGLU happens in the epilogue; second product: 128 down rows), K in
// steps of 64 (one 128-byte swizzle atom per row).
//
// One persistent CTA per SM, 16 warps, specialised:
//   warp 0        issues the MMAs (one elected lane): waits for a filled stage,
//                 4 x tcgen05.mma (K=16 each) per stage, tcgen05.commit to
//                 release the stage, and after the last K step to publish the
//                 accumulator (two accumulators in TMEM: epilogue of tile i
//                 overlaps the MMAs of tile i+1)
//   warp 1        allocates / frees tensor memory
//   warps 4..7    epilogue: tcgen05.ld of their 32 TMEM lanes, SwiGLU or row
//                 scaling in registers, stores
//   warp 2        loads the activation tiles: one tiled TMA copy
//                 (cp.async.bulk.tensor.2d, 128B swizzle) of 128 slots x 64
//                 values per stage from the slot-ordered activation matrix
//                 (first product: x gathered once into sorted-slot order;
//                 second: the SwiGLU output, which is already slot-ordered);
//                 rows past the tensor's end are zero-filled by the copy engine
//   warps 8..15   weight producers, two groups of four warps on alternating K
//                 steps; a thread owns one weight row of the tile: 32 bytes of
//                 packed codes per K step -> 64 fp16 values (exact integer
//                 codes from the mantissa trick, then one HFMA2 with the
//                 group's scale and bias) -> eight swizzled 16-byte shared stores
// Stages are handed over with mbarriers (full: the 4 warps of the producer group
// that owns the stage + the TMA transaction bytes, empty: one tcgen05.commit).  Every wait is bounded; on expiry the CTA records a
// status, all roles leave their loops and tensor memory is freed.
// Every copy is issued per CTA; the kernel uses no thread-block clusters.
#include <cuda.h>

#include <type_traits>

#include "decode_common.cuh"

namespace imx {

namespace {

using namespace decode;

constexpr int kStages = 5;
constexpr int kTileM = 128, kTileN = 128, kTileK = 64;
constexpr int kABytes = kTileM * kTileK * 2;      // 16 KB
constexpr int kBBytes = kTileN * kTileK * 2;      // 16 KB
constexpr int kQBytes = kTileN * kTileK / 2;       // 4 KB of packed 4-bit codes (128 rows x 32 bytes)
constexpr int kStageBytes = kABytes + kBBytes + kQBytes;   // 36 KB: A (fp16) | B (fp16, dequantized) | Q (packed)
constexpr int kSpin = 1 << 22;
constexpr uint32_t kTmemCols = 256;               // two 128-column fp32 accumulators

struct Bars {                                     // shared-memory control block
    uint64_t qfull[kStages];                      // A tile + packed codes landed (TMA bytes)
    uint64_t full[kStages];                       // B dequantized: the stage is ready for the MMA
    uint64_t empty[kStages];                      // MMAs that read the stage retired
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint64_t sfull[2];                            // scales/biases of a tile landed
    uint64_t sempty[2];                           // ... and were consumed by both producer groups
    uint32_t tmem_base;
    int abort;
};

// Tensor maps of one launch: activations, packed weights and scales/biases of the
// routed experts' stacked matrix ([0]) and of the extra expert's matrices ([1], [2]).
struct PrefillMaps {
    CUtensorMap a;
    CUtensorMap w[3];
    CUtensorMap s[3];
    CUtensorMap b[3];
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
// kind::f16: D fp32, A/B fp16 K-major, N = 128, M = 128
constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(kTileN >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(kIdesc), "r"(accumulate), "r"(0u)
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

// What a tile is made of.
struct TileInfo {
    int expert, slot0, rows, ntile, extra;
    int K, n_out;           // reduction length, output rows of this expert's matrix
};

template <bool SWIGLU>
__device__ __forceinline__ TileInfo tile_info(const GroupedArgs& a, int tile, int nt_r, int nt_x, int tiles_r) {
    // tiles of the routed experts first (nt_r column tiles per unit), then the extra expert's
    TileInfo t;
    const int n_r = a.n_units[1];
    int unit, nt;
    if (tile < tiles_r) {
        unit = tile / nt_r;
        nt = nt_r;
        t.ntile = tile - unit * nt_r;
    } else {
        const int l = tile - tiles_r;
        unit = n_r + l / nt_x;
        nt = nt_x;
        t.ntile = l - (l / nt_x) * nt_x;
    }
    (void)nt;
    const WorkUnit u = a.units[unit];
    t.expert = u.expert;
    t.slot0 = u.slot0;
    t.rows = u.rows;
    t.extra = u.expert >= a.set.num_experts;
    t.K = SWIGLU ? a.set.n_in : (t.extra ? a.set.x_mid : a.set.n_mid);
    t.n_out = SWIGLU ? (t.extra ? a.set.x_mid : a.set.n_mid) : a.set.n_in;
    return t;
}

// Weight matrix and first row of the B tile's row `brow` (0..127).
template <bool SWIGLU>
__device__ __forceinline__ void b_row(const GroupedArgs& a, const TileInfo& t, int brow, QMat& m, int& row) {
    const ExpertSet& S = a.set;
    if (SWIGLU) {
        const bool up = brow >= 64;
        m = t.extra ? (up ? S.x_up : S.x_gate) : (up ? S.up : S.gate);
        if (!t.extra) {
            m.w += (size_t)t.expert * S.gu_stride_w;
            m.scales += (size_t)t.expert * S.gu_stride_s;
            m.biases += (size_t)t.expert * S.gu_stride_s;
        }
        row = t.ntile * 64 + (up ? brow - 64 : brow);
    } else {
        m = t.extra ? S.x_down : S.down;
        if (!t.extra) {
            m.w += (size_t)t.expert * S.dn_stride_w;
            m.scales += (size_t)t.expert * S.dn_stride_s;
            m.biases += (size_t)t.expert * S.dn_stride_s;
        }
        row = t.ntile * 128 + brow;
    }
}

__device__ __forceinline__ __half2 bf16_to_half2(uint16_t b) {
    return __float2half2_rn(__uint_as_float((uint32_t)b << 16));
}

// PW producer warps in PW / 4 groups (a group of four warps dequantizes one stage; group j takes the K
// steps j, j + PW/4, ...); the block has 8 + PW warps.
template <bool SWIGLU, bool G128, int PW>
__global__ void __launch_bounds__(256 + 32 * PW, 1)
prefill_umma_kernel(const GroupedArgs a, const int nt_r, const int nt_x, const int srow_max,
                    const __grid_constant__ PrefillMaps maps) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    // [kStages stages][2 tiles x (scales | biases) x 128 rows x srow_max bytes][control block]
    const uint32_t sc_bytes = 2u * 128u * (uint32_t)srow_max;          // one tile's scales + biases
    Bars* bars = reinterpret_cast<Bars*>(base + kStages * kStageBytes + 2 * sc_bytes);
    const uint32_t sbase = smem_u32(base);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    volatile int* abort_flag = &bars->abort;

    const int n_r = a.n_units[1], n_x = a.n_units[0] - n_r;
    const int tiles_r = n_r * nt_r;
    const int total = tiles_r + n_x * nt_x;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&bars->qfull[s]), 1);
            mbar_init(smem_u32(&bars->full[s]), 4);
            mbar_init(smem_u32(&bars->empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bars->acc_full[b]), 1);
            mbar_init(smem_u32(&bars->acc_empty[b]), 4);
            mbar_init(smem_u32(&bars->sfull[b]), 1);
            mbar_init(smem_u32(&bars->sempty[b]), PW);
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
        int n = 0, it = 0;
        for (int tile = blockIdx.x; tile < total; tile += gridDim.x, ++it) {
            const TileInfo t = tile_info<SWIGLU>(a, tile, nt_r, nt_x, tiles_r);
            const int buf = it & 1;
            if (!mbar_wait(smem_u32(&bars->acc_empty[buf]), ((it >> 1) & 1) ^ 1, abort_flag)) break;
            tc_fence_after();
            const int ksteps = t.K / kTileK;
            bool ok = true;
            for (int ks = 0; ks < ksteps; ++ks, ++n) {
                const int s = n % kStages;
                if (!mbar_wait(smem_u32(&bars->full[s]), (n / kStages) & 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                if (lane == 0) {
                    const uint64_t da = smem_desc(sbase + s * kStageBytes);
                    const uint64_t db = smem_desc(sbase + s * kStageBytes + kABytes);
#pragma unroll
                    for (int kk = 0; kk < kTileK / 16; ++kk)
                        umma_f16(tmem + buf * kTileN, da + 2 * kk, db + 2 * kk, (ks > 0 || kk > 0) ? 1u : 0u);
                    umma_commit(smem_u32(&bars->empty[s]));                 // stage free once these MMAs retire
                    if (ks == ksteps - 1) umma_commit(smem_u32(&bars->acc_full[buf]));
                }
                __syncwarp();
            }
            if (!ok) break;
        }
    } else if (warp == 2) {
        // ── loader (TMA): activations, packed codes, scales/biases ──────────
        const uint32_t sc_base = sbase + kStages * kStageBytes;
        int n = 0, it = 0;
        for (int tile = blockIdx.x; tile < total; tile += gridDim.x, ++it) {
            const TileInfo t = tile_info<SWIGLU>(a, tile, nt_r, nt_x, tiles_r);
            const int ksteps = t.K / kTileK;
            // which maps and which rows the two 64-row halves of the B tile come from
            int mi0, mi1, row0, row1;
            if (SWIGLU) {
                if (t.extra) { mi0 = 1; mi1 = 2; row0 = row1 = t.ntile * 64; }
                else { mi0 = mi1 = 0; row0 = t.expert * 2 * a.set.n_mid + t.ntile * 64; row1 = row0 + a.set.n_mid; }
            } else {
                mi0 = mi1 = t.extra ? 1 : 0;
                row0 = (t.extra ? 0 : t.expert * a.set.n_in) + t.ntile * 128;
                row1 = row0 + 64;
            }
            const CUtensorMap* w0 = mi0 == 0 ? &maps.w[0] : (mi0 == 1 ? &maps.w[1] : &maps.w[2]);
            const CUtensorMap* w1 = mi1 == 0 ? &maps.w[0] : (mi1 == 1 ? &maps.w[1] : &maps.w[2]);
            const CUtensorMap* s0 = mi0 == 0 ? &maps.s[0] : (mi0 == 1 ? &maps.s[1] : &maps.s[2]);
            const CUtensorMap* s1 = mi1 == 0 ? &maps.s[0] : (mi1 == 1 ? &maps.s[1] : &maps.s[2]);
            const CUtensorMap* b0 = mi0 == 0 ? &maps.b[0] : (mi0 == 1 ? &maps.b[1] : &maps.b[2]);
            const CUtensorMap* b1 = mi1 == 0 ? &maps.b[0] : (mi1 == 1 ? &maps.b[1] : &maps.b[2]);
            // scales and biases of the whole tile (rows x K/group), one buffer per tile parity
            const int sbuf = it & 1;
            if (!mbar_wait(smem_u32(&bars->sempty[sbuf]), ((it >> 1) & 1) ^ 1, abort_flag)) break;
            if (lane == 0) {
                const uint32_t srow = (uint32_t)(t.K / (G128 ? 128 : 64)) * 2;     // bytes per row
                const uint32_t bar = smem_u32(&bars->sfull[sbuf]);
                const uint32_t dst = sc_base + sbuf * sc_bytes;
                mbar_expect_tx(bar, 4 * 64 * srow);
                tma_load_2d(dst, s0, 0, row0, bar);
                tma_load_2d(dst + 64 * srow, s1, 0, row1, bar);
                tma_load_2d(dst + 128 * srow, b0, 0, row0, bar);
                tma_load_2d(dst + 192 * srow, b1, 0, row1, bar);
            }
            __syncwarp();
            bool ok = true;
            for (int ks = 0; ks < ksteps; ++ks, ++n) {
                const int s = n % kStages;
                if (!mbar_wait(smem_u32(&bars->empty[s]), ((n / kStages) & 1) ^ 1, abort_flag)) { ok = false; break; }
                if (lane == 0) {
                    const uint32_t bar = smem_u32(&bars->qfull[s]);
                    const uint32_t stage = sbase + s * kStageBytes;
                    mbar_expect_tx(bar, kABytes + kQBytes);
                    tma_load_2d(stage, &maps.a, ks * kTileK, t.slot0, bar);
                    tma_load_2d(stage + kABytes + kBBytes, w0, ks * (kTileK / 2), row0, bar);
                    tma_load_2d(stage + kABytes + kBBytes + kQBytes / 2, w1, ks * (kTileK / 2), row1, bar);
                }
                __syncwarp();
            }
            if (!ok) break;
        }
    } else if (warp >= 4 && warp < 8) {
        // ── epilogue ────────────────────────────────────────────────────────
        const int q = warp - 4;
        int it = 0;
        for (int tile = blockIdx.x; tile < total; tile += gridDim.x, ++it) {
            const TileInfo t = tile_info<SWIGLU>(a, tile, nt_r, nt_x, tiles_r);
            const int buf = it & 1;
            if (!mbar_wait(smem_u32(&bars->acc_full[buf]), (it >> 1) & 1, abort_flag)) break;
            tc_fence_after();
            const int row = q * 32 + lane;
            const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + buf * kTileN;
            const bool valid = row < t.rows;
            const int slot = t.slot0 + row;
            if (SWIGLU) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t g[32], u[32];
                    tmem_ld32(taddr + h * 32, g);
                    tmem_ld32(taddr + 64 + h * 32, u);
                    if (h == 1) {                       // all of this warp's TMEM reads are done
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&bars->acc_empty[buf]));
                    }
                    if (valid) {
                        __half* dst = a.act + (size_t)slot * a.act_stride + t.ntile * 64 + h * 32;
#pragma unroll
                        for (int blk = 0; blk < 2; ++blk) {
                            __half2 o[8];
#pragma unroll
                            for (int p = 0; p < 16; p += 2) {
                                const int f0 = blk * 16 + Codec<4>::order(p), f1 = blk * 16 + Codec<4>::order(p + 1);
                                const float v0 = silu_f(__uint_as_float(g[f0])) * __uint_as_float(u[f0]);
                                const float v1 = silu_f(__uint_as_float(g[f1])) * __uint_as_float(u[f1]);
                                o[p >> 1] = __halves2half2(f32_to_f16_sat(v0), f32_to_f16_sat(v1));
                            }
                            *reinterpret_cast<uint4*>(dst + blk * 16) = *reinterpret_cast<uint4*>(&o[0]);
                            *reinterpret_cast<uint4*>(dst + blk * 16 + 8) = *reinterpret_cast<uint4*>(&o[4]);
                        }
                    }
                }
            } else {
                const float sc = (valid && a.row_scale) ? a.row_scale[slot] : 1.f;
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                    uint32_t d[32];
                    tmem_ld32(taddr + h * 32, d);
                    if (h == 3) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&bars->acc_empty[buf]));
                    }
                    if (valid && a.out16 != nullptr) {
                        // fp16 rows: half the bytes for this store and for the combine stage's reads
                        __half* dst = a.out16 + (size_t)slot * a.set.n_in + t.ntile * 128 + h * 32;
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            __half2 o[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                o[e] = __halves2half2(f32_to_f16_sat(__uint_as_float(d[i + 2 * e]) * sc),
                                                      f32_to_f16_sat(__uint_as_float(d[i + 2 * e + 1]) * sc));
                            *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(o);
                        }
                    } else if (valid) {
                        float* dst = a.out + (size_t)slot * a.set.n_in + t.ntile * 128 + h * 32;
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            *reinterpret_cast<float4*>(dst + i) =
                                make_float4(__uint_as_float(d[i]) * sc, __uint_as_float(d[i + 1]) * sc,
                                            __uint_as_float(d[i + 2]) * sc, __uint_as_float(d[i + 3]) * sc);
                    }
                }
            }
        }
    } else if (warp >= 8) {
        // ── producers ───────────────────────────────────────────────────────
        // PW / 4 groups of four warps: group j fills the K steps j, j + PW / 4, ..., so PW / 4
        // stages are being produced at once.  Inside a group a
        // thread owns one weight row of the tile: 32 bytes of packed codes per K step
        // (prefetched one of its own steps ahead), dequantized into eight 16-byte chunks.
        const int grp_id = (warp - 8) >> 2;
        const int gtid = tid - 256 - grp_id * 128;        // 0..127 = B row
        const int brow = gtid;
        const uint32_t sc_base = sbase + kStages * kStageBytes;
        const uint32_t bdst = (uint32_t)(kABytes + (brow >> 3) * 1024 + (brow & 7) * 128);
        const __half2 c1024 = __float2half2_rn(1024.f), c64 = __float2half2_rn(64.f);
        int n_tile0 = 0, it = 0;                          // stage counter at the start of the tile
        for (int tile = blockIdx.x; tile < total; tile += gridDim.x, ++it) {
            const TileInfo t = tile_info<SWIGLU>(a, tile, nt_r, nt_x, tiles_r);
            const int ksteps = t.K / kTileK;
            const int sbuf = it & 1;
            const uint32_t srow = (uint32_t)(t.K / (G128 ? 128 : 64)) * 2;
            // this row's scales (first half of the buffer) and biases (second half)
            const uint32_t s_addr = sc_base + sbuf * sc_bytes + (uint32_t)brow * srow;
            const uint32_t b_addr = s_addr + 128 * srow;
            if (!mbar_wait(smem_u32(&bars->sfull[sbuf]), (it >> 1) & 1, abort_flag)) break;
            uint4 sv = make_uint4(0, 0, 0, 0), bv = make_uint4(0, 0, 0, 0);   // eight groups' scales / biases
            int cur_blk = -1;
            bool ok = true;
            for (int ks = grp_id; ks < ksteps; ks += PW / 4) {
                const int n = n_tile0 + ks;
                const int s = n % kStages;
                const int gi = G128 ? (ks >> 1) : ks;     // group of this K step
                if ((gi >> 3) != cur_blk) {
                    cur_blk = gi >> 3;
                    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(sv.x), "=r"(sv.y), "=r"(sv.z), "=r"(sv.w)
                                 : "r"(s_addr + (uint32_t)cur_blk * 16));
                    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(bv.x), "=r"(bv.y), "=r"(bv.z), "=r"(bv.w)
                                 : "r"(b_addr + (uint32_t)cur_blk * 16));
                }
                const int e = gi & 7;
                const uint32_t sw = e < 4 ? (e < 2 ? sv.x : sv.y) : (e < 6 ? sv.z : sv.w);
                const uint32_t bw = e < 4 ? (e < 2 ? bv.x : bv.y) : (e < 6 ? bv.z : bv.w);
                const __half2 sc2 = bf16_to_half2((uint16_t)((e & 1) ? (sw >> 16) : (sw & 0xffffu)));
                const __half2 bi2 = bf16_to_half2((uint16_t)((e & 1) ? (bw >> 16) : (bw & 0xffffu)));
                if (!mbar_wait(smem_u32(&bars->qfull[s]), (n / kStages) & 1, abort_flag)) { ok = false; break; }
                const uint32_t stage = sbase + s * kStageBytes;
                uint32_t words[8];
                const uint32_t q_addr = stage + kABytes + kBBytes + (uint32_t)brow * 32;
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                             : "=r"(words[0]), "=r"(words[1]), "=r"(words[2]), "=r"(words[3]) : "r"(q_addr));
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                             : "=r"(words[4]), "=r"(words[5]), "=r"(words[6]), "=r"(words[7]) : "r"(q_addr + 16));
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    // eight codes of a word -> (0,4) (1,5) (2,6) (3,7): the order the activation rows use
                    uint32_t r[4];
                    const uint32_t v = words[j], v8 = v >> 8;
                    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(r[0]) : "r"(v));
                    asm("lop3.b32 %0, %1, 0x00f000f0, 0x54005400, 0xea;" : "=r"(r[1]) : "r"(v));
                    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(r[2]) : "r"(v8));
                    asm("lop3.b32 %0, %1, 0x00f000f0, 0x54005400, 0xea;" : "=r"(r[3]) : "r"(v8));
                    __half2 o[4];
#pragma unroll
                    for (int e2 = 0; e2 < 4; ++e2) {
                        const __half2 qh = __hsub2(*reinterpret_cast<__half2*>(&r[e2]), (e2 & 1) ? c64 : c1024);   // exact code
                        o[e2] = __hfma2(qh, sc2, bi2);                                                        // scale*q + bias
                    }
                    const uint32_t dst = stage + bdst + (((uint32_t)j ^ (uint32_t)(brow & 7)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(*reinterpret_cast<uint32_t*>(&o[0])),
                                 "r"(*reinterpret_cast<uint32_t*>(&o[1])), "r"(*reinterpret_cast<uint32_t*>(&o[2])),
                                 "r"(*reinterpret_cast<uint32_t*>(&o[3]))
                                 : "memory");
                }
                fence_async_proxy();                 // generic-proxy writes -> visible to the tensor-core reads
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars->full[s]));
            }
            if (!ok) break;
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars->sempty[sbuf]));   // this warp is done with the tile's scales
            n_tile0 += ksteps;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
    if (tid == 0 && bars->abort && a.status != nullptr) atomicExch(a.status, 3);
}

}  // namespace

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int make_tensor_map_2d(const void* base, CUtensorMapDataType dt, size_t esize, size_t rows, size_t cols,
                       size_t ld_bytes, int box_cols, int box_rows, bool swizzle128, CUtensorMap* out,
                       bool promote256) {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        IMX_CHECK_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
        IMX_REQUIRE(p != nullptr && q == cudaDriverEntryPointSuccess, "cuTensorMapEncodeTiled is not available");
        fn = (EncodeTiledFn)p;
    }
    IMX_REQUIRE(((uintptr_t)base % 16) == 0 && ld_bytes % 16 == 0 && (box_cols * esize) % 16 == 0,
                "tensor map: a matrix is not 16-byte aligned (base %p, row pitch %zu)", base, ld_bytes);
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                          promote256 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    IMX_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with %d", (int)r);
    return IMX_OK;
}

bool prefill_umma_supported(const ExpertSet& s) {
    const QFormat& f = s.fmt;
    if (f.mode != IMX_MODE_AFFINE || f.bits != 4) return false;
    if (f.group != 64 && f.group != 128) return false;
    // a row of scales must be whole 16-byte pieces (TMA box, 16-byte shared loads): K % (8 * group) == 0
    const int q = 8 * f.group;
    if (s.n_in % q || s.n_mid % q) return false;
    if (s.has_extra && s.x_mid % q) return false;
    if (s.n_in / f.group > 256 || s.n_mid / f.group > 256 || (s.has_extra && s.x_mid / f.group > 256)) return false;
    return true;
}

namespace {

// packed codes + scales + biases maps of one stacked quantized matrix [rows, K]
int make_q_maps(const QMat& m, size_t rows, int K, int group, CUtensorMap* w, CUtensorMap* sc, CUtensorMap* bi) {
    const int groups = K / group;
    IMX_TRY(make_tensor_map_2d(m.w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, rows, (size_t)K / 2, (size_t)K / 2, kTileK / 2, 64, false, w));
    IMX_TRY(make_tensor_map_2d(m.scales, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, rows, groups, (size_t)groups * 2, groups, 64, false, sc));
    IMX_TRY(make_tensor_map_2d(m.biases, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, rows, groups, (size_t)groups * 2, groups, 64, false, bi));
    return IMX_OK;
}

}  // namespace

int launch_prefill_umma(const GroupedArgs& a, cudaStream_t stream, cudaEvent_t mid) {
    IMX_REQUIRE(prefill_umma_supported(a.set), "prefill path: format/shape not supported");
    IMX_REQUIRE((a.row_index == nullptr || a.xs != nullptr) && a.n_slots > 0,
                "prefill path: slot-ordered activation buffer missing");
    if (a.max_units == 0) return IMX_OK;
    const ExpertSet& s = a.set;
    const int g = s.fmt.group;
    const bool g128 = g == 128;
    const int x_mid = s.has_extra ? s.x_mid : s.n_mid;
    const int mid_max = s.n_mid > x_mid ? s.n_mid : x_mid;
    const int srow_gu = s.n_in / g * 2, srow_dn = mid_max / g * 2;
    auto smem_for = [](int srow) { return (size_t)kStages * kStageBytes + 4u * 128u * (size_t)srow + sizeof(Bars) + 1024; };
    IMX_REQUIRE(smem_for(srow_gu) <= 227 * 1024 && smem_for(srow_dn) <= 227 * 1024, "prefill path: sizes exceed shared memory");
    static int sms = 0;
    if (sms == 0) {
        int dev = 0, v = 0;
        IMX_CHECK_CUDA(cudaGetDevice(&dev));
        IMX_CHECK_CUDA(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev));
        sms = v;
    }
    // activations in sorted-slot order (the `take_axis` of moe.rs:124-127, once for all experts)
    const __half* xsrc = a.in;                     // already slot-ordered when there is no row index
    if (a.row_index != nullptr) {
        IMX_TRY(launch_gather_rows(a.in, a.row_index, a.n_slots, (size_t)s.n_in * 2, a.xs, stream));
        xsrc = a.xs;
    }
    PrefillMaps gu, dn;
    IMX_TRY(make_tensor_map_2d(xsrc, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (size_t)a.n_slots, (size_t)s.n_in, (size_t)s.n_in * 2, kTileK,
                     kTileM, true, &gu.a));
    IMX_TRY(make_tensor_map_2d(a.act, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (size_t)a.n_slots, (size_t)mid_max, (size_t)a.act_stride * 2,
                     kTileK, kTileM, true, &dn.a));
    // routed experts: gate and up rows live in one stacked matrix [E*2I, H]; down in [E*H, I]
    IMX_TRY(make_q_maps(s.gate, (size_t)s.num_experts * 2 * s.n_mid, s.n_in, g, &gu.w[0], &gu.s[0], &gu.b[0]));
    IMX_TRY(make_q_maps(s.down, (size_t)s.num_experts * s.n_in, s.n_mid, g, &dn.w[0], &dn.s[0], &dn.b[0]));
    if (s.has_extra) {
        IMX_TRY(make_q_maps(s.x_gate, (size_t)s.x_mid, s.n_in, g, &gu.w[1], &gu.s[1], &gu.b[1]));
        IMX_TRY(make_q_maps(s.x_up, (size_t)s.x_mid, s.n_in, g, &gu.w[2], &gu.s[2], &gu.b[2]));
        IMX_TRY(make_q_maps(s.x_down, (size_t)s.n_in, s.x_mid, g, &dn.w[1], &dn.s[1], &dn.b[1]));
    } else {
        gu.w[1] = gu.w[0]; gu.s[1] = gu.s[0]; gu.b[1] = gu.b[0];
        dn.w[1] = dn.w[0]; dn.s[1] = dn.s[0]; dn.b[1] = dn.b[0];
    }
    if (!s.has_extra) { gu.w[2] = gu.w[0]; gu.s[2] = gu.s[0]; gu.b[2] = gu.b[0]; }
    dn.w[2] = dn.w[0]; dn.s[2] = dn.s[0]; dn.b[2] = dn.b[0];
    const size_t smem_gu = smem_for(srow_gu), smem_dn = smem_for(srow_dn);
    auto run = [&](auto pw_tag) -> int {
        constexpr int PW = decltype(pw_tag)::value;
        auto k_gu = g128 ? prefill_umma_kernel<true, true, PW> : prefill_umma_kernel<true, false, PW>;
        auto k_dn = g128 ? prefill_umma_kernel<false, true, PW> : prefill_umma_kernel<false, false, PW>;
        static bool configured = false;      // once per instantiation, outside any stream capture (first call)
        if (!configured) {
            IMX_CHECK_CUDA(cudaFuncSetAttribute(prefill_umma_kernel<true, true, PW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
            IMX_CHECK_CUDA(cudaFuncSetAttribute(prefill_umma_kernel<true, false, PW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
            IMX_CHECK_CUDA(cudaFuncSetAttribute(prefill_umma_kernel<false, true, PW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
            IMX_CHECK_CUDA(cudaFuncSetAttribute(prefill_umma_kernel<false, false, PW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
            configured = true;
        }
        k_gu<<<sms, 256 + 32 * PW, smem_gu, stream>>>(a, s.n_mid / 64, x_mid / 64, srow_gu, gu);
        IMX_CHECK_CUDA(cudaGetLastError());
        if (mid) IMX_CHECK_CUDA(cudaEventRecord(mid, stream));
        k_dn<<<sms, 256 + 32 * PW, smem_dn, stream>>>(a, s.n_in / 128, s.n_in / 128, srow_dn, dn);
        IMX_CHECK_CUDA(cudaGetLastError());
        return IMX_OK;
    };
    // 8 producer warps: 12 and 16 measured the same (the producers are not what the MMAs wait for)
    return run(std::integral_constant<int, 8>{});
}

}  // namespace imx
