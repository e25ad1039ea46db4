// Router stage of the MoE block (mlx/src/nn/moe.rs:67-82 and :174-177):
//   logits = x . W_r^T  (bf16 inputs, fp32 accumulation)
//   probs  = softmax(logits) in fp32
//   top-k of probs in descending order, lower expert id first among equals
//   weights = probs[top] (/ their sum when norm_topk_prob)
//   shared gate = sigmoid(x . w_sg)
// plus an fp16 copy of x, the operand type of the expert products.
//
// One thread-block CLUSTER per token: the experts are split across the
// cluster's CTAs (so a 64-token decode batch still fills the GPU), partial
// logit vectors are written into the leader CTA's shared memory through
// distributed shared memory, and one warp of the leader does softmax/top-k
// with shuffle reductions.  HBM traffic is W_r once (L2-resident afterwards)
// plus x; the stage is latency-bound, not bandwidth-bound.
#include <cooperative_groups.h>

#include "decode_common.cuh"

namespace cg = cooperative_groups;

namespace imx {

namespace {

constexpr int kRouteThreads = 256;

// Block order of the fp16 copy by code width (0: rows stay as they are): position p of a block of 16 takes
// value order16<BITS>(p) of the source block.
template <int BITS>
__host__ __device__ constexpr int order16(int p) {
    if constexpr (BITS == 0) return p;
    else return decode::Codec<BITS>::order(p);
}
// Which of them `order` is, or -1.
inline int order_bits(const Order16& order) {
    const int widths[4] = {0, 4, 8, 2};
    for (int w = 0; w < 4; ++w) {
        bool same = true;
        for (int i = 0; i < 16; ++i) {
            const int want = widths[w] == 0 ? order16<0>(i) : (widths[w] == 4 ? order16<4>(i) : (widths[w] == 8 ? order16<8>(i) : order16<2>(i)));
            same = same && order.o[i] == want;
        }
        if (same) return widths[w];
    }
    return -1;
}
// One block of 16 bf16 values -> fp16 in block order BITS, pairs 1 and 3 of every 8 stored values times sc_odd:
// two 16-byte loads, the permutation in registers, two 16-byte stores.
template <int BITS>
__device__ __forceinline__ void convert_block16(const __nv_bfloat16* __restrict__ src, __half* __restrict__ dst, float sc_odd) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(src)), b = __ldg(reinterpret_cast<const uint4*>(src) + 1);
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float in[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        in[2 * i] = __uint_as_float(w[i] << 16);
        in[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
    uint32_t o[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        const float sc = (q & 1) ? sc_odd : 1.f;
        const __half2 h = __halves2half2(f32_to_f16_sat(in[order16<BITS>(2 * q)] * sc), f32_to_f16_sat(in[order16<BITS>(2 * q + 1)] * sc));
        o[q] = *reinterpret_cast<const uint32_t*>(&h);
    }
    reinterpret_cast<uint4*>(dst)[0] = make_uint4(o[0], o[1], o[2], o[3]);
    reinterpret_cast<uint4*>(dst)[1] = make_uint4(o[4], o[5], o[6], o[7]);
}


template <int JMAX>
__device__ void softmax_topk_warp(const float* s_logits, int E, int k, bool norm, int32_t* out_idx,
                                  float* out_w) {
    const int lane = threadIdx.x & 31;
    float p[JMAX];
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < JMAX; ++j) {
        int e = lane + 32 * j;
        p[j] = e < E ? s_logits[e] : -INFINITY;
        m = fmaxf(m, p[j]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < JMAX; ++j) {
        int e = lane + 32 * j;
        p[j] = e < E ? expf(p[j] - m) : 0.f;
        s += p[j];
    }
    s = warp_sum(s);
#pragma unroll
    for (int j = 0; j < JMAX; ++j) {
        int e = lane + 32 * j;
        p[j] = e < E ? p[j] / s : -1.f;   // -1 marks "not selectable"
    }
    float my_w = 0.f;
    int my_i = 0;
    float wsum = 0.f;
    // every lane keeps the best of its own candidates (lowest id first among equals); a round is then two
    // warp reductions (largest probability, lowest id that has it) and a rescan in the winning lane only.
    // Probabilities are >= 0 and the "taken" mark is -1, so the int view of the floats orders them.
    float bv;
    int bj;
    auto rescan = [&]() {
        bv = -1.f;
        bj = 0;
#pragma unroll
        for (int j = 0; j < JMAX; ++j) {
            if (p[j] > bv) {
                bv = p[j];
                bj = j;
            }
        }
    };
    rescan();
    for (int r = 0; r < k; ++r) {
        const int mine = __float_as_int(bv);
        const int top = __reduce_max_sync(0xffffffffu, mine);
        const int win = __reduce_min_sync(0xffffffffu, mine == top ? lane + 32 * bj : 0x7fffffff);
        const float wv = __int_as_float(top);
        if (mine == top && lane + 32 * bj == win) {
#pragma unroll
            for (int j = 0; j < JMAX; ++j)
                if (j == bj) p[j] = -1.f;
            rescan();
        }
        if (lane == (r & 31)) {
            my_w = wv;
            my_i = win;
        }
        wsum += wv;
        if ((r & 31) == 31 || r == k - 1) {      // flush up to 32 results
            int slot = (r & ~31) + lane;
            if (slot <= r) {
                out_idx[slot] = my_i;
                out_w[slot] = my_w;               // normalised below
            }
        }
    }
    __syncwarp();
    if (norm) {
        for (int slot = lane; slot < k; slot += 32) out_w[slot] = out_w[slot] / wsum;
    }
}

__global__ void __launch_bounds__(kRouteThreads)
route_kernel(const __nv_bfloat16* __restrict__ x, int H, const __nv_bfloat16* __restrict__ Wr,
             const float* __restrict__ logit_bias, int E, int k, int norm,
             const __nv_bfloat16* __restrict__ w_sg, int32_t* __restrict__ topk_idx,
             float* __restrict__ topk_w, float* __restrict__ shared_gate,
             __half* __restrict__ x16, const Order16 order) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* s_x = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    float* s_logits = reinterpret_cast<float*>(smem_raw + (size_t)H * 2);

    cg::cluster_group cluster = cg::this_cluster();
    const int cs = (int)cluster.num_blocks();
    const int rank = (int)cluster.block_rank();
    const int token = blockIdx.x / cs;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int nwarps = kRouteThreads / 32;

    const __nv_bfloat16* xr = x + (size_t)token * H;
    for (int c = tid * 8; c < H; c += kRouteThreads * 8) {
        uint4 v = *reinterpret_cast<const uint4*>(xr + c);
        *reinterpret_cast<uint4*>(s_x + c) = v;
    }
    __syncthreads();
    if (rank == 0 && x16 != nullptr) {
        // fp16 copy; inside every block of 16 the values are stored in the
        // order the expert kernels consume them (identity for the generic path)
        __half2* dst = reinterpret_cast<__half2*>(x16 + (size_t)token * H);
        for (int i = tid; i < H / 2; i += kRouteThreads) {
            const int blk = (2 * i) & ~15, p = (2 * i) & 15;
            const float sc = (i & 1) ? order.pair_scale_odd : 1.f;
            const float a = __bfloat162float(s_x[blk + order.o[p]]) * sc;
            const float b = __bfloat162float(s_x[blk + order.o[p + 1]]) * sc;
            dst[i] = __halves2half2(f32_to_f16_sat(a), f32_to_f16_sat(b));
        }
    }

    float* leader_logits = cluster.map_shared_rank(s_logits, 0);
    const int per = (E + cs - 1) / cs;
    const int e_lo = rank * per;
    const int e_hi = min(E, e_lo + per);
    // the last CTA of the cluster also owns the shared-gate dot product (index E)
    const int n_rows = (e_hi - e_lo) + ((rank == cs - 1 && w_sg != nullptr) ? 1 : 0);
    // Each warp takes kRowsPerPass weight rows at a time so that their loads
    // are independent and in flight together (the stage is latency-bound).
    constexpr int kRowsPerPass = 4;
    for (int r0 = warp * kRowsPerPass; r0 < n_rows; r0 += nwarps * kRowsPerPass) {
        const __nv_bfloat16* wrow[kRowsPerPass];
        float acc[kRowsPerPass];
#pragma unroll
        for (int j = 0; j < kRowsPerPass; ++j) {
            const int r = min(r0 + j, n_rows - 1);           // clamp: duplicates are discarded below
            wrow[j] = (e_lo + r >= e_hi) ? w_sg : Wr + (size_t)(e_lo + r) * H;
            acc[j] = 0.f;
        }
#pragma unroll 4
        for (int c = lane * 8; c < H; c += 256) {
            uint4 wv[kRowsPerPass];
#pragma unroll
            for (int j = 0; j < kRowsPerPass; ++j) wv[j] = __ldg(reinterpret_cast<const uint4*>(wrow[j] + c));
            const uint4 xv = *reinterpret_cast<const uint4*>(s_x + c);
            const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
            for (int j = 0; j < kRowsPerPass; ++j) {
                const __nv_bfloat162* wb = reinterpret_cast<const __nv_bfloat162*>(&wv[j]);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 wf = __bfloat1622float2(wb[i]);
                    const float2 xf = __bfloat1622float2(xb[i]);
                    acc[j] = fmaf(wf.x, xf.x, acc[j]);
                    acc[j] = fmaf(wf.y, xf.y, acc[j]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < kRowsPerPass; ++j) {
            const float v = warp_sum(acc[j]);
            const int r = r0 + j;
            if (lane == 0 && r < n_rows) {
                if (e_lo + r >= e_hi) {
                    shared_gate[token] = 1.0f / (1.0f + expf(-v));
                } else {
                    leader_logits[e_lo + r] = v + (logit_bias != nullptr ? logit_bias[e_lo + r] : 0.f);
                }
            }
        }
    }
    cluster.sync();
    if (rank == 0 && warp == 0) {
        int32_t* oi = topk_idx + (size_t)token * k;
        float* ow = topk_w + (size_t)token * k;
        const int j = (E + 31) / 32;
        if (j <= 1) softmax_topk_warp<1>(s_logits, E, k, norm, oi, ow);
        else if (j <= 2) softmax_topk_warp<2>(s_logits, E, k, norm, oi, ow);
        else if (j <= 4) softmax_topk_warp<4>(s_logits, E, k, norm, oi, ow);
        else if (j <= 8) softmax_topk_warp<8>(s_logits, E, k, norm, oi, ow);
        else if (j <= 16) softmax_topk_warp<16>(s_logits, E, k, norm, oi, ow);
        else softmax_topk_warp<32>(s_logits, E, k, norm, oi, ow);
    }
}


// ── prefill-size router: logits on the tensor cores ─────────────────────────
// 32 tokens x all experts per CTA with mma.sync m16n8k16 (bf16 x bf16 -> fp32):
// activations and router rows stream through shared memory in K chunks of 64
// (16-byte cp.async, double buffered), the fp32 logits of the tile land in
// shared memory and each warp finishes its share of the tokens with the same
// warp softmax/top-k as the decode-size kernel.  W warps per CTA: each takes
// E / W experts of the product and 32 / W tokens of the epilogue (eight warps
// from 64 experts on: the epilogue is half of the kernel's time and serial per
// warp).
constexpr int kRT = 32;            // tokens per CTA
constexpr int kRK = 64;            // K chunk
constexpr int kRPad = 72;          // bf16 per smem row (64 + 8: conflict-free fragment loads)

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NT, int W>   // E = 32 * NT experts, W warps
__global__ void __launch_bounds__(W * 32)
route_mma_kernel(const __nv_bfloat16* __restrict__ x, int n_tokens, int H, const __nv_bfloat16* __restrict__ Wr,
                 const float* __restrict__ logit_bias, int k, int norm, const __nv_bfloat16* __restrict__ w_sg,
                 int32_t* __restrict__ topk_idx, float* __restrict__ topk_w, float* __restrict__ shared_gate,
                 __half* __restrict__ x16, const Order16 order, const int obits) {
    constexpr int E = 32 * NT;
    constexpr int kRThreads = W * 32;
    constexpr int NW = 4 * NT / W;            // n-tiles of 8 experts per warp
    static_assert(NW >= 1 && NW * W == 4 * NT, "experts must divide evenly over the warps");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* s_x = reinterpret_cast<__nv_bfloat16*>(smem_raw);                 // [2][kRT][kRPad]
    __nv_bfloat16* s_w = s_x + 2 * kRT * kRPad;                                      // [2][E][kRPad]
    float* s_logits = reinterpret_cast<float*>(smem_raw);                            // [kRT][E] (reuses the buffers)
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int tok0 = blockIdx.x * kRT;

    auto load_chunk = [&](int buf, int kc) {
        // activations: 32 rows x 8 chunks of 16 bytes
        for (int c = tid; c < kRT * 8; c += kRThreads) {
            const int r = c >> 3, ch = c & 7;
            const int tok = tok0 + r;
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(s_x + (buf * kRT + r) * kRPad + ch * 8);
            const __nv_bfloat16* src = x + (size_t)(tok < n_tokens ? tok : 0) * H + kc * kRK + ch * 8;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(tok < n_tokens ? 16 : 0) : "memory");
        }
        for (int c = tid; c < E * 8; c += kRThreads) {
            const int r = c >> 3, ch = c & 7;
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(s_w + (buf * E + r) * kRPad + ch * 8);
            const __nv_bfloat16* src = Wr + (size_t)r * H + kc * kRK + ch * 8;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, 16;" ::"r"(dst), "l"(src) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float acc[2][NW][4];
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int n = 0; n < NW; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[m][n][i] = 0.f;

    const int nchunks = H / kRK;
    load_chunk(0, 0);
    for (int kc = 0; kc < nchunks; ++kc) {
        const int buf = kc & 1;
        if (kc + 1 < nchunks) {
            load_chunk(buf ^ 1, kc + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const __nv_bfloat16* xs = s_x + buf * kRT * kRPad;
        const __nv_bfloat16* ws = s_w + (buf * E + warp * (8 * NW)) * kRPad;
#pragma unroll
        for (int kk = 0; kk < kRK / 16; ++kk) {
            uint32_t af[2][4];
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                const __nv_bfloat16* p = xs + (m * 16 + g) * kRPad + kk * 16 + 2 * t;
                af[m][0] = *reinterpret_cast<const uint32_t*>(p);
                af[m][1] = *reinterpret_cast<const uint32_t*>(p + 8 * kRPad);
                af[m][2] = *reinterpret_cast<const uint32_t*>(p + 8);
                af[m][3] = *reinterpret_cast<const uint32_t*>(p + 8 * kRPad + 8);
            }
#pragma unroll
            for (int n = 0; n < NW; ++n) {
                const __nv_bfloat16* p = ws + (n * 8 + g) * kRPad + kk * 16 + 2 * t;
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(p);
                const uint32_t b1 = *reinterpret_cast<const uint32_t*>(p + 8);
                mma_bf16(acc[0][n], af[0][0], af[0][1], af[0][2], af[0][3], b0, b1);
                mma_bf16(acc[1][n], af[1][0], af[1][1], af[1][2], af[1][3], b0, b1);
            }
        }
        __syncthreads();
    }
    // logits (+ bias) of the tile into shared memory
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int n = 0; n < NW; ++n) {
            const int e = warp * (8 * NW) + n * 8 + 2 * t;
            const float b0 = logit_bias ? logit_bias[e] : 0.f, b1 = logit_bias ? logit_bias[e + 1] : 0.f;
            s_logits[(m * 16 + g) * E + e] = acc[m][n][0] + b0;
            s_logits[(m * 16 + g) * E + e + 1] = acc[m][n][1] + b1;
            s_logits[(m * 16 + g + 8) * E + e] = acc[m][n][2] + b0;
            s_logits[(m * 16 + g + 8) * E + e + 1] = acc[m][n][3] + b1;
        }
    __syncthreads();
    // each warp finishes its tokens: softmax/top-k, shared gate, fp16 copy
    for (int r = warp * (kRT / W); r < (warp + 1) * (kRT / W); ++r) {
        const int tok = tok0 + r;
        if (tok >= n_tokens) break;
        softmax_topk_warp<NT>(s_logits + r * E, E, k, norm, topk_idx + (size_t)tok * k, topk_w + (size_t)tok * k);
        const __nv_bfloat16* xr = x + (size_t)tok * H;
        if (w_sg != nullptr) {
            float acc_g = 0.f;
            for (int c = lane * 8; c < H; c += 256) {
                const uint4 xv = __ldg(reinterpret_cast<const uint4*>(xr + c));
                const uint4 wv = __ldg(reinterpret_cast<const uint4*>(w_sg + c));
                const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&xv);
                const __nv_bfloat162* wb = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 xf = __bfloat1622float2(xb[i]), wf = __bfloat1622float2(wb[i]);
                    acc_g = fmaf(xf.x, wf.x, acc_g);
                    acc_g = fmaf(xf.y, wf.y, acc_g);
                }
            }
            acc_g = warp_sum(acc_g);
            if (lane == 0) shared_gate[tok] = 1.0f / (1.0f + expf(-acc_g));
        }
        if (x16 != nullptr && obits >= 0) {
            // a block of 16 per lane at a time, in the order the expert kernels of this code width read
            __half* dst = x16 + (size_t)tok * H;
            for (int c = lane * 16; c < H; c += 32 * 16) {
                if (obits == 4) convert_block16<4>(xr + c, dst + c, order.pair_scale_odd);
                else if (obits == 8) convert_block16<8>(xr + c, dst + c, order.pair_scale_odd);
                else if (obits == 2) convert_block16<2>(xr + c, dst + c, order.pair_scale_odd);
                else convert_block16<0>(xr + c, dst + c, order.pair_scale_odd);
            }
        } else if (x16 != nullptr) {
            __half2* dst = reinterpret_cast<__half2*>(x16 + (size_t)tok * H);
            for (int i = lane; i < H / 2; i += 32) {
                const int blk = (2 * i) & ~15, p = (2 * i) & 15;
                const float sc = (i & 1) ? order.pair_scale_odd : 1.f;
                const float a = __bfloat162float(xr[blk + order.o[p]]) * sc;
                const float b = __bfloat162float(xr[blk + order.o[p + 1]]) * sc;
                dst[i] = __halves2half2(f32_to_f16_sat(a), f32_to_f16_sat(b));
            }
        }
    }
}


// ── decode-size router on the tensor cores, split over K ────────────────────
// One CTA per (32 experts, K slice, 32 tokens): the two bf16 tiles are copied to
// shared memory once, multiplied with mma.sync m16n8k16, and the fp32 partial
// logits go to the workspace; route_finish_kernel adds the slices and does
// softmax/top-k with one warp per token.  Every CTA also writes, for a few
// token rows of its tile, the K slice of the fp16 copy of x, its group sums
// (for the decode expert kernels) and the partial shared-gate dot product.  W_r is read once
// per token block instead of once per token.
constexpr int kSkThreads = 128;

__global__ void __launch_bounds__(kSkThreads)
route_splitk_kernel(const __nv_bfloat16* __restrict__ x, int n_tokens, int H, const __nv_bfloat16* __restrict__ Wr,
                    const float* __restrict__ logit_bias, int E, int k, int norm, const __nv_bfloat16* __restrict__ w_sg,
                    int32_t* __restrict__ topk_idx, float* __restrict__ topk_w, float* __restrict__ shared_gate,
                    __half* __restrict__ x16, const Order16 order, int ks, const RouteScratch rs) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int pad = ks + 8;                                                          // bf16 per row: conflict-free fragment loads
    __nv_bfloat16* s_x = reinterpret_cast<__nv_bfloat16*>(smem_raw);                 // [32][pad]
    __nv_bfloat16* s_w = s_x + 32 * pad;                                             // [32][pad]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int eb = blockIdx.x, split = blockIdx.y, tb = blockIdx.z;
    const int n_pad = gridDim.z * 32;
    const int tok0 = tb * 32, k0 = split * ks;

    const int cpr = ks >> 3;                                                         // 16-byte pieces per row
    for (int c = tid; c < 32 * cpr; c += kSkThreads) {
        const int r = c / cpr, ch = c - r * cpr;
        const int tok = tok0 + r;
        const uint32_t dx = (uint32_t)__cvta_generic_to_shared(s_x + r * pad + ch * 8);
        const __nv_bfloat16* sx = x + (size_t)(tok < n_tokens ? tok : 0) * H + k0 + ch * 8;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dx), "l"(sx), "r"(tok < n_tokens ? 16 : 0) : "memory");
        const uint32_t dw = (uint32_t)__cvta_generic_to_shared(s_w + r * pad + ch * 8);
        const __nv_bfloat16* sw = Wr + (size_t)(eb * 32 + r) * H + k0 + ch * 8;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, 16;" ::"r"(dw), "l"(sw) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    if (rs.inv_rms != nullptr) {
        // the block's input is RMSNorm(x): normalise the tile in place (everything below reads the tile)
        const __nv_bfloat16* lw = reinterpret_cast<const __nv_bfloat16*>(rs.ln_weight);
        for (int c = tid; c < 32 * ks; c += kSkThreads) {
            const int r = c / ks, col = c - r * ks;
            const int tok = tok0 + r;
            if (tok < n_tokens)
                s_x[r * pad + col] = rms_norm_apply(s_x[r * pad + col], rs.inv_rms[tok], lw ? lw[k0 + col] : s_x[0], lw != nullptr);
        }
        __syncthreads();
    }

    float acc[2][4];
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[m][i] = 0.f;
    const __nv_bfloat16* ws = s_w + (warp * 8 + g) * pad + 2 * t;
    for (int kk = 0; kk < ks; kk += 16) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(ws + kk);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(ws + kk + 8);
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            const __nv_bfloat16* p = s_x + (m * 16 + g) * pad + kk + 2 * t;
            mma_bf16(acc[m], *reinterpret_cast<const uint32_t*>(p), *reinterpret_cast<const uint32_t*>(p + 8 * pad),
                     *reinterpret_cast<const uint32_t*>(p + 8), *reinterpret_cast<const uint32_t*>(p + 8 * pad + 8), b0, b1);
        }
    }
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        const int e = eb * 32 + warp * 8 + 2 * t;
        float* p = rs.partials + ((size_t)split * n_pad + tok0 + m * 16 + g) * E + e;
        *reinterpret_cast<float2*>(p) = make_float2(acc[m][0], acc[m][1]);
        *reinterpret_cast<float2*>(p + (size_t)8 * E) = make_float2(acc[m][2], acc[m][3]);
    }

    {
        // fp16 copy, group sums and shared-gate partial of this K slice: the token rows of the tile are dealt
        // out over the expert-block CTAs (row r goes to CTA r mod #blocks), then over the CTA's warps
        const int groups = H >> 6;
        for (int r = eb + warp * (int)gridDim.x; r < 32; r += 4 * (int)gridDim.x) {
            const int tok = tok0 + r;
            if (tok >= n_tokens) break;
            const __nv_bfloat16* xr = s_x + r * pad;
            if (x16 != nullptr) {
                // fp16 copy of the slice in the expert kernels' order; 32 pairs = one group of 64 per pass
                __half2* dst = reinterpret_cast<__half2*>(x16 + (size_t)tok * H + k0);
                for (int q = 0; q < (ks >> 6); ++q) {
                    const int i = q * 32 + lane;
                    const int blk = (2 * i) & ~15, p = (2 * i) & 15;
                    const float sc = (i & 1) ? order.pair_scale_odd : 1.f;
                    const __half2 h = __halves2half2(f32_to_f16_sat(__bfloat162float(xr[blk + order.o[p]]) * sc),
                                                     f32_to_f16_sat(__bfloat162float(xr[blk + order.o[p + 1]]) * sc));
                    dst[i] = h;
                    if (rs.gsum_x != nullptr) {
                        // sum of the values the products will see, in units of 2^-24
                        const float2 f = __half22float2(h);
                        float v = f.x + f.y;
                        if ((i & 1) && order.pair_scale_odd != 1.f) v *= 1.f / order.pair_scale_odd;
                        v = warp_sum(v);
                        if (lane == 0) rs.gsum_x[(size_t)tok * groups + (k0 >> 6) + q] = v * 5.9604644775390625e-8f;
                    }
                }
            }
            if (w_sg != nullptr) {
                float accg = 0.f;
                for (int c = lane * 8; c < ks; c += 256) {
                    const uint4 xv = *reinterpret_cast<const uint4*>(xr + c);
                    const uint4 wv = __ldg(reinterpret_cast<const uint4*>(w_sg + k0 + c));
                    const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&xv);
                    const __nv_bfloat162* wb = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 xf = __bfloat1622float2(xb[i]), wf = __bfloat1622float2(wb[i]);
                        accg = fmaf(xf.x, wf.x, accg);
                        accg = fmaf(xf.y, wf.y, accg);
                    }
                }
                accg = warp_sum(accg);
                if (lane == 0) rs.sg_partials[(size_t)split * n_pad + tok] = accg;
            }
        }
    }

}

// Second half of the split-K router: one warp per token adds the K slices in slice
// order (so the sums do not depend on timing) and does softmax / top-k.
__global__ void __launch_bounds__(kSkThreads)
route_finish_kernel(int n_tokens, int n_pad, int n_splits, const float* __restrict__ logit_bias, int E, int k, int norm,
                    int has_sg, int32_t* __restrict__ topk_idx, float* __restrict__ topk_w,
                    float* __restrict__ shared_gate, const RouteScratch rs) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* my_logits = reinterpret_cast<float*>(smem_raw) + warp * E;
    const int tok = blockIdx.x * (kSkThreads / 32) + warp;
    if (tok >= n_tokens) return;
    // 4 experts per lane and pass (16-byte loads), all slices of a pass in flight together
    for (int e = lane * 4; e < E; e += 128) {
        const float* p = rs.partials + (size_t)tok * E + e;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s0 = 0; s0 < n_splits; s0 += 8) {
            float4 part[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                part[u] = s0 + u < n_splits ? __ldcg(reinterpret_cast<const float4*>(p + (size_t)(s0 + u) * n_pad * E))
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                v.x += part[u].x; v.y += part[u].y; v.z += part[u].z; v.w += part[u].w;
            }
        }
        if (logit_bias != nullptr) {
            v.x += logit_bias[e]; v.y += logit_bias[e + 1]; v.z += logit_bias[e + 2]; v.w += logit_bias[e + 3];
        }
        *reinterpret_cast<float4*>(my_logits + e) = v;
    }
    __syncwarp();
    int32_t* oi = topk_idx + (size_t)tok * k;
    float* ow = topk_w + (size_t)tok * k;
    const int j = (E + 31) / 32;
    if (j <= 1) softmax_topk_warp<1>(my_logits, E, k, norm, oi, ow);
    else if (j <= 2) softmax_topk_warp<2>(my_logits, E, k, norm, oi, ow);
    else if (j <= 4) softmax_topk_warp<4>(my_logits, E, k, norm, oi, ow);
    else if (j <= 8) softmax_topk_warp<8>(my_logits, E, k, norm, oi, ow);
    else if (j <= 16) softmax_topk_warp<16>(my_logits, E, k, norm, oi, ow);
    else softmax_topk_warp<32>(my_logits, E, k, norm, oi, ow);
    if (has_sg && lane == 0) {
        float v = 0.f;
        for (int s = 0; s < n_splits; ++s) v += __ldcg(rs.sg_partials + (size_t)s * n_pad + tok);
        shared_gate[tok] = 1.0f / (1.0f + expf(-v));
    }
}

template <int NT>
int launch_route_mma(const void* x, int n, int H, const void* Wr, const float* logit_bias, int k, int norm,
                     const void* w_sg, int32_t* topk_idx, float* topk_w, float* shared_gate, void* x16,
                     const Order16& order, cudaStream_t stream) {
    constexpr int E = 32 * NT;
    const size_t stage = (size_t)2 * (kRT + E) * kRPad * sizeof(__nv_bfloat16);
    const size_t logits = (size_t)kRT * E * sizeof(float);
    const size_t smem = stage > logits ? stage : logits;
    constexpr int W = NT >= 2 ? 8 : 4;
    IMX_CHECK_CUDA(cudaFuncSetAttribute(route_mma_kernel<NT, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    route_mma_kernel<NT, W><<<ceil_div(n, kRT), W * 32, smem, stream>>>(
        (const __nv_bfloat16*)x, n, H, (const __nv_bfloat16*)Wr, logit_bias, k, norm, (const __nv_bfloat16*)w_sg,
        topk_idx, topk_w, shared_gate, (__half*)x16, order,
        ((uintptr_t)x % 16 == 0 && (uintptr_t)x16 % 16 == 0) ? order_bits(order) : -1); IMX_LAUNCHED();
    IMX_CHECK_CUDA(cudaGetLastError());
    return IMX_OK;
}

}  // namespace

int route_slice(int H) {
    if (H % 256 == 0 && H / 256 <= 32) return 256;
    if (H % 128 == 0 && H / 128 <= 32) return 128;
    if (H % 64 == 0 && H / 64 <= 32) return 64;
    return 0;
}

int launch_route(const void* x, int n, int H, const void* Wr, const float* logit_bias, int E, int k,
                 int norm, const void* w_sg, int32_t* topk_idx, float* topk_w, float* shared_gate,
                 void* x16, const int* order16, cudaStream_t stream, float pair_scale_odd, const RouteScratch* rs,
                 bool* sums_done) {
    IMX_REQUIRE(n >= 0 && H > 0 && H % 16 == 0, "route: hidden (%d) must be a positive multiple of 16", H);
    Order16 order;
    for (int i = 0; i < 16; ++i) order.o[i] = (int8_t)(order16 ? order16[i] : i);
    order.pair_scale_odd = pair_scale_odd;
    IMX_REQUIRE(E >= 1 && E <= 1024, "route: num_experts (%d) must be in 1..1024", E);
    IMX_REQUIRE(k >= 1 && k <= E, "route: top_k (%d) must be in 1..num_experts (%d)", k, E);
    IMX_REQUIRE(w_sg == nullptr || shared_gate != nullptr, "route: shared gate weight without output");
    if (sums_done != nullptr) *sums_done = false;
    if (n == 0) return IMX_OK;
    const int ks = route_slice(H);
    if (rs != nullptr && rs->partials != nullptr && n < kRouteSplitMaxTokens && ks > 0 && E % 32 == 0 && x16 != nullptr) {
        const size_t tiles = (size_t)2 * 32 * (ks + 8) * sizeof(__nv_bfloat16);
        const dim3 grid((unsigned)(E / 32), (unsigned)(H / ks), (unsigned)ceil_div(n, 32));
        route_splitk_kernel<<<grid, kSkThreads, tiles, stream>>>(
            (const __nv_bfloat16*)x, n, H, (const __nv_bfloat16*)Wr, logit_bias, E, k, norm, (const __nv_bfloat16*)w_sg,
            topk_idx, topk_w, shared_gate, (__half*)x16, order, ks, *rs); IMX_LAUNCHED();
        IMX_CHECK_CUDA(cudaGetLastError());
        route_finish_kernel<<<ceil_div(n, kSkThreads / 32), kSkThreads, (size_t)(kSkThreads / 32) * E * sizeof(float), stream>>>(
            n, (int)grid.z * 32, (int)grid.y, logit_bias, E, k, norm, w_sg != nullptr, topk_idx, topk_w, shared_gate, *rs); IMX_LAUNCHED();
        IMX_CHECK_CUDA(cudaGetLastError());
        if (sums_done != nullptr) *sums_done = rs->gsum_x != nullptr;
        return IMX_OK;
    }
    if (n >= 256 && H % kRK == 0 && E % 32 == 0 && E <= 256) {
        switch (E / 32) {
            case 1: return launch_route_mma<1>(x, n, H, Wr, logit_bias, k, norm, w_sg, topk_idx, topk_w, shared_gate, x16, order, stream);
            case 2: return launch_route_mma<2>(x, n, H, Wr, logit_bias, k, norm, w_sg, topk_idx, topk_w, shared_gate, x16, order, stream);
            case 4: return launch_route_mma<4>(x, n, H, Wr, logit_bias, k, norm, w_sg, topk_idx, topk_w, shared_gate, x16, order, stream);
            case 8: return launch_route_mma<8>(x, n, H, Wr, logit_bias, k, norm, w_sg, topk_idx, topk_w, shared_gate, x16, order, stream);
            default: break;
        }
    }
    // cluster size: enough CTAs to cover the GPU at small N, experts split evenly
    int cs = 1;
    while (cs < 8 && (long)n * cs < 296 && E / (cs * 2) >= 16) cs *= 2;
    size_t smem = (size_t)H * 2 + (size_t)E * 4;
    IMX_REQUIRE(smem <= 200 * 1024, "route: hidden %d / experts %d exceed shared memory", H, E);
    IMX_CHECK_CUDA(cudaFuncSetAttribute(route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)(n * cs));
    lc.blockDim = dim3(kRouteThreads);
    lc.dynamicSmemBytes = smem;
    lc.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cs;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    lc.attrs = attr;
    lc.numAttrs = 1;
    IMX_CHECK_CUDA(cudaLaunchKernelEx(&lc, route_kernel, (const __nv_bfloat16*)x, H,
                                      (const __nv_bfloat16*)Wr, logit_bias, E, k, norm,
                                      (const __nv_bfloat16*)w_sg, topk_idx, topk_w, shared_gate,
                                      (__half*)x16, order));
    return IMX_OK;
}

}  // namespace imx
