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
#include "decode_common.cuh"

namespace imx {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kStages = 4;          // register prefetch depth (iterations of 128 codes)

using namespace decode;

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
    if (!a.second_only) {
        decode_mma_kernel<BITS, true><<<grid, kThreads, 0, stream>>>(a, mid_max / 16, g128); IMX_LAUNCHED();
        IMX_CHECK_CUDA(cudaGetLastError());
    }
    if (mid) IMX_CHECK_CUDA(cudaEventRecord(mid, stream));
    decode_mma_kernel<BITS, false><<<grid, kThreads, 0, stream>>>(a, s.n_in / 32, g128); IMX_LAUNCHED();
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

void expert_block_order(const QFormat& f, int order[16]) {
    decode_block_order(f.mode == IMX_MODE_AFFINE ? f.bits : 0, order);
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
