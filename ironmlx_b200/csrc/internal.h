// Internal launcher declarations shared by the .cu files of the library.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace imx {

// A slice of one expert's sorted slots handled by one CTA pass of the decode
// kernels: `rows` consecutive slots starting at `slot0`, all of expert
// `expert` (== num_experts for the shared expert).
struct WorkUnit {
    int32_t expert;
    int32_t slot0;
    int32_t rows;
    int32_t pad;
};

// Order of the 16 values inside each block of an fp16 activation row.
// Stored pairs (2p, 2p+1) with odd p are multiplied by pair_scale_odd (1, or
// 1/16 for the decode kernel that reads 4-bit codes as fp16 subnormals).
struct Order16 {
    int8_t o[16];
    float pair_scale_odd;
};

// Ints cleared by the sort stage before every pass of the expert kernels:
// [0, 8) scheduler counters, then one "partial ready" flag per warp of the two
// stream-K decode kernels (kFlagWarps each), then the arrival counters of the
// tensor-map decode kernel's cut tile pairs (TmapRoom::pair_slots of them).
constexpr int kFlagWarps = 4096;
constexpr int kSchedFixed = 8 + 2 * kFlagWarps;
// Room of the tensor-map decode kernel's hand-off buffers: tile pairs whose reduction goes out in several
// chunks (only the last pairs of a launch do) and chunks per pair.
constexpr int kTmapFinePairs = 4096;
struct TmapRoom {
    int pair_slots;
    int cut;
};
TmapRoom decode_tmap_room(int n_in, int n_mid, int x_mid);
inline int sched_ints(const TmapRoom& r) { return kSchedFixed + r.pair_slots; }
constexpr int kUnitRows = 8;       // slots per decode work unit (the n=8 side of the MMA)

struct SortExtras {
    const float* topk_w = nullptr;
    int top_k = 1;
    int32_t* tok_of_slot = nullptr;
    float* w_of_slot = nullptr;
    const float* shared_gate = nullptr;
    int n_tokens = 0;                 // tokens the shared expert serves: slots [n_assign, n_assign + n_tokens)
    int shared_token0 = 0;            // ... namely tokens shared_token0 .. shared_token0 + n_tokens - 1
    WorkUnit* units = nullptr;
    int32_t* n_units = nullptr;
    int unit_rows = kUnitRows;
    int32_t* sched = nullptr;
    int sched_ints = kSchedFixed;     // words of sched to clear
};

// Workspace of the split-K router (decode sizes): all pointers together or none.
struct RouteScratch {
    float* partials;      // [H / route_slice(H)][32 ceil(n / 32)][E] partial logits
    float* sg_partials;   // [H / route_slice(H)][32 ceil(n / 32)] partial shared-gate dot products
    float* gsum_x;        // [n][H / 64] group sums of the fp16 copy in units of 2^-24, or nullptr
    const float* inv_rms; // [n] per-token RMSNorm factor: the tiles of x are normalised as they are loaded (or nullptr)
    const void* ln_weight;// bf16 [H] RMSNorm weight that goes with inv_rms (or nullptr)
};
constexpr int kRouteSplitMaxTokens = 1024;   // the split-K router serves batches below this
int route_slice(int H);                      // K slice of the split-K router (0: not applicable)

int launch_route(const void* x, int n, int H, const void* Wr, const float* logit_bias, int E, int k,
                 int norm, const void* w_sg, int32_t* topk_idx, float* topk_w, float* shared_gate,
                 void* x16, const int* order16, cudaStream_t stream, float pair_scale_odd = 1.f,
                 const RouteScratch* rs = nullptr, bool* sums_done = nullptr);

// Order of the 16 values of each block of an fp16 activation row as the
// expert kernels of a bit width read them (identity for the generic path).
void decode_block_order(int bits, int order[16]);
// The same for a format: affine widths by their unpack order, mxfp8 / nvfp4 in natural order.
void expert_block_order(const QFormat& f, int order[16]);

size_t sort_scratch_bytes(int n_assign, int E);
int launch_sort(const int32_t* ids, int A, int E, int32_t* counts, int32_t* offsets, int32_t* perm,
                int32_t* inv_perm, void* scratch, size_t scratch_bytes, const SortExtras* ex,
                cudaStream_t stream);

int launch_sort_static(const int32_t* ids, int A, int E, int32_t* counts, int32_t* offsets, int32_t* perm,
                       int32_t* inv_perm, cudaStream_t stream);

// Weights of the experts seen by the grouped kernels: `num_experts` stacked
// matrices plus one optional extra "expert" (id == num_experts) with its own
// pointers (the shared expert, whose gate and up projections are separate
// tensors).
struct ExpertSet {
    QFormat fmt;
    int num_experts;
    // first product: gate rows [0, n_mid) and up rows of the same expert
    QMat gate, up;                 // expert 0's matrices
    size_t gu_stride_w, gu_stride_s;   // bytes between consecutive experts
    QMat down;
    size_t dn_stride_w, dn_stride_s;
    int has_extra;
    QMat x_gate, x_up, x_down;     // the extra expert
    int n_in;                      // H
    int n_mid;                     // I   (routed experts)
    int x_mid;                     // Is  (extra expert)
};

// act[slot, :] = silu(gate_e(a)) * up_e(a), a = in[row_index[slot]] (fp16), act fp16.
// out[slot, :] = row_scale[slot] * down_e(act[slot]) (fp32).
struct GroupedArgs {
    ExpertSet set;
    const __half* in;              // fp16 [.., n_in]
    const int32_t* row_index;      // per slot, row of `in` (nullptr: slot itself)
    __half* xs;                    // [n_slots, n_in] scratch: `in` gathered into slot order (prefill path)
    int n_slots;                   // slots covered by row_index / act / out
    const WorkUnit* units;
    const int32_t* n_units;
    int max_units;
    int32_t* sched;                // [sched_ints(room)]: counters, the stream-K hand-off flags, the pair counters
    float* partials;               // [kFlagWarps][8][32] fp32 hand-off slots (stream-K decode kernels)
    float* psum;                   // [n_slots, act_stride / 16] fp32 sums of every 16 columns of the SwiGLU rows (tensor-map decode kernel)
    int32_t* pair_count;           // tensor-map decode kernel: arrivals per cut tile pair (sched + kSchedFixed), zero between launches
    float* pair_partials;          // ... and [pair_slots][pair_cut][8][32] fp32 partial sums of the pairs' chunks
    int pair_slots, pair_cut;      // room of the two (TmapRoom)
    float* gsum_x;                 // [n_in_rows, n_in / 64] fp32 group sums of the rows of `in`
    int n_in_rows;                 // rows of `in`
    const int32_t* n_rows_dev;     // device-side count of rows of `in` that are in use (nullptr: all n_in_rows)
    int gsum_x_ready;              // the router already filled gsum_x
    __half* act;                   // fp16 [n_slots, act_stride]
    int act_stride;
    const float* row_scale;        // per slot or nullptr
    float* out;                    // fp32 [n_slots, n_in]
    __half* out16;                 // prefill path only: the same rows as fp16 instead (out is then unused), or nullptr
    const int32_t* out_index;      // prefill path only: output row of each slot (nullptr: the slot itself)
    int32_t* status;               // device status word
    int second_only;               // run the second product alone: out = act . down^T (a plain quantized matmul)
    const int32_t* slots_end_dev;  // prefill path, optional: slots [*slots_end_dev, slots_resume) hold nothing (expert
    int slots_resume;              // parallelism: assignments of other ranks' experts); the gather skips them
};

bool decode_mma_supported(const ExpertSet& s);
// `mid`, when given, is recorded between the first and the second product.
int launch_decode_mma(const GroupedArgs& a, cudaStream_t stream, cudaEvent_t mid = nullptr);
// Tensor-map fed decode kernel (affine 4-bit, group 64); the preferred decode kernel where it applies.
bool decode_tmap_supported(const ExpertSet& s);
int launch_decode_tmap(const GroupedArgs& a, cudaStream_t stream, cudaEvent_t mid = nullptr);
void testing_decode_handoff(int spin_limit, int withhold);
// Decode kernel of the block-scaled float formats (mxfp8, nvfp4).
bool decode_fp_supported(const ExpertSet& s);
int launch_decode_fp(const GroupedArgs& a, cudaStream_t stream, cudaEvent_t mid = nullptr);
// Prefill path: work units of up to kPrefillUnitRows sorted slots on tcgen05/TMEM.
constexpr int kPrefillUnitRows = 256;
// Prefill path for every tensor-core format: the dequantized weights are the A operand, handed to the MMA
// through tensor memory.  variant 0: as shipped; 1: one weight tile per activation tile and streamed
// activations everywhere; 2: the dequantized tile through shared memory (1 and 2 are cross-checks).
bool prefill_tc_supported(const ExpertSet& s, bool second_only = false);
int launch_prefill_tc(const GroupedArgs& a, cudaStream_t stream, cudaEvent_t mid = nullptr, int variant = 0);
// The current device: its ordinal and SM count (cached per device).
struct DeviceInfo {
    int ordinal;
    int sms;
};
int current_device(DeviceInfo* out);
unsigned long long launch_count();   // kernels this library has launched (or recorded into a capture) so far
// One-time set-up per (device, kernel family): attributes such as the dynamic shared-memory limit are per
// device, so a process that drives several GPUs sets them on each.  The first call on a device should come
// before any stream capture.
enum { kSetupDecodeTmap = 0, kSetupPrefillTc = 1 };
bool device_needs_setup(int ordinal, int family);
void device_mark_setup(int ordinal, int family);
// Tiled TMA descriptor of a 2-D row-major matrix [rows, cols] of `esize`-byte elements, `ld_bytes` between
// rows, read in boxes of box_cols x box_rows (128-byte swizzle on request); reads past the end return zeros.
int make_tensor_map_2d(const void* base, CUtensorMapDataType dt, size_t esize, size_t rows, size_t cols,
                       size_t ld_bytes, int box_cols, int box_rows, bool swizzle128, CUtensorMap* out,
                       bool promote256 = false, int swizzle_bytes = 0);   // swizzle_bytes: 32 / 64 when swizzle128 is false
int launch_generic_grouped(const GroupedArgs& a, cudaStream_t stream, cudaEvent_t mid = nullptr);

// `residual` (bf16 [n, H] or nullptr) is added to the fp32 sums before the one rounding.
// rows / shared_rows are fp32, or fp16 with rows_f16 (the prefill path's expert rows).
int launch_combine(const void* rows, const float* row_scale, const int32_t* inv_perm, int n, int k, int H,
                   const void* shared_rows, void* y, cudaStream_t stream, bool f32_out = false,
                   const void* residual = nullptr, bool rows_f16 = false, const float* shared_scale = nullptr);
// (shared_scale: per-token factor of the shared rows when they arrive ungated; nullptr: already gated)
// y = w * T(x * rsqrt(mean(x^2) + eps)) per row (y may be null), inv_out[row] = the factor (may be null).
int launch_rms_norm(const void* x, int n, int H, const void* w, float eps, void* y, float* inv_out, cudaStream_t stream);
// dst[j, :] = src[index[j], :]; rows [*skip_from_dev, skip_to) are left alone when skip_from_dev is given
// (slots no expert of this rank owns).
int launch_gather_rows(const void* src, const int32_t* index, int n_rows, size_t row_bytes, void* dst,
                       cudaStream_t stream, const int32_t* skip_from_dev = nullptr, int skip_to = 0);

// Builds the unit list for a caller-given offsets array (stage-level API).  extra_from >= 0: the units of that
// (last) expert are listed as the extra expert's.
int launch_build_units(const int32_t* offsets, int E, int unit_rows, WorkUnit* units, int32_t* n_units,
                       int32_t* sched, int sched_ints, cudaStream_t stream, int extra_from = -1);

int launch_dequantize(const QMat& w, int rows, int in, QFormat f, int out_dtype, void* out,
                      cudaStream_t stream);
int launch_quantize(const float* w, int rows, int in, QFormat f, float gscale, void* wp, void* scales,
                    void* biases, cudaStream_t stream);
int launch_qmm(const void* x, int m, const QMat& w, int n_out, int in, int transpose, QFormat f, void* y,
               const int32_t* lhs_index, const int32_t* rhs_index, size_t w_stride, size_t s_stride,
               cudaStream_t stream);

int validate_format(int mode, int bits, int group, QFormat* out);

// ── pieces of the fused forward shared with the expert-parallel layer ─────────
// Hands out 256-byte aligned pieces of a caller-provided buffer (base == nullptr: only sizes).
struct Carver {
    uint8_t* base;
    size_t off = 0;
    explicit Carver(void* p) : base((uint8_t*)p) {}
    template <typename T>
    T* take(size_t count) {
        off = align_up(off, 256);
        T* p = base ? (T*)(base + off) : nullptr;
        off += count * sizeof(T);
        return p;
    }
};

// Scheduler words and the tensor-map decode kernel's hand-off buffers of a workspace, carved together.
struct SchedWs {
    int32_t* sched;
    int n_ints;
    float* pair_partials;
    TmapRoom room;
};
inline SchedWs carve_sched(Carver& cv, int n_in, int n_mid, int x_mid) {
    SchedWs w;
    w.room = decode_tmap_room(n_in, n_mid, x_mid);
    w.n_ints = sched_ints(w.room);
    w.sched = cv.take<int32_t>((size_t)w.n_ints);
    w.pair_partials = cv.take<float>((size_t)w.room.pair_slots * w.room.cut * 256);
    return w;
}
inline void use_sched(GroupedArgs& ga, const SchedWs& w) {
    ga.sched = w.sched;
    ga.pair_count = w.sched + kSchedFixed;
    ga.pair_partials = w.pair_partials;
    ga.pair_slots = w.room.pair_slots;
    ga.pair_cut = w.room.cut;
}
int check_config(const imx_moe_config* c, QFormat* f);
int make_expert_set(const imx_moe_config& c, const QFormat& f, const imx_qtensor& gate_up, const imx_qtensor& down,
                    int num_experts, const imx_moe_weights* shared, ExpertSet* out);
int pick_path(const imx_moe_config& c, const ExpertSet& s, long n_rows, int* path);
void path_block_order(int path, const QFormat& f, int order[16]);
int run_experts(int path, const GroupedArgs& ga, cudaStream_t stream, cudaEvent_t mid = nullptr);
bool is_prefill(int path);
int unit_rows_for(int path);
int max_units_for(int A, int E, int n_shared_tokens);

}  // namespace imx
