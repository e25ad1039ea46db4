// extern "C" entry points (include/ironmlx_b200.h): argument validation,
// workspace carving and stage orchestration.  No device allocation happens
// here; every scratch byte comes from the caller's workspace.
#include <cstring>

#include "internal.h"
#include "../../include/ironmlx_b200_testing.h"

namespace imx {

static thread_local std::string g_error;

void set_error(const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_error = buf;
}
const char* last_error() { return g_error.c_str(); }

// (the helpers below are shared with the expert-parallel layer, ep.cu: declared in internal.h)

// Workspace of the fused forward.
struct ForwardWs {
    int32_t* status;      // [16]: [0] device status word
    SchedWs sw;           // scheduler words and the tensor-map decode kernel's hand-off buffers
    int32_t* n_units;     // [4]: total, routed
    float* partials;      // [kFlagWarps][256] hand-off slots of the stream-K decode kernels
    float* psum;          // [A + N, act_stride / 16] sums of every 16 columns of the SwiGLU rows (tensor-map decode kernel)
    float* gsum_x;        // [N, H / 64] group sums of the fp16 copy of x
    float* inv_rms;          // [N] RMSNorm factor per token (decoder-layer tail)
    __nv_bfloat16* xn;       // [N, H] normalised input where the router cannot normalise its own tiles
    float* route_partials;   // split-K router: [splits][32 ceil(N / 32)][E]
    float* route_sg;         // split-K router: [splits][32 ceil(N / 32)]
    int32_t* topk_idx;    // [A]
    float* topk_w;        // [A]
    float* shared_gate;   // [N]
    __half* x16;          // [N, H]
    int32_t* counts;      // [E]
    int32_t* offsets;     // [E+1]
    int32_t* perm;        // [A]
    int32_t* inv_perm;    // [A]
    int32_t* tok_of_slot; // [A + N]
    float* w_of_slot;     // [A + N]
    WorkUnit* units;      // [max_units]
    void* sort_scratch;
    size_t sort_scratch_bytes;
    __half* act;          // [A + N, act_stride]
    __half* xs;           // [A + N, H] activations in slot order (prefill path)
    float* rows;          // [A + N, H]
    int max_units;
    int act_stride;
    size_t bytes;
};

int max_units_for(int A, int E, int n_shared_tokens) {
    return (A + kUnitRows - 1) / kUnitRows + E + (n_shared_tokens + kUnitRows - 1) / kUnitRows + 1;
}

ForwardWs carve_forward(const imx_moe_config& c, int n, void* base) {
    ForwardWs w = {};
    const int A = n * c.top_k;
    const int ns = c.shared_intermediate > 0 ? n : 0;
    Carver cv(base);
    w.status = cv.take<int32_t>(16);
    w.max_units = max_units_for(A, c.num_experts, ns);
    w.sw = carve_sched(cv, c.hidden, c.intermediate, c.shared_intermediate);
    w.n_units = cv.take<int32_t>(4);
    w.partials = cv.take<float>((size_t)kFlagWarps * 256);
    w.topk_idx = cv.take<int32_t>(A);
    w.topk_w = cv.take<float>(A);
    w.shared_gate = cv.take<float>(n);
    w.x16 = cv.take<__half>((size_t)n * c.hidden);
    w.counts = cv.take<int32_t>(c.num_experts);
    w.offsets = cv.take<int32_t>(c.num_experts + 1);
    w.perm = cv.take<int32_t>(A);
    w.inv_perm = cv.take<int32_t>(A);
    w.tok_of_slot = cv.take<int32_t>(A + ns);
    w.w_of_slot = cv.take<float>(A + ns);
    w.units = cv.take<WorkUnit>(w.max_units);
    w.sort_scratch_bytes = sort_scratch_bytes(A, c.num_experts);
    w.sort_scratch = cv.take<uint8_t>(w.sort_scratch_bytes);
    w.act_stride = c.intermediate > c.shared_intermediate ? c.intermediate : c.shared_intermediate;
    w.act = cv.take<__half>((size_t)(A + ns) * w.act_stride);
    w.xs = cv.take<__half>((size_t)(A + ns) * c.hidden);
    w.rows = cv.take<float>((size_t)(A + ns) * c.hidden);
    w.psum = cv.take<float>((size_t)(A + ns) * (w.act_stride / 16 + 1));
    w.gsum_x = cv.take<float>((size_t)n * (c.hidden / 64 + 1));
    w.inv_rms = cv.take<float>((size_t)n);
    w.xn = cv.take<__nv_bfloat16>((size_t)n * c.hidden);
    const int slice = route_slice(c.hidden);
    if (n < kRouteSplitMaxTokens && slice > 0) {
        const size_t splits = (size_t)c.hidden / slice, n_pad = (size_t)(n + 31) / 32 * 32;
        w.route_partials = cv.take<float>(splits * n_pad * c.num_experts);
        w.route_sg = cv.take<float>(splits * n_pad);
    }
    w.bytes = align_up(cv.off, 256);
    return w;
}

int check_config(const imx_moe_config* c, QFormat* f) {
    IMX_REQUIRE(c != nullptr, "config is NULL");
    IMX_TRY(validate_format(c->mode, c->bits, c->group_size, f));
    IMX_REQUIRE(c->hidden > 0 && c->hidden % 16 == 0, "hidden (%d) must be a positive multiple of 16", c->hidden);
    IMX_REQUIRE(c->num_experts >= 1 && c->num_experts <= 1023, "num_experts (%d) must be in 1..1023", c->num_experts);
    IMX_REQUIRE(c->top_k >= 1 && c->top_k <= c->num_experts && c->top_k <= 64,
                "top_k (%d) must be in 1..min(num_experts, 64)", c->top_k);
    IMX_REQUIRE(c->intermediate > 0 && c->intermediate % f->group == 0 && c->intermediate % 8 == 0,
                "intermediate (%d) must be a positive multiple of the group size and of 8", c->intermediate);
    IMX_REQUIRE(c->shared_intermediate >= 0 && c->shared_intermediate % f->group == 0 &&
                    c->shared_intermediate % 8 == 0,
                "shared_intermediate (%d) must be a multiple of the group size and of 8", c->shared_intermediate);
    IMX_REQUIRE(c->hidden % f->group == 0, "hidden (%d) must be a multiple of the group size (%d)", c->hidden, f->group);
    IMX_REQUIRE(c->path >= IMX_PATH_AUTO && c->path <= IMX_PATH_PREFILL_SMEM, "unknown path %d", c->path);
    return IMX_OK;
}

QMat to_qmat(const imx_qtensor& t) {
    QMat m;
    m.w = (const uint8_t*)t.w;
    m.scales = (const uint8_t*)t.scales;
    m.biases = (const uint8_t*)t.biases;
    m.global_scale = t.global_scale == 0.f ? 1.f : t.global_scale;
    return m;
}

int check_qtensor(const imx_qtensor& t, const QFormat& f, const char* name) {
    IMX_REQUIRE(t.w != nullptr && t.scales != nullptr, "%s: weight and scales are required", name);
    IMX_REQUIRE(f.mode != IMX_MODE_AFFINE || t.biases != nullptr, "%s: affine mode needs biases", name);
    IMX_REQUIRE(((uintptr_t)t.w % 16) == 0 && ((uintptr_t)t.scales % 4) == 0 &&
                    (t.biases == nullptr || ((uintptr_t)t.biases % 4) == 0),
                "%s: tensors must be 16-byte (weights) / 4-byte (scales, biases) aligned", name);
    return IMX_OK;
}

// Fills an ExpertSet from stacked gate_up / down tensors (+ optional shared expert).
int make_expert_set(const imx_moe_config& c, const QFormat& f, const imx_qtensor& gate_up,
                    const imx_qtensor& down, int num_experts, const imx_moe_weights* shared, ExpertSet* out) {
    ExpertSet s = {};
    s.fmt = f;
    s.num_experts = num_experts;
    s.n_in = c.hidden;
    s.n_mid = c.intermediate;
    IMX_TRY(check_qtensor(gate_up, f, "gate_up"));
    IMX_TRY(check_qtensor(down, f, "down"));
    const size_t gu_row_w = packed_row_bytes(c.hidden, f.bits), gu_row_s = scale_row_bytes(c.hidden, f);
    const size_t dn_row_w = packed_row_bytes(c.intermediate, f.bits), dn_row_s = scale_row_bytes(c.intermediate, f);
    s.gate = to_qmat(gate_up);
    s.up = s.gate;                                   // up rows follow the I gate rows (qwen35.rs:674-687)
    s.up.w += (size_t)c.intermediate * gu_row_w;
    s.up.scales += (size_t)c.intermediate * gu_row_s;
    if (s.up.biases) s.up.biases += (size_t)c.intermediate * gu_row_s;
    s.gu_stride_w = 2 * (size_t)c.intermediate * gu_row_w;
    s.gu_stride_s = 2 * (size_t)c.intermediate * gu_row_s;
    s.down = to_qmat(down);
    s.dn_stride_w = (size_t)c.hidden * dn_row_w;
    s.dn_stride_s = (size_t)c.hidden * dn_row_s;
    s.has_extra = 0;
    s.x_mid = 0;
    if (shared != nullptr && c.shared_intermediate > 0) {
        IMX_TRY(check_qtensor(shared->shared_gate_proj, f, "shared_expert.gate_proj"));
        IMX_TRY(check_qtensor(shared->shared_up_proj, f, "shared_expert.up_proj"));
        IMX_TRY(check_qtensor(shared->shared_down_proj, f, "shared_expert.down_proj"));
        s.has_extra = 1;
        s.x_mid = c.shared_intermediate;
        s.x_gate = to_qmat(shared->shared_gate_proj);
        s.x_up = to_qmat(shared->shared_up_proj);
        s.x_down = to_qmat(shared->shared_down_proj);
    }
    *out = s;
    return IMX_OK;
}

bool is_prefill(int path) {
    return path == IMX_PATH_PREFILL || path == IMX_PATH_PREFILL_SMEM || path == IMX_PATH_PREFILL_PLAIN;
}
int unit_rows_for(int path) { return is_prefill(path) ? kPrefillUnitRows : kUnitRows; }
bool is_decode(int path) { return path == IMX_PATH_DECODE || path == IMX_PATH_DECODE_REGS; }
bool decode_supported(const ExpertSet& s) { return decode_mma_supported(s) || decode_fp_supported(s); }

// Which expert kernels run for this call.  AUTO: tensor-memory GEMM tiles once
// experts see enough rows to fill them, the decode kernels below that.
int pick_path(const imx_moe_config& c, const ExpertSet& s, long n_rows, int* path) {
    int p = c.path;
    const bool many = n_rows >= 32L * s.num_experts;
    if (p == IMX_PATH_AUTO) {
        if (many && prefill_tc_supported(s)) p = IMX_PATH_PREFILL;
        else p = decode_supported(s) ? IMX_PATH_DECODE : IMX_PATH_GENERIC;
    }
    IMX_REQUIRE(!(p == IMX_PATH_PREFILL || p == IMX_PATH_PREFILL_SMEM || p == IMX_PATH_PREFILL_PLAIN) || prefill_tc_supported(s),
                "the prefill path supports affine 2/4/8-bit, mxfp8 and nvfp4 with hidden %% 128 == 0, intermediate %% 64 == 0 "
                "and whole 16-byte rows of scales");
    IMX_REQUIRE(!is_decode(p) || decode_supported(s),
                "the decode path supports affine 2/4/8-bit (group 64/128), mxfp8 and nvfp4, sizes that are multiples of 128");
    IMX_REQUIRE(p != IMX_PATH_DECODE_REGS || decode_mma_supported(s), "the register-pipelined decode kernel is affine only");
    *path = p;
    return IMX_OK;
}

// Order of the 16 values inside each block of the fp16 activation rows the chosen kernels read.
void path_block_order(int path, const QFormat& f, int order[16]) {
    if (path == IMX_PATH_GENERIC) decode_block_order(0, order);
    else expert_block_order(f, order);
}

int run_experts(int path, const GroupedArgs& ga, cudaStream_t stream, cudaEvent_t mid) {
    if (path == IMX_PATH_PREFILL) return launch_prefill_tc(ga, stream, mid, 0);
    if (path == IMX_PATH_PREFILL_PLAIN) return launch_prefill_tc(ga, stream, mid, 1);
    if (path == IMX_PATH_PREFILL_SMEM) return launch_prefill_tc(ga, stream, mid, 2);
    if (is_decode(path) && decode_fp_supported(ga.set)) return launch_decode_fp(ga, stream, mid);
    if (path == IMX_PATH_DECODE && decode_tmap_supported(ga.set)) return launch_decode_tmap(ga, stream, mid);
    if (is_decode(path)) return launch_decode_mma(ga, stream, mid);
    return launch_generic_grouped(ga, stream, mid);
}



namespace {
struct ExpertsWs {
    int32_t* status;     // [16]: [0] device status word (first in the scratch: imx_moe_status reads it there)
    SchedWs sw;
    int32_t* n_units;
    float* partials;
    WorkUnit* units;
    __half* act;
    __half* xperm;       // activations re-ordered for the decode kernels
    __half* xs;          // activations gathered into slot order (prefill path)
    float* psum;
    float* gsum_x;
    int max_units;
    size_t bytes;
};
ExpertsWs carve_experts(const imx_moe_config& c, int n_rows, int n_src_rows, void* base) {
    ExpertsWs w = {};
    Carver cv(base);
    w.status = cv.take<int32_t>(16);
    w.max_units = max_units_for(n_rows, c.num_experts, 0);
    w.sw = carve_sched(cv, c.hidden, c.intermediate, 0);
    w.n_units = cv.take<int32_t>(4);
    w.partials = cv.take<float>((size_t)kFlagWarps * 256);
    w.units = cv.take<WorkUnit>(w.max_units);
    w.act = cv.take<__half>((size_t)n_rows * c.intermediate);
    w.xperm = cv.take<__half>((size_t)n_src_rows * c.hidden);
    w.xs = w.xperm;      // the prefill path uses one or the other
    w.psum = cv.take<float>((size_t)n_rows * (c.intermediate / 16 + 1));
    w.gsum_x = cv.take<float>((size_t)n_src_rows * (c.hidden / 64 + 1));
    w.bytes = align_up(cv.off, 256);
    return w;
}

__global__ void permute_rows_kernel(const __half* __restrict__ src, const int32_t* __restrict__ row_index,
                                    int H, __half* __restrict__ dst, const Order16 order,
                                    const int32_t* __restrict__ n_rows_dev) {
    const int r = blockIdx.x;
    if (n_rows_dev != nullptr && r >= *n_rows_dev) return;      // rows past the last sorted slot are nobody's
    const __half* s = src + (size_t)(row_index ? row_index[r] : r) * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const __half v = s[(i & ~15) + order.o[i & 15]];
        dst[(size_t)r * H + i] = (i & 2) ? __float2half_rn(__half2float(v) * order.pair_scale_odd) : v;
    }
}
}  // namespace

namespace {
struct RouteWs {
    float* partials;
    float* sg;
    size_t bytes;
};
RouteWs carve_route(int n, int hidden, int num_experts, void* base) {
    RouteWs w = {};
    Carver cv(base);
    const int slice = route_slice(hidden);
    if (n > 0 && n < kRouteSplitMaxTokens && slice > 0 && num_experts % 32 == 0) {
        const size_t splits = (size_t)hidden / slice, n_pad = (size_t)(n + 31) / 32 * 32;
        w.partials = cv.take<float>(splits * n_pad * num_experts);
        w.sg = cv.take<float>(splits * n_pad);
    }
    w.bytes = align_up(cv.off, 256);
    return w;
}
}  // namespace

}  // namespace imx

using namespace imx;

extern "C" {

const char* imx_last_error(void) { return last_error(); }
const char* imx_version(void) { return "ironmlx_b200 0.2 (sm_100a)"; }
unsigned long long imx_launch_count(void) { return launch_count(); }

int imx_moe_workspace_bytes(const imx_moe_config* cfg, int n_tokens, size_t* bytes) {
    QFormat f;
    IMX_TRY(check_config(cfg, &f));
    IMX_REQUIRE(n_tokens >= 0 && bytes != nullptr, "workspace_bytes: bad arguments");
    *bytes = carve_forward(*cfg, n_tokens, nullptr).bytes;
    return IMX_OK;
}

// The glue of the decoder layer around the block (qwen35.rs:271-276), when asked for.
struct LayerTail {
    const void* ln_weight;   // RMSNorm weight (bf16 [H]) or nullptr
    float eps;
};

static int forward_impl(const imx_moe_config* cfg, const imx_moe_weights* w, const void* x, int n_tokens,
                        void* y, void* workspace, size_t workspace_bytes, void* stream_,
                        const imx_moe_trace* trace, cudaEvent_t* ev, const LayerTail* tail = nullptr) {
    QFormat f;
    IMX_TRY(check_config(cfg, &f));
    IMX_REQUIRE(w != nullptr && w->router_w != nullptr, "forward: router weight is required");
    IMX_REQUIRE(n_tokens >= 0, "forward: negative token count");
    if (n_tokens == 0) return IMX_OK;
    IMX_REQUIRE(x != nullptr && y != nullptr, "forward: x and y are required");
    IMX_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)y % 16) == 0, "forward: x and y must be 16-byte aligned");
    const imx_moe_config& c = *cfg;
    const bool has_shared = c.shared_intermediate > 0;
    IMX_REQUIRE(!has_shared || w->shared_expert_gate_w != nullptr, "forward: shared_expert_gate weight is required");
    if (workspace == nullptr || ((uintptr_t)workspace % 256) != 0) {
        set_error("forward: workspace must be a 256-byte aligned device pointer");
        return IMX_ERR_WORKSPACE;
    }
    ForwardWs ws = carve_forward(c, n_tokens, workspace);
    if (workspace_bytes < ws.bytes) {
        set_error("forward: workspace of %zu bytes needed for %d tokens, %zu given", ws.bytes, n_tokens, workspace_bytes);
        return IMX_ERR_WORKSPACE;
    }
    cudaStream_t stream = (cudaStream_t)stream_;
    ExpertSet set;
    IMX_TRY(make_expert_set(c, f, w->gate_up, w->down, c.num_experts, has_shared ? w : nullptr, &set));
    int path;
    IMX_TRY(pick_path(c, set, (long)n_tokens * c.top_k, &path));

    const int A = n_tokens * c.top_k;
    int order[16];
    path_block_order(path, f, order);
    auto mark = [&](int i) -> cudaError_t { return ev ? cudaEventRecord(ev[i], stream) : cudaSuccess; };
    const bool tmap_decode = path == IMX_PATH_DECODE && decode_tmap_supported(set);
    RouteScratch rscratch = {ws.route_partials, ws.route_sg, tmap_decode ? ws.gsum_x : nullptr, nullptr, nullptr};
    bool sums_done = false;
    IMX_CHECK_CUDA(mark(0));
    const void* router_in = x;
    if (tail != nullptr) {
        // y = x + MoE(rms_norm(x)): the split-K router normalises its tiles itself from the per-token factor;
        // the other routers read a normalised copy
        IMX_REQUIRE(tail->ln_weight == nullptr || ((uintptr_t)tail->ln_weight % 16) == 0, "forward: ln_weight must be 16-byte aligned");
        const bool in_router = ws.route_partials != nullptr && c.num_experts % 32 == 0;
        IMX_TRY(launch_rms_norm(x, n_tokens, c.hidden, tail->ln_weight, tail->eps, in_router ? nullptr : ws.xn, ws.inv_rms, stream));
        if (in_router) {
            rscratch.inv_rms = ws.inv_rms;
            rscratch.ln_weight = tail->ln_weight;
        } else {
            router_in = ws.xn;
        }
    }
    IMX_TRY(launch_route(router_in, n_tokens, c.hidden, w->router_w, w->router_logit_bias, c.num_experts, c.top_k,
                         c.norm_topk_prob, has_shared ? w->shared_expert_gate_w : nullptr, ws.topk_idx,
                         ws.topk_w, ws.shared_gate, ws.x16, order, stream,
                         tmap_decode ? 0.0625f : 1.f, ws.route_partials ? &rscratch : nullptr, &sums_done));
    IMX_CHECK_CUDA(mark(1));
    SortExtras ex;
    ex.topk_w = ws.topk_w;
    ex.top_k = c.top_k;
    ex.tok_of_slot = ws.tok_of_slot;
    ex.w_of_slot = ws.w_of_slot;
    ex.shared_gate = has_shared ? ws.shared_gate : nullptr;
    ex.n_tokens = n_tokens;
    ex.units = ws.units;
    ex.n_units = ws.n_units;
    ex.unit_rows = unit_rows_for(path);
    ex.sched = ws.sw.sched;
    ex.sched_ints = ws.sw.n_ints;
    IMX_TRY(launch_sort(ws.topk_idx, A, c.num_experts, ws.counts, ws.offsets, ws.perm, ws.inv_perm,
                        ws.sort_scratch, ws.sort_scratch_bytes, &ex, stream));
    IMX_CHECK_CUDA(mark(2));
    GroupedArgs ga = {};
    ga.set = set;
    ga.in = ws.x16;
    ga.row_index = ws.tok_of_slot;
    ga.xs = ws.xs;
    ga.n_slots = A + (has_shared ? n_tokens : 0);
    ga.units = ws.units;
    ga.n_units = ws.n_units;
    ga.max_units = ws.max_units;
    use_sched(ga, ws.sw);
    ga.partials = ws.partials;
    ga.psum = ws.psum;
    ga.gsum_x = ws.gsum_x;
    ga.n_in_rows = n_tokens;
    ga.gsum_x_ready = sums_done ? 1 : 0;
    ga.act = ws.act;
    ga.act_stride = ws.act_stride;
    // the tensor-core path leaves the rows unweighted: routing weight and shared-expert gate are applied by the
    // combine stage (one multiply per row it reads anyway) instead of per element in the GEMM epilogue
    const bool scale_in_combine = is_prefill(path);
    ga.row_scale = scale_in_combine ? nullptr : ws.w_of_slot;
    ga.out = ws.rows;
    // the tensor-memory path keeps the expert rows in fp16 (in the same buffer): at its sizes the rows are the
    // largest tensor of the step, and one extra 2^-12 rounding per row is far inside the tolerance
    const bool rows_f16 = is_prefill(path);
    ga.out16 = rows_f16 ? reinterpret_cast<__half*>(ws.rows) : nullptr;
    ga.status = ws.status;
    IMX_TRY(run_experts(path, ga, stream, ev ? ev[3] : nullptr));
    IMX_CHECK_CUDA(mark(4));
    const void* shared_rows = nullptr;
    if (has_shared)
        shared_rows = rows_f16 ? (const void*)(reinterpret_cast<const __half*>(ws.rows) + (size_t)A * c.hidden)
                               : (const void*)(ws.rows + (size_t)A * c.hidden);
    IMX_TRY(launch_combine(ws.rows, scale_in_combine ? ws.w_of_slot : nullptr, ws.inv_perm, n_tokens, c.top_k, c.hidden, shared_rows,
                           y, stream, false, tail != nullptr ? x : nullptr, rows_f16,
                           scale_in_combine && has_shared ? ws.w_of_slot + A : nullptr));
    IMX_CHECK_CUDA(mark(5));
    if (trace != nullptr) {
        auto cp = [&](void* dst, const void* src, size_t bytes) -> cudaError_t {
            return dst ? cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, stream) : cudaSuccess;
        };
        IMX_CHECK_CUDA(cp(trace->topk_idx, ws.topk_idx, (size_t)A * 4));
        IMX_CHECK_CUDA(cp(trace->topk_w, ws.topk_w, (size_t)A * 4));
        IMX_CHECK_CUDA(cp(trace->counts, ws.counts, (size_t)c.num_experts * 4));
        IMX_CHECK_CUDA(cp(trace->offsets, ws.offsets, (size_t)(c.num_experts + 1) * 4));
        IMX_CHECK_CUDA(cp(trace->perm, ws.perm, (size_t)A * 4));
        IMX_CHECK_CUDA(cp(trace->inv_perm, ws.inv_perm, (size_t)A * 4));
        if (has_shared) IMX_CHECK_CUDA(cp(trace->shared_gate, ws.shared_gate, (size_t)n_tokens * 4));
    }
    return IMX_OK;
}

int imx_moe_forward(const imx_moe_config* cfg, const imx_moe_weights* w, const void* x, int n_tokens,
                    void* y, void* workspace, size_t workspace_bytes, void* stream_,
                    const imx_moe_trace* trace) {
    return forward_impl(cfg, w, x, n_tokens, y, workspace, workspace_bytes, stream_, trace, nullptr);
}

int imx_moe_forward_residual(const imx_moe_config* cfg, const imx_moe_weights* w, const void* h, const void* ln_weight,
                             float eps, int n_tokens, void* y, void* workspace, size_t workspace_bytes, void* stream_,
                             const imx_moe_trace* trace) {
    const LayerTail tail = {ln_weight, eps};
    return forward_impl(cfg, w, h, n_tokens, y, workspace, workspace_bytes, stream_, trace, nullptr, &tail);
}

int imx_rms_norm(const void* x, int n_rows, int hidden, const void* weight, float eps, void* y, void* stream) {
    IMX_REQUIRE(y != nullptr, "rms_norm: y is required");
    return launch_rms_norm(x, n_rows, hidden, weight, eps, y, nullptr, (cudaStream_t)stream);
}

int imx_moe_forward_timed(const imx_moe_config* cfg, const imx_moe_weights* w, const void* x, int n_tokens,
                          void* y, void* workspace, size_t workspace_bytes, void* stream_, float* stage_ms) {
    IMX_REQUIRE(stage_ms != nullptr, "forward_timed: stage_ms is required");
    cudaEvent_t ev[6] = {};
    for (int i = 0; i < 6; ++i) IMX_CHECK_CUDA(cudaEventCreate(&ev[i]));
    int st = forward_impl(cfg, w, x, n_tokens, y, workspace, workspace_bytes, stream_, nullptr, ev);
    if (st == IMX_OK && n_tokens > 0) {
        cudaError_t e = cudaEventSynchronize(ev[5]);
        for (int i = 0; i < 5 && e == cudaSuccess; ++i) e = cudaEventElapsedTime(&stage_ms[i], ev[i], ev[i + 1]);
        if (e != cudaSuccess) {
            set_error("forward_timed: %s", cudaGetErrorString(e));
            st = IMX_ERR_CUDA;
        }
    }
    for (int i = 0; i < 6; ++i) cudaEventDestroy(ev[i]);
    return st;
}

int imx_moe_forward_host(const imx_moe_config* cfg, const imx_moe_weights* w, const void* x_host,
                         int n_tokens, void* y_host, void* workspace, size_t workspace_bytes,
                         void* stream_) {
    size_t need = 0;
    IMX_TRY(imx_moe_workspace_bytes(cfg, n_tokens, &need));
    IMX_REQUIRE(n_tokens >= 0 && (n_tokens == 0 || (x_host != nullptr && y_host != nullptr)),
                "forward_host: x_host and y_host are required");
    if (n_tokens == 0) return IMX_OK;
    const size_t xy = align_up((size_t)n_tokens * cfg->hidden * 2, 256);
    if (workspace == nullptr || ((uintptr_t)workspace % 256) != 0 || workspace_bytes < need + 2 * xy) {
        set_error("forward_host: 256-byte aligned workspace of %zu bytes needed, %zu given", need + 2 * xy,
                  workspace_bytes);
        return IMX_ERR_WORKSPACE;
    }
    cudaStream_t stream = (cudaStream_t)stream_;
    uint8_t* xd = (uint8_t*)workspace + need;
    uint8_t* yd = xd + xy;
    IMX_CHECK_CUDA(cudaMemcpyAsync(xd, x_host, (size_t)n_tokens * cfg->hidden * 2, cudaMemcpyHostToDevice, stream));
    IMX_TRY(imx_moe_forward(cfg, w, xd, n_tokens, yd, workspace, need, stream_, nullptr));
    IMX_CHECK_CUDA(cudaMemcpyAsync(y_host, yd, (size_t)n_tokens * cfg->hidden * 2, cudaMemcpyDeviceToHost, stream));
    IMX_CHECK_CUDA(cudaStreamSynchronize(stream));
    return IMX_OK;
}

int imx_moe_status(void* workspace, void* stream_) {
    IMX_REQUIRE(workspace != nullptr, "status: workspace is NULL");
    cudaStream_t stream = (cudaStream_t)stream_;
    int32_t host[8] = {0};
    IMX_CHECK_CUDA(cudaMemcpyAsync(host, workspace, sizeof(host), cudaMemcpyDeviceToHost, stream));
    IMX_CHECK_CUDA(cudaStreamSynchronize(stream));
    if (host[0] != 0) {
        set_error("a kernel recorded device status %d (detail %d, %d)", host[0], host[1], host[2]);
        IMX_CHECK_CUDA(cudaMemsetAsync(workspace, 0, sizeof(host), stream));
        return IMX_ERR_DEVICE;
    }
    return IMX_OK;
}

void imx_testing_decode_handoff(int spin_limit, int withhold) { testing_decode_handoff(spin_limit, withhold); }

int imx_moe_saturations(void* workspace, void* stream_, long long* count) {
    IMX_REQUIRE(workspace != nullptr && count != nullptr, "saturations: workspace and count are required");
    cudaStream_t stream = (cudaStream_t)stream_;
    int32_t v = 0;
    int32_t* word = reinterpret_cast<int32_t*>(workspace) + kStatusSaturations;
    IMX_CHECK_CUDA(cudaMemcpyAsync(&v, word, sizeof(v), cudaMemcpyDeviceToHost, stream));
    IMX_CHECK_CUDA(cudaStreamSynchronize(stream));
    if (v != 0) IMX_CHECK_CUDA(cudaMemsetAsync(word, 0, sizeof(v), stream));
    *count = v;
    return IMX_OK;
}

int imx_moe_route(const void* x, int n_tokens, int hidden, const void* router_w, const float* logit_bias,
                  int num_experts, int top_k, int norm_topk_prob, const void* shared_gate_w,
                  int32_t* topk_idx, float* topk_w, float* shared_gate, void* x_f16, void* stream) {
    IMX_REQUIRE(n_tokens >= 0, "route: negative token count");
    if (n_tokens == 0) return IMX_OK;
    IMX_REQUIRE(x && router_w && topk_idx && topk_w, "route: x, router_w, topk_idx and topk_w are required");
    return launch_route(x, n_tokens, hidden, router_w, logit_bias, num_experts, top_k, norm_topk_prob,
                        shared_gate_w, topk_idx, topk_w, shared_gate, x_f16, nullptr, (cudaStream_t)stream);
}

int imx_moe_route_scratch_bytes(int n_tokens, int hidden, int num_experts, size_t* bytes) {
    using namespace imx;
    IMX_REQUIRE(bytes != nullptr && n_tokens >= 0 && hidden > 0 && num_experts >= 1, "route_scratch_bytes: bad arguments");
    *bytes = carve_route(n_tokens, hidden, num_experts, nullptr).bytes;
    return IMX_OK;
}

int imx_moe_route_ws(const void* x, int n_tokens, int hidden, const void* router_w, const float* logit_bias,
                     int num_experts, int top_k, int norm_topk_prob, const void* shared_gate_w,
                     int32_t* topk_idx, float* topk_w, float* shared_gate, void* x_f16, void* scratch,
                     size_t scratch_bytes, void* stream) {
    using namespace imx;
    IMX_REQUIRE(n_tokens >= 0, "route: negative token count");
    if (n_tokens == 0) return IMX_OK;
    IMX_REQUIRE(x && router_w && topk_idx && topk_w, "route: x, router_w, topk_idx and topk_w are required");
    RouteWs ws = carve_route(n_tokens, hidden, num_experts, scratch);
    IMX_REQUIRE(ws.bytes == 0 || (scratch != nullptr && ((uintptr_t)scratch % 256) == 0 && scratch_bytes >= ws.bytes),
                "route: scratch of %zu bytes (256-byte aligned) needed, %zu given", ws.bytes, scratch_bytes);
    RouteScratch rs = {ws.partials, ws.sg, nullptr, nullptr, nullptr};
    return launch_route(x, n_tokens, hidden, router_w, logit_bias, num_experts, top_k, norm_topk_prob,
                        shared_gate_w, topk_idx, topk_w, shared_gate, x_f16, nullptr, (cudaStream_t)stream, 1.f,
                        ws.partials ? &rs : nullptr, nullptr);
}

int imx_moe_sort_scratch_bytes(int n_assign, int num_experts, size_t* bytes) {
    IMX_REQUIRE(n_assign >= 0 && num_experts >= 1 && bytes != nullptr, "sort_scratch_bytes: bad arguments");
    *bytes = sort_scratch_bytes(n_assign, num_experts);
    return IMX_OK;
}

int imx_moe_sort(const int32_t* expert_ids, int n_assign, int num_experts, int32_t* counts, int32_t* offsets,
                 int32_t* perm, int32_t* inv_perm, void* scratch, size_t scratch_bytes, void* stream) {
    IMX_REQUIRE(n_assign >= 0 && (n_assign == 0 || expert_ids != nullptr), "sort: expert_ids is required");
    return launch_sort(expert_ids, n_assign, num_experts, counts, offsets, perm, inv_perm, scratch,
                       scratch_bytes, nullptr, (cudaStream_t)stream);
}

int imx_moe_sort_static(const int32_t* expert_ids, int n_assign, int num_experts, int32_t* counts,
                        int32_t* offsets, int32_t* perm, int32_t* inv_perm, void* stream) {
    IMX_REQUIRE(n_assign >= 0 && (n_assign == 0 || expert_ids != nullptr), "sort_static: expert_ids is required");
    IMX_REQUIRE(offsets && perm && inv_perm, "sort_static: offsets, perm and inv_perm are required");
    return launch_sort_static(expert_ids, n_assign, num_experts, counts, offsets, perm, inv_perm,
                              (cudaStream_t)stream);
}

int imx_moe_experts_scratch_bytes(const imx_moe_config* cfg, int n_rows, size_t* bytes) {
    QFormat f;
    IMX_TRY(check_config(cfg, &f));
    IMX_REQUIRE(n_rows >= 0 && bytes != nullptr, "experts_scratch_bytes: bad arguments");
    *bytes = carve_experts(*cfg, n_rows, n_rows, nullptr).bytes;
    return IMX_OK;
}

int imx_moe_experts(const imx_moe_config* cfg, const imx_qtensor* gate_up, const imx_qtensor* down,
                    int num_experts, const void* x_f16, const int32_t* row_index, const int32_t* offsets,
                    int n_rows, int max_rows_per_expert, const float* row_scale, float* out, void* scratch,
                    size_t scratch_bytes, void* stream_) {
    (void)max_rows_per_expert;
    QFormat f;
    IMX_TRY(check_config(cfg, &f));
    IMX_REQUIRE(gate_up && down && offsets, "experts: gate_up, down and offsets are required");
    IMX_REQUIRE(num_experts >= 1 && num_experts <= 1023 && n_rows >= 0, "experts: bad sizes");
    if (n_rows == 0) return IMX_OK;
    IMX_REQUIRE(x_f16 && out, "experts: x_f16 and out are required");
    imx_moe_config c = *cfg;
    c.num_experts = num_experts;
    ExpertsWs ws = carve_experts(c, n_rows, n_rows, scratch);
    if (scratch == nullptr || ((uintptr_t)scratch % 256) != 0 || scratch_bytes < ws.bytes) {
        set_error("experts: 256-byte aligned scratch of %zu bytes needed, %zu given", ws.bytes, scratch_bytes);
        return IMX_ERR_WORKSPACE;
    }
    cudaStream_t stream = (cudaStream_t)stream_;
    ExpertSet set;
    IMX_TRY(make_expert_set(c, f, *gate_up, *down, num_experts, nullptr, &set));
    int path;
    IMX_TRY(pick_path(c, set, (long)n_rows, &path));
    IMX_TRY(launch_build_units(offsets, num_experts, unit_rows_for(path), ws.units,
                               ws.n_units, ws.sw.sched, ws.sw.n_ints, stream));
    GroupedArgs ga = {};
    ga.set = set;
    ga.in = (const __half*)x_f16;
    ga.row_index = row_index;
    if (path != IMX_PATH_GENERIC) {
        // gather the rows once, in the block order the decode kernels read
        int o[16];
        path_block_order(path, f, o);
        Order16 order;
        for (int i = 0; i < 16; ++i) order.o[i] = (int8_t)o[i];
        order.pair_scale_odd = path == IMX_PATH_DECODE && decode_tmap_supported(set) ? 0.0625f : 1.f;
        permute_rows_kernel<<<n_rows, 256, 0, stream>>>((const __half*)x_f16, row_index, c.hidden, ws.xperm, order,
                                                        offsets + num_experts); IMX_LAUNCHED();
        IMX_CHECK_CUDA(cudaGetLastError());
        ga.in = ws.xperm;
        ga.row_index = nullptr;
    }
    ga.units = ws.units;
    ga.n_units = ws.n_units;
    ga.max_units = ws.max_units;
    use_sched(ga, ws.sw);
    ga.partials = ws.partials;
    ga.psum = ws.psum;
    ga.gsum_x = ws.gsum_x;
    ga.n_in_rows = n_rows;
    ga.n_rows_dev = offsets + num_experts;
    ga.gsum_x_ready = 0;
    ga.act = ws.act;
    ga.act_stride = c.intermediate;
    ga.row_scale = row_scale;
    ga.out = out;
    ga.status = ws.status;
    ga.xs = ws.xs;
    ga.n_slots = n_rows;
    return run_experts(path, ga, stream);
}

int imx_moe_combine(const float* rows, const int32_t* inv_perm, int n_tokens, int top_k, int hidden,
                    const float* shared_rows, void* y, void* stream) {
    IMX_REQUIRE(n_tokens >= 0, "combine: negative token count");
    if (n_tokens == 0) return IMX_OK;
    IMX_REQUIRE(rows && inv_perm && y, "combine: rows, inv_perm and y are required");
    return launch_combine(rows, nullptr, inv_perm, n_tokens, top_k, hidden, shared_rows, y, (cudaStream_t)stream);
}

int imx_moe_combine_scaled(const float* rows, const float* row_scale, const int32_t* inv_perm, int n_tokens,
                           int top_k, int hidden, const float* shared_rows, void* y, void* stream) {
    IMX_REQUIRE(n_tokens >= 0, "combine: negative token count");
    if (n_tokens == 0) return IMX_OK;
    IMX_REQUIRE(rows && row_scale && inv_perm && y, "combine_scaled: rows, row_scale, inv_perm and y are required");
    return launch_combine(rows, row_scale, inv_perm, n_tokens, top_k, hidden, shared_rows, y, (cudaStream_t)stream);
}

int imx_moe_combine_partial(const float* rows, const float* row_scale, const int32_t* inv_perm, int n_tokens,
                            int top_k, int hidden, float* y_f32, void* stream) {
    IMX_REQUIRE(n_tokens >= 0, "combine: negative token count");
    if (n_tokens == 0) return IMX_OK;
    IMX_REQUIRE(rows && inv_perm && y_f32, "combine_partial: rows, inv_perm and y_f32 are required");
    return launch_combine(rows, row_scale, inv_perm, n_tokens, top_k, hidden, nullptr, y_f32, (cudaStream_t)stream, true);
}

int imx_gather_rows(const void* src, const int32_t* index, int n_rows, size_t row_bytes, void* dst, void* stream) {
    IMX_REQUIRE(n_rows >= 0, "gather_rows: negative row count");
    if (n_rows == 0) return IMX_OK;
    IMX_REQUIRE(src && index && dst, "gather_rows: src, index and dst are required");
    return launch_gather_rows(src, index, n_rows, row_bytes, dst, (cudaStream_t)stream);
}

int imx_dequantize(const imx_qtensor* w, int rows, int in, int group_size, int bits, int mode, int out_dtype,
                   void* out, void* stream) {
    QFormat f;
    IMX_TRY(validate_format(mode, bits, group_size, &f));
    IMX_REQUIRE(w != nullptr && out != nullptr && rows >= 0 && in > 0, "dequantize: bad arguments");
    IMX_TRY(check_qtensor(*w, f, "dequantize"));
    return launch_dequantize(to_qmat(*w), rows, in, f, out_dtype, out, (cudaStream_t)stream);
}

int imx_quantized_matmul(const void* x, int m, const imx_qtensor* w, int n_out, int in, int transpose,
                         int group_size, int bits, int mode, void* y, void* stream) {
    QFormat f;
    IMX_TRY(validate_format(mode, bits, group_size, &f));
    IMX_REQUIRE(x && w && y && m >= 0 && n_out > 0 && in > 0, "quantized_matmul: bad arguments");
    IMX_TRY(check_qtensor(*w, f, "quantized_matmul"));
    return launch_qmm(x, m, to_qmat(*w), n_out, in, transpose, f, y, nullptr, nullptr, 0, 0, (cudaStream_t)stream);
}

int imx_quantize(const float* w, int rows, int in, int group_size, int bits, int mode, float global_scale,
                 void* w_packed, void* scales, void* biases, void* stream) {
    QFormat f;
    IMX_TRY(validate_format(mode, bits, group_size, &f));
    IMX_REQUIRE(w && w_packed && scales && rows >= 0 && in > 0, "quantize: bad arguments");
    return launch_quantize(w, rows, in, f, global_scale, w_packed, scales, biases, (cudaStream_t)stream);
}

int imx_gather_qmm(const void* x, const int32_t* lhs_index, const imx_qtensor* w, const int32_t* rhs_index,
                   int n_rows, int n_out, int in, int group_size, int bits, int mode, void* y, void* stream) {
    QFormat f;
    IMX_TRY(validate_format(mode, bits, group_size, &f));
    IMX_REQUIRE(x && w && y && rhs_index && n_rows >= 0 && n_out > 0 && in > 0, "gather_qmm: bad arguments");
    IMX_TRY(check_qtensor(*w, f, "gather_qmm"));
    const size_t w_stride = (size_t)n_out * packed_row_bytes(in, f.bits);
    const size_t s_stride = (size_t)n_out * scale_row_bytes(in, f);
    return launch_qmm(x, n_rows, to_qmat(*w), n_out, in, 1, f, y, lhs_index, rhs_index, w_stride, s_stride,
                      (cudaStream_t)stream);
}

}  // extern "C"
