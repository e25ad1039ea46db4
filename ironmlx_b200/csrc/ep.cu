// Expert parallelism of the MoE block behind the C ABI: one process per GPU,
// the E experts in contiguous blocks of E / R per rank, tokens sharded evenly,
// the router, the shared expert and its gate replicated.  The reference has no
// distributed code (no collective and no communicator anywhere in its tree);
// what this has to reproduce is the single-device result of
// mlx/src/nn/moe.rs:55-183, whose expert loop (moe.rs:117-144) is what gets
// sharded.
//
// Two schedules, NCCL for every byte that crosses NVLink:
//
//   gathered (decode-size batches, fixed shapes, no host synchronisation, so a
//   step can be captured in a CUDA graph):
//     all-gather the tokens -> route all of them (the router is replicated) ->
//     sort the assignments that fall into the local block of experts (the others
//     drop out of the sort, moe.rs:100) -> the local experts and, for the local
//     tokens, the shared expert in ONE pair of grouped launches -> fp32 partial
//     sums per token -> reduce-scatter to the token owners -> add the shared
//     rows, round once.
//
//   all-to-all (prefill-size batches):
//     route and sort the local tokens by global expert id (a contiguous block of
//     experts per rank: the stable sort is already grouped by destination rank,
//     then expert, then flat index) -> all-gather the [E] count vectors (the one
//     host synchronisation: the split sizes of the exchange are host values, and
//     they are checked before any row moves) -> dispatch fp16 rows with grouped
//     ncclSend/ncclRecv into local memory -> the tensor-core expert kernels read
//     the received rows through a row index (expert-major order, no second sort)
//     and their second product's epilogue writes every result row straight into
//     the buffer that travels back -> return exchange -> weighted combine on the
//     source rank in ascending slot order: the same order and the same fp16 rows
//     as on one GPU, so the result is bit-identical to the single-GPU block.
//
// NCCL is resolved at run time (dlopen of the library the process already has,
// else libnccl.so.2): the C ABI library carries no link-time dependency on it.
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <mutex>
#include <vector>

#include "internal.h"

struct imx_ep_ctx {
    imx_moe_config cfg;        // the whole block (num_experts = E over all ranks)
    int rank, world, e_loc;
    int device;
    ncclComm_t comm;
    bool own_comm;
    int32_t* host_counts;      // pinned [world * E]
    std::vector<size_t> send_rows, recv_rows;
    cudaEvent_t ev[6];         // phase boundaries of a timed all-to-all call
    bool have_events;
};

namespace imx {

namespace {

struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*);
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
    ncclResult_t (*ReduceScatter)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*GroupStart)();
    ncclResult_t (*GroupEnd)();
    const char* (*GetErrorString)(ncclResult_t);
    bool ok;
};

const NcclApi* nccl_api() {
    static NcclApi api = {};
    static std::once_flag once;
    std::call_once(once, [] {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);      // the copy the process already uses, if any
        if (h == nullptr) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (h == nullptr) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (h == nullptr) return;
        bool ok = true;
        auto sym = [&](const char* name) -> void* {
            void* p = dlsym(h, name);
            if (p == nullptr) ok = false;
            return p;
        };
        api.GetUniqueId = (decltype(api.GetUniqueId))sym("ncclGetUniqueId");
        api.CommInitRank = (decltype(api.CommInitRank))sym("ncclCommInitRank");
        api.CommDestroy = (decltype(api.CommDestroy))sym("ncclCommDestroy");
        api.AllGather = (decltype(api.AllGather))sym("ncclAllGather");
        api.ReduceScatter = (decltype(api.ReduceScatter))sym("ncclReduceScatter");
        api.Send = (decltype(api.Send))sym("ncclSend");
        api.Recv = (decltype(api.Recv))sym("ncclRecv");
        api.GroupStart = (decltype(api.GroupStart))sym("ncclGroupStart");
        api.GroupEnd = (decltype(api.GroupEnd))sym("ncclGroupEnd");
        api.GetErrorString = (decltype(api.GetErrorString))sym("ncclGetErrorString");
        api.ok = ok;
    });
    return api.ok ? &api : nullptr;
}

#define IMX_CHECK_NCCL(expr)                                                                   \
    do {                                                                                       \
        ncclResult_t _r = (expr);                                                              \
        if (_r != ncclSuccess) {                                                               \
            ::imx::set_error("%s failed: %s (%s:%d)", #expr, nc->GetErrorString(_r), __FILE__, __LINE__); \
            return IMX_ERR_CUDA;                                                               \
        }                                                                                      \
    } while (0)

// ids[i] - base (ids outside the local block fall out of [0, E_loc) and are dropped by the sort); also
// ident[i] = i for the final combine of the gathered schedule.
__global__ void local_ids_kernel(const int32_t* __restrict__ ids, int n, int base, int32_t* __restrict__ out,
                                 int32_t* __restrict__ ident, int n_ident) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = ids[i] - base;
    if (i < n_ident) ident[i] = i;
}

// All-to-all schedule, after the dispatch: the received rows are ordered (source rank, local expert, flat
// index).  Block e < E_loc writes, for local expert e, the rows of its slots in expert-major order
// (row_index) and offsets2[e]; block E_loc appends the shared expert's slots (the local tokens, whose fp16
// rows sit behind the `cap` received rows) and closes offsets2.  counts: [R][E] assignments per (source, expert).
__global__ void __launch_bounds__(256)
ep_regroup_kernel(const int32_t* __restrict__ counts, int R, int E, int e_lo, int E_loc, int cap, int n_local,
                  int has_shared, int32_t* __restrict__ row_index, int32_t* __restrict__ offsets2) {
    __shared__ int s_red[256];
    __shared__ int s_src0[64], s_dst0[64];     // per source: first received row / first slot of this expert's segment
    const int e = blockIdx.x, tid = threadIdx.x;
    // rows of local experts before e (all sources), and the total
    int before = 0, total = 0;
    for (int i = tid; i < R * E_loc; i += 256) {
        const int s = i / E_loc, el = i - s * E_loc;
        const int c = counts[s * E + e_lo + el];
        total += c;
        if (el < e) before += c;
    }
    s_red[tid] = before;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (tid < o) s_red[tid] += s_red[tid + o];
        __syncthreads();
    }
    before = s_red[0];
    __syncthreads();
    s_red[tid] = total;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (tid < o) s_red[tid] += s_red[tid + o];
        __syncthreads();
    }
    total = s_red[0];
    __syncthreads();
    if (e == E_loc) {
        if (tid == 0) {
            offsets2[E_loc] = total;
            offsets2[E_loc + 1] = total + (has_shared ? n_local : 0);
        }
        if (has_shared)
            for (int t = tid; t < n_local; t += 256) row_index[total + t] = cap + t;
        return;
    }
    if (tid == 0) {
        offsets2[e] = before;
        int recv_base = 0, dst = before;
        for (int s = 0; s < R; ++s) {
            int in_src_before = 0, src_total = 0;
            for (int el = 0; el < E_loc; ++el) {
                const int c = counts[s * E + e_lo + el];
                if (el < e) in_src_before += c;
                src_total += c;
            }
            s_src0[s] = recv_base + in_src_before;
            s_dst0[s] = dst;
            dst += counts[s * E + e_lo + e];
            recv_base += src_total;
        }
    }
    __syncthreads();
    for (int s = 0; s < R; ++s) {
        const int len = counts[s * E + e_lo + e];
        for (int j = tid; j < len; j += 256) row_index[s_dst0[s] + j] = s_src0[s] + j;
    }
}

// Gathered schedule, last step: y = bf16(sum over the ranks of a token's partial row + gate * shared-expert row).
__global__ void finish_rows_kernel(const float* __restrict__ mine, const __half* __restrict__ shared, const float* __restrict__ gate,
                                   int H, __nv_bfloat16* __restrict__ y) {
    const size_t t = blockIdx.x;
    const float g = gate != nullptr ? gate[t] : 1.f;
    for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
        float4 v = *reinterpret_cast<const float4*>(mine + t * H + c);
        if (shared != nullptr) {
            const uint2 q = *reinterpret_cast<const uint2*>(shared + t * H + c);
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&q.x));
            const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&q.y));
            v.x += a.x * g; v.y += a.y * g; v.z += b.x * g; v.w += b.y * g;
        }
        __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        uint2 o;
        o.x = *reinterpret_cast<uint32_t*>(&lo);
        o.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(y + t * H + c) = o;
    }
}

struct Common {
    int32_t* status;
    SchedWs sw;
    int32_t* n_units;
    float* partials;
};

// Workspace of the gathered schedule for n local tokens.
struct GatherWs {
    Common c;
    __nv_bfloat16* xg;
    int32_t* topk_idx;
    float* topk_w;
    float* shared_gate;
    __half* x16;
    float* route_partials;
    float* route_sg;
    float* gsum_x;
    int32_t* ids_local;
    int32_t* ident;
    int32_t* counts;
    int32_t* offsets;
    int32_t* perm;
    int32_t* inv_perm;
    int32_t* tok_of_slot;
    float* w_of_slot;
    WorkUnit* units;
    void* sort_scratch;
    size_t sort_scratch_bytes;
    __half* act;
    __half* xs;           // activations in slot order (tensor-core kernels: batches with >= 32 rows per local expert)
    float* rows;
    float* psum;
    float* partial;
    float* mine;
    int max_units, act_stride;
    size_t bytes;
};

GatherWs carve_gather(const imx_ep_ctx& x, int n, void* base) {
    const imx_moe_config& c = x.cfg;
    GatherWs w = {};
    const int nA = n * x.world, A = nA * c.top_k, ns = c.shared_intermediate > 0 ? n : 0;
    Carver cv(base);
    w.c.status = cv.take<int32_t>(16);
    w.max_units = max_units_for(A, x.e_loc, ns);
    w.c.sw = carve_sched(cv, c.hidden, c.intermediate, c.shared_intermediate);
    w.c.n_units = cv.take<int32_t>(4);
    w.c.partials = cv.take<float>((size_t)kFlagWarps * 256);
    w.xg = cv.take<__nv_bfloat16>((size_t)nA * c.hidden);
    w.topk_idx = cv.take<int32_t>(A);
    w.topk_w = cv.take<float>(A);
    w.shared_gate = cv.take<float>(nA);
    w.x16 = cv.take<__half>((size_t)nA * c.hidden);
    const int slice = route_slice(c.hidden);
    if (nA < kRouteSplitMaxTokens && slice > 0 && c.num_experts % 32 == 0) {
        const size_t splits = (size_t)c.hidden / slice, n_pad = (size_t)(nA + 31) / 32 * 32;
        w.route_partials = cv.take<float>(splits * n_pad * c.num_experts);
        w.route_sg = cv.take<float>(splits * n_pad);
    }
    w.gsum_x = cv.take<float>((size_t)nA * (c.hidden / 64 + 1));
    w.ids_local = cv.take<int32_t>(A);
    w.ident = cv.take<int32_t>(n);
    w.counts = cv.take<int32_t>(x.e_loc);
    w.offsets = cv.take<int32_t>(x.e_loc + 1);
    w.perm = cv.take<int32_t>(A);
    w.inv_perm = cv.take<int32_t>(A);
    w.tok_of_slot = cv.take<int32_t>(A + ns);
    w.w_of_slot = cv.take<float>(A + ns);
    w.units = cv.take<WorkUnit>(w.max_units);
    w.sort_scratch_bytes = sort_scratch_bytes(A, x.e_loc);
    w.sort_scratch = cv.take<uint8_t>(w.sort_scratch_bytes);
    w.act_stride = c.intermediate > c.shared_intermediate ? c.intermediate : c.shared_intermediate;
    w.act = cv.take<__half>((size_t)(A + ns) * w.act_stride);
    if ((long)A / x.world >= 32L * x.e_loc) w.xs = cv.take<__half>((size_t)(A + ns) * c.hidden);
    w.rows = cv.take<float>((size_t)(A + ns) * c.hidden);
    w.psum = cv.take<float>((size_t)(A + ns) * (w.act_stride / 16 + 1));
    w.partial = cv.take<float>((size_t)nA * c.hidden);
    w.mine = cv.take<float>((size_t)n * c.hidden);
    w.bytes = align_up(cv.off, 256);
    return w;
}

// Workspace of the all-to-all schedule for n local tokens: sized for the worst case, every assignment of
// every rank landing here (cap = R * n * k rows).
struct A2aWs {
    Common c;
    int32_t* topk_idx;
    float* topk_w;
    float* shared_gate;
    float* route_partials;
    float* route_sg;
    int32_t* counts;          // [E]
    int32_t* offsets;         // [E + 1]
    int32_t* perm;
    int32_t* inv_perm;
    int32_t* tok_of_slot;
    float* w_of_slot;
    void* sort_scratch;
    size_t sort_scratch_bytes;
    __half* send_buf;         // [A, H] rows in sorted (destination, expert, flat index) order
    int32_t* all_counts;      // [R][E]
    __half* recv_buf;         // [cap + n, H]: received rows, then the local tokens' fp16 rows (written by the router)
    int32_t* row_index;       // [cap + n]: row of recv_buf behind each expert-major slot
    int32_t* offsets2;        // [E_loc + 2]
    WorkUnit* units;
    __half* act;              // [cap + n, act_stride]
    __half* xs;               // [cap + n, H]: rows gathered into slot order for the tensor-core kernels
    __half* ret_buf;          // [cap + n, H]: expert rows in received order, shared rows behind them
    __half* rows_back;        // [A, H]: this rank's rows, back in its sorted slot order
    int cap, max_units, act_stride;
    size_t bytes;
};

A2aWs carve_a2a(const imx_ep_ctx& x, int n, void* base) {
    const imx_moe_config& c = x.cfg;
    A2aWs w = {};
    const int A = n * c.top_k, ns = c.shared_intermediate > 0 ? n : 0;
    w.cap = A * x.world;
    Carver cv(base);
    w.c.status = cv.take<int32_t>(16);
    w.c.sw = carve_sched(cv, 0, 0, 0);        // this schedule runs the tensor-core kernels only: no hand-off buffers
    w.c.n_units = cv.take<int32_t>(4);
    w.c.partials = cv.take<float>((size_t)kFlagWarps * 256);
    w.topk_idx = cv.take<int32_t>(A);
    w.topk_w = cv.take<float>(A);
    w.shared_gate = cv.take<float>(n);
    const int slice = route_slice(c.hidden);
    if (n < kRouteSplitMaxTokens && slice > 0 && c.num_experts % 32 == 0) {
        const size_t splits = (size_t)c.hidden / slice, n_pad = (size_t)(n + 31) / 32 * 32;
        w.route_partials = cv.take<float>(splits * n_pad * c.num_experts);
        w.route_sg = cv.take<float>(splits * n_pad);
    }
    w.counts = cv.take<int32_t>(c.num_experts);
    w.offsets = cv.take<int32_t>(c.num_experts + 1);
    w.perm = cv.take<int32_t>(A);
    w.inv_perm = cv.take<int32_t>(A);
    w.tok_of_slot = cv.take<int32_t>(A);
    w.w_of_slot = cv.take<float>(A);
    w.sort_scratch_bytes = sort_scratch_bytes(A, c.num_experts);
    w.sort_scratch = cv.take<uint8_t>(w.sort_scratch_bytes);
    w.send_buf = cv.take<__half>((size_t)A * c.hidden);
    w.all_counts = cv.take<int32_t>((size_t)x.world * c.num_experts);
    w.recv_buf = cv.take<__half>((size_t)(w.cap + n) * c.hidden);
    w.row_index = cv.take<int32_t>(w.cap + ns);
    w.offsets2 = cv.take<int32_t>(x.e_loc + 2);
    w.max_units = max_units_for(w.cap, x.e_loc, ns);
    w.units = cv.take<WorkUnit>(w.max_units);
    w.act_stride = c.intermediate > c.shared_intermediate ? c.intermediate : c.shared_intermediate;
    w.act = cv.take<__half>((size_t)(w.cap + ns) * w.act_stride);
    w.xs = cv.take<__half>((size_t)(w.cap + ns) * c.hidden);
    w.ret_buf = cv.take<__half>((size_t)(w.cap + ns) * c.hidden);
    w.rows_back = cv.take<__half>((size_t)A * c.hidden);
    w.bytes = align_up(cv.off, 256);
    return w;
}

imx_moe_config local_config(const imx_ep_ctx& x) {
    imx_moe_config c = x.cfg;
    c.num_experts = x.e_loc;
    return c;
}

int forward_gathered(imx_ep_ctx& x, const imx_moe_weights* w, const void* xin, int n, void* y, void* workspace,
                     size_t ws_bytes, cudaStream_t stream, imx_ep_info* info) {
    const NcclApi* nc = nccl_api();
    const imx_moe_config& c = x.cfg;
    QFormat f;
    IMX_TRY(check_config(&c, &f));
    const GatherWs ws = carve_gather(x, n, workspace);
    if (ws_bytes < ws.bytes) {
        set_error("ep_forward (gathered): workspace of %zu bytes needed for %d local tokens, %zu given", ws.bytes, n, ws_bytes);
        return IMX_ERR_WORKSPACE;
    }
    const int R = x.world, nA = n * R, A = nA * c.top_k;
    const bool has_shared = c.shared_intermediate > 0;
    const imx_moe_config cl = local_config(x);
    ExpertSet set;
    IMX_TRY(make_expert_set(cl, f, w->gate_up, w->down, x.e_loc, has_shared ? w : nullptr, &set));
    int path;
    IMX_TRY(pick_path(cl, set, (long)A / R, &path));
    if (is_prefill(path) && ws.xs == nullptr) {      // (cannot happen: the workspace has the buffer at these sizes)
        imx_moe_config cd = cl;
        cd.path = IMX_PATH_DECODE;
        if (pick_path(cd, set, (long)A / R, &path) != IMX_OK) path = IMX_PATH_GENERIC;
    }
    const bool tc = is_prefill(path);                // tensor-core kernels: fp16 rows, routing weight applied in the combine
    const bool tmap_decode = path == IMX_PATH_DECODE && decode_tmap_supported(set);

    IMX_CHECK_NCCL(nc->AllGather(xin, ws.xg, (size_t)n * c.hidden, ncclBfloat16, x.comm, stream));
    int order[16];
    path_block_order(path, f, order);
    RouteScratch rs = {ws.route_partials, ws.route_sg, tmap_decode ? ws.gsum_x : nullptr, nullptr, nullptr};
    bool sums_done = false;
    IMX_TRY(launch_route(ws.xg, nA, c.hidden, w->router_w, w->router_logit_bias, c.num_experts, c.top_k, c.norm_topk_prob,
                         has_shared ? w->shared_expert_gate_w : nullptr, ws.topk_idx, ws.topk_w, ws.shared_gate, ws.x16, order,
                         stream, tmap_decode ? 0.0625f : 1.f, ws.route_partials ? &rs : nullptr, &sums_done));
    const int nmax = A > n ? A : n;
    local_ids_kernel<<<(nmax + 255) / 256, 256, 0, stream>>>(ws.topk_idx, A, x.rank * x.e_loc, ws.ids_local, ws.ident, n); IMX_LAUNCHED();
    IMX_CHECK_CUDA(cudaGetLastError());
    SortExtras ex;
    ex.topk_w = ws.topk_w;
    ex.top_k = c.top_k;
    ex.tok_of_slot = ws.tok_of_slot;
    ex.w_of_slot = ws.w_of_slot;
    ex.shared_gate = has_shared ? ws.shared_gate : nullptr;
    ex.n_tokens = n;
    ex.shared_token0 = x.rank * n;
    ex.units = ws.units;
    ex.n_units = ws.c.n_units;
    ex.unit_rows = unit_rows_for(path);
    ex.sched = ws.c.sw.sched;
    ex.sched_ints = ws.c.sw.n_ints;
    IMX_TRY(launch_sort(ws.ids_local, A, x.e_loc, ws.counts, ws.offsets, ws.perm, ws.inv_perm, ws.sort_scratch,
                        ws.sort_scratch_bytes, &ex, stream));
    GroupedArgs ga = {};
    ga.set = set;
    ga.in = ws.x16;
    ga.row_index = ws.tok_of_slot;
    ga.xs = ws.xs;
    ga.slots_end_dev = ws.offsets + x.e_loc;         // the sorted slots end where the local experts' rows end ...
    ga.slots_resume = A;                             // ... and the shared expert's slots follow the A assignment slots
    ga.n_slots = A + (has_shared ? n : 0);
    ga.units = ws.units;
    ga.n_units = ws.c.n_units;
    ga.max_units = ws.max_units;
    use_sched(ga, ws.c.sw);
    ga.partials = ws.c.partials;
    ga.psum = ws.psum;
    ga.gsum_x = ws.gsum_x;
    ga.n_in_rows = nA;
    ga.gsum_x_ready = sums_done ? 1 : 0;
    ga.act = ws.act;
    ga.act_stride = ws.act_stride;
    ga.row_scale = tc ? nullptr : ws.w_of_slot;
    ga.out = ws.rows;
    ga.out16 = tc ? reinterpret_cast<__half*>(ws.rows) : nullptr;
    ga.status = ws.c.status;
    IMX_TRY(run_experts(path, ga, stream));
    // fp32 partial sums over the local experts, for all tokens (dropped assignments contribute nothing)
    IMX_TRY(launch_combine(ws.rows, tc ? ws.w_of_slot : nullptr, ws.inv_perm, nA, c.top_k, c.hidden, nullptr, ws.partial, stream, true,
                           nullptr, tc));
    IMX_CHECK_NCCL(nc->ReduceScatter(ws.partial, ws.mine, (size_t)n * c.hidden, ncclFloat, ncclSum, x.comm, stream));
    if (tc) {
        // the shared expert's rows of the local tokens are fp16 and ungated on this path
        finish_rows_kernel<<<n, 256, 0, stream>>>(ws.mine, has_shared ? reinterpret_cast<const __half*>(ws.rows) + (size_t)A * c.hidden : nullptr,
                                                 has_shared ? ws.shared_gate + (size_t)x.rank * n : nullptr, c.hidden,
                                                 (__nv_bfloat16*)y); IMX_LAUNCHED();
        IMX_CHECK_CUDA(cudaGetLastError());
    } else {
        IMX_TRY(launch_combine(ws.mine, nullptr, ws.ident, n, 1, c.hidden, has_shared ? ws.rows + (size_t)A * c.hidden : nullptr, y,
                               stream));
    }
    if (info != nullptr) {
        info->schedule = IMX_EP_GATHERED;
        info->rows_received = -1;
        info->bytes_sent = (unsigned long long)(R - 1) * n * c.hidden * 2 + (unsigned long long)(R - 1) * n * c.hidden * 4;
        info->bytes_received = info->bytes_sent;
    }
    return IMX_OK;
}

int forward_a2a(imx_ep_ctx& x, const imx_moe_weights* w, const void* xin, int n, void* y, void* workspace, size_t ws_bytes,
                cudaStream_t stream, imx_ep_info* info, const imx_moe_trace* trace) {
    const NcclApi* nc = nccl_api();
    const imx_moe_config& c = x.cfg;
    QFormat f;
    IMX_TRY(check_config(&c, &f));
    const A2aWs ws = carve_a2a(x, n, workspace);
    if (ws_bytes < ws.bytes) {
        set_error("ep_forward (all-to-all): workspace of %zu bytes needed for %d local tokens, %zu given", ws.bytes, n, ws_bytes);
        return IMX_ERR_WORKSPACE;
    }
    const int R = x.world, E = c.num_experts, H = c.hidden, A = n * c.top_k;
    const bool has_shared = c.shared_intermediate > 0;
    const imx_moe_config cl = local_config(x);
    ExpertSet set;
    IMX_TRY(make_expert_set(cl, f, w->gate_up, w->down, x.e_loc, has_shared ? w : nullptr, &set));
    IMX_REQUIRE(prefill_tc_supported(set),
                "ep_forward (all-to-all): this schedule runs the tensor-core expert kernels, which do not take this "
                "format/shape; use the gathered schedule");
    const int path = IMX_PATH_PREFILL;
    int order[16];
    path_block_order(path, f, order);
    const bool timed = info != nullptr && info->want_timing != 0;
    if (timed && !x.have_events) {
        for (int i = 0; i < 6; ++i) IMX_CHECK_CUDA(cudaEventCreate(&x.ev[i]));
        x.have_events = true;
    }
    auto mark = [&](int i) -> cudaError_t { return timed ? cudaEventRecord(x.ev[i], stream) : cudaSuccess; };
    IMX_CHECK_CUDA(mark(0));

    // 1. route the local tokens; their fp16 rows land behind the receive buffer's `cap` rows, where the shared
    //    expert's slots will find them
    __half* x16 = ws.recv_buf + (size_t)ws.cap * H;
    RouteScratch rs = {ws.route_partials, ws.route_sg, nullptr, nullptr, nullptr};
    IMX_TRY(launch_route(xin, n, H, w->router_w, w->router_logit_bias, E, c.top_k, c.norm_topk_prob,
                         has_shared ? w->shared_expert_gate_w : nullptr, ws.topk_idx, ws.topk_w, ws.shared_gate, x16, order,
                         stream, 1.f, ws.route_partials ? &rs : nullptr, nullptr));
    // 2. stable sort by global expert id, rows packed in that order
    SortExtras ex;
    ex.topk_w = ws.topk_w;
    ex.top_k = c.top_k;
    ex.tok_of_slot = ws.tok_of_slot;
    ex.w_of_slot = ws.w_of_slot;
    IMX_TRY(launch_sort(ws.topk_idx, A, E, ws.counts, ws.offsets, ws.perm, ws.inv_perm, ws.sort_scratch, ws.sort_scratch_bytes,
                        &ex, stream));
    IMX_TRY(launch_gather_rows(x16, ws.tok_of_slot, A, (size_t)H * 2, ws.send_buf, stream));
    IMX_CHECK_CUDA(mark(1));
    // 3. everyone's counts; the split sizes are host values: the one synchronisation of the step
    IMX_CHECK_NCCL(nc->AllGather(ws.counts, ws.all_counts, (size_t)E, ncclInt32, x.comm, stream));
    IMX_CHECK_CUDA(cudaMemcpyAsync(x.host_counts, ws.all_counts, sizeof(int32_t) * R * E, cudaMemcpyDeviceToHost, stream));
    IMX_CHECK_CUDA(cudaStreamSynchronize(stream));
    size_t sent_total = 0, n_recv = 0;
    for (int p = 0; p < R; ++p) {
        size_t s = 0, r = 0;
        for (int e = 0; e < x.e_loc; ++e) {
            const int cs = x.host_counts[(size_t)x.rank * E + p * x.e_loc + e];      // mine, for rank p's experts
            const int cr = x.host_counts[(size_t)p * E + x.rank * x.e_loc + e];      // rank p's, for my experts
            IMX_REQUIRE(cs >= 0 && cr >= 0, "ep_forward: negative count in the exchange (rank %d, expert %d)", p, e);
            s += (size_t)cs;
            r += (size_t)cr;
        }
        x.send_rows[p] = s;
        x.recv_rows[p] = r;
        sent_total += s;
        n_recv += r;
    }
    // a rank that disagrees about the exchange must not reach the data collectives
    IMX_REQUIRE(sent_total == (size_t)A, "ep_forward: dispatch counts sum to %zu, expected %d assignments", sent_total, A);
    IMX_REQUIRE(n_recv <= (size_t)ws.cap, "ep_forward: %zu rows to receive exceed the workspace capacity %d", n_recv, ws.cap);
    // 4. dispatch
    {
        size_t so = 0, ro = 0;
        IMX_CHECK_NCCL(nc->GroupStart());
        for (int p = 0; p < R; ++p) {
            if (p != x.rank) {
                if (x.send_rows[p]) IMX_CHECK_NCCL(nc->Send(ws.send_buf + so * H, x.send_rows[p] * H, ncclHalf, p, x.comm, stream));
                if (x.recv_rows[p]) IMX_CHECK_NCCL(nc->Recv(ws.recv_buf + ro * H, x.recv_rows[p] * H, ncclHalf, p, x.comm, stream));
            }
            so += x.send_rows[p];
            ro += x.recv_rows[p];
        }
        IMX_CHECK_NCCL(nc->GroupEnd());
        so = ro = 0;
        for (int p = 0; p < x.rank; ++p) { so += x.send_rows[p]; ro += x.recv_rows[p]; }
        if (x.send_rows[x.rank])
            IMX_CHECK_CUDA(cudaMemcpyAsync(ws.recv_buf + ro * H, ws.send_buf + so * H, x.send_rows[x.rank] * H * 2,
                                           cudaMemcpyDeviceToDevice, stream));
    }
    IMX_CHECK_CUDA(mark(2));
    // 5. expert-major view of the received rows (+ the shared expert's slots), unit list
    ep_regroup_kernel<<<x.e_loc + 1, 256, 0, stream>>>(ws.all_counts, R, E, x.rank * x.e_loc, x.e_loc, ws.cap, n, has_shared ? 1 : 0,
                                                     ws.row_index, ws.offsets2); IMX_LAUNCHED();
    IMX_CHECK_CUDA(cudaGetLastError());
    IMX_TRY(launch_build_units(ws.offsets2, x.e_loc + (has_shared ? 1 : 0), unit_rows_for(path), ws.units, ws.c.n_units, ws.c.sw.sched,
                               ws.c.sw.n_ints, stream, has_shared ? x.e_loc : -1));
    // 6. the experts: rows come in through row_index, results leave through it (row j of ret_buf is the result
    //    of row j of recv_buf)
    GroupedArgs ga = {};
    ga.set = set;
    ga.in = ws.recv_buf;
    ga.row_index = ws.row_index;
    ga.xs = ws.xs;
    ga.n_slots = (int)n_recv + (has_shared ? n : 0);
    ga.units = ws.units;
    ga.n_units = ws.c.n_units;
    ga.max_units = ws.max_units;
    use_sched(ga, ws.c.sw);
    ga.partials = ws.c.partials;
    ga.n_in_rows = ws.cap + n;
    ga.act = ws.act;
    ga.act_stride = ws.act_stride;
    ga.row_scale = nullptr;
    ga.out16 = ws.ret_buf;
    ga.out_index = ws.row_index;
    ga.status = ws.c.status;
    if (ga.n_slots > 0) IMX_TRY(run_experts(path, ga, stream));
    IMX_CHECK_CUDA(mark(3));
    // 7. the rows travel back: what came from rank p returns to rank p, into this rank's sorted slot order
    {
        size_t so = 0, ro = 0;
        IMX_CHECK_NCCL(nc->GroupStart());
        for (int p = 0; p < R; ++p) {
            if (p != x.rank) {
                if (x.recv_rows[p]) IMX_CHECK_NCCL(nc->Send(ws.ret_buf + ro * H, x.recv_rows[p] * H, ncclHalf, p, x.comm, stream));
                if (x.send_rows[p]) IMX_CHECK_NCCL(nc->Recv(ws.rows_back + so * H, x.send_rows[p] * H, ncclHalf, p, x.comm, stream));
            }
            so += x.send_rows[p];
            ro += x.recv_rows[p];
        }
        IMX_CHECK_NCCL(nc->GroupEnd());
        so = ro = 0;
        for (int p = 0; p < x.rank; ++p) { so += x.send_rows[p]; ro += x.recv_rows[p]; }
        if (x.send_rows[x.rank])
            IMX_CHECK_CUDA(cudaMemcpyAsync(ws.rows_back + so * H, ws.ret_buf + ro * H, x.send_rows[x.rank] * H * 2,
                                           cudaMemcpyDeviceToDevice, stream));
    }
    IMX_CHECK_CUDA(mark(4));
    // 8. weighted combine on the source rank, ascending slot order; the shared rows sit behind the received ones
    IMX_TRY(launch_combine(ws.rows_back, ws.w_of_slot, ws.inv_perm, n, c.top_k, H,
                           has_shared ? ws.ret_buf + (size_t)ws.cap * H : nullptr, y, stream, false, nullptr, true,
                           has_shared ? ws.shared_gate : nullptr));
    IMX_CHECK_CUDA(mark(5));
    if (trace != nullptr) {
        auto cp = [&](void* dst, const void* src, size_t bytes) -> cudaError_t {
            return dst ? cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, stream) : cudaSuccess;
        };
        IMX_CHECK_CUDA(cp(trace->topk_idx, ws.topk_idx, (size_t)A * 4));
        IMX_CHECK_CUDA(cp(trace->topk_w, ws.topk_w, (size_t)A * 4));
        IMX_CHECK_CUDA(cp(trace->counts, ws.counts, (size_t)E * 4));
        IMX_CHECK_CUDA(cp(trace->offsets, ws.offsets, (size_t)(E + 1) * 4));
        IMX_CHECK_CUDA(cp(trace->perm, ws.perm, (size_t)A * 4));
        IMX_CHECK_CUDA(cp(trace->inv_perm, ws.inv_perm, (size_t)A * 4));
        if (has_shared) IMX_CHECK_CUDA(cp(trace->shared_gate, ws.shared_gate, (size_t)n * 4));
    }
    if (timed) {
        // local preparation, dispatch (count exchange, host round trip, rows), experts, return, combine
        IMX_CHECK_CUDA(cudaEventSynchronize(x.ev[5]));
        for (int i = 0; i < 5; ++i) IMX_CHECK_CUDA(cudaEventElapsedTime(&info->phase_ms[i], x.ev[i], x.ev[i + 1]));
    }
    if (info != nullptr) {
        info->schedule = IMX_EP_ALL_TO_ALL;
        info->rows_received = (long long)n_recv;
        info->bytes_sent = (unsigned long long)(sent_total - x.send_rows[x.rank]) * H * 2 +
                           (unsigned long long)(n_recv - x.recv_rows[x.rank]) * H * 2;
        info->bytes_received = info->bytes_sent;
    }
    return IMX_OK;
}

int pick_schedule(const imx_ep_ctx& x, int n, int schedule) {
    if (schedule != IMX_EP_AUTO) return schedule;
    // Decode-size batches: fixed shapes and no host round trip.  Beyond that, whichever moves fewer bytes: the
    // gathered schedule sends a token's bf16 row out and its fp32 partial row back once per other rank,
    // (R - 1) * 6 * H bytes; the all-to-all schedule sends the fp16 rows of its k assignments both ways,
    // 2 * k * (R - 1) / R * 2 * H bytes -- fewer from 2 k < 3 R on (top-8: eight ranks and more).
    if ((long)n * x.world <= 1023) return IMX_EP_GATHERED;
    if ((long)n * x.world * x.cfg.top_k > (1L << 24)) return IMX_EP_ALL_TO_ALL;
    return 2 * x.cfg.top_k >= 3 * x.world ? IMX_EP_GATHERED : IMX_EP_ALL_TO_ALL;
}

}  // namespace

}  // namespace imx

using namespace imx;

extern "C" {

int imx_ep_unique_id(void* id128) {
    const NcclApi* nc = nccl_api();
    IMX_REQUIRE(nc != nullptr, "NCCL (libnccl.so.2) could not be loaded");
    IMX_REQUIRE(id128 != nullptr, "ep_unique_id: output is NULL");
    ncclUniqueId id;
    IMX_CHECK_NCCL(nc->GetUniqueId(&id));
    memcpy(id128, &id, sizeof(id));
    return IMX_OK;
}

static int ep_new(const imx_moe_config* cfg, int rank, int world, imx_ep_ctx** out) {
    QFormat f;
    IMX_TRY(check_config(cfg, &f));
    IMX_REQUIRE(out != nullptr, "ep_create: output is NULL");
    IMX_REQUIRE(world >= 1 && world <= 64 && rank >= 0 && rank < world, "ep_create: rank %d of %d", rank, world);
    IMX_REQUIRE(cfg->num_experts % world == 0, "ep_create: num_experts (%d) must be divisible by the number of ranks (%d)",
                cfg->num_experts, world);
    imx_ep_ctx* x = new imx_ep_ctx();
    x->cfg = *cfg;
    x->rank = rank;
    x->world = world;
    x->e_loc = cfg->num_experts / world;
    x->comm = nullptr;
    x->own_comm = false;
    x->host_counts = nullptr;
    x->send_rows.assign(world, 0);
    x->recv_rows.assign(world, 0);
    x->have_events = false;
    if (cudaGetDevice(&x->device) != cudaSuccess ||
        cudaMallocHost((void**)&x->host_counts, sizeof(int32_t) * (size_t)world * cfg->num_experts) != cudaSuccess) {
        set_error("ep_create: pinned host buffer for the count matrix could not be allocated");
        delete x;
        return IMX_ERR_CUDA;
    }
    *out = x;
    return IMX_OK;
}

int imx_ep_create(const imx_moe_config* cfg, const void* unique_id, int rank, int world, imx_ep_ctx** out) {
    const NcclApi* nc = nccl_api();
    IMX_REQUIRE(nc != nullptr, "NCCL (libnccl.so.2) could not be loaded");
    IMX_REQUIRE(unique_id != nullptr, "ep_create: unique id is NULL");
    imx_ep_ctx* x = nullptr;
    IMX_TRY(ep_new(cfg, rank, world, &x));
    ncclUniqueId id;
    memcpy(&id, unique_id, sizeof(id));
    ncclResult_t r = nc->CommInitRank(&x->comm, world, id, rank);
    if (r != ncclSuccess) {
        set_error("ncclCommInitRank failed: %s", nc->GetErrorString(r));
        cudaFreeHost(x->host_counts);
        delete x;
        return IMX_ERR_CUDA;
    }
    x->own_comm = true;
    *out = x;
    return IMX_OK;
}

int imx_ep_create_from_comm(const imx_moe_config* cfg, void* nccl_comm, int rank, int world, imx_ep_ctx** out) {
    IMX_REQUIRE(nccl_api() != nullptr, "NCCL (libnccl.so.2) could not be loaded");
    IMX_REQUIRE(nccl_comm != nullptr, "ep_create_from_comm: communicator is NULL");
    imx_ep_ctx* x = nullptr;
    IMX_TRY(ep_new(cfg, rank, world, &x));
    x->comm = (ncclComm_t)nccl_comm;
    *out = x;
    return IMX_OK;
}

void* imx_ep_comm(const imx_ep_ctx* x) { return x == nullptr ? nullptr : (void*)x->comm; }

int imx_ep_destroy(imx_ep_ctx* x) {
    if (x == nullptr) return IMX_OK;
    const NcclApi* nc = nccl_api();
    if (x->own_comm && x->comm != nullptr && nc != nullptr) nc->CommDestroy(x->comm);
    if (x->host_counts != nullptr) cudaFreeHost(x->host_counts);
    if (x->have_events)
        for (int i = 0; i < 6; ++i) cudaEventDestroy(x->ev[i]);
    delete x;
    return IMX_OK;
}

int imx_ep_workspace_bytes(const imx_ep_ctx* x, int n_local, int schedule, size_t* bytes) {
    IMX_REQUIRE(x != nullptr && bytes != nullptr && n_local >= 0, "ep_workspace_bytes: bad arguments");
    const int s = pick_schedule(*x, n_local, schedule);
    IMX_REQUIRE(s == IMX_EP_GATHERED || s == IMX_EP_ALL_TO_ALL, "ep_workspace_bytes: unknown schedule %d", schedule);
    *bytes = s == IMX_EP_GATHERED ? carve_gather(*x, n_local, nullptr).bytes : carve_a2a(*x, n_local, nullptr).bytes;
    return IMX_OK;
}

int imx_ep_forward(imx_ep_ctx* x, const imx_moe_weights* w, const void* xin, int n_local, void* y, void* workspace,
                   size_t workspace_bytes, void* stream, int schedule, imx_ep_info* info, const imx_moe_trace* trace) {
    IMX_REQUIRE(x != nullptr && w != nullptr && w->router_w != nullptr, "ep_forward: context and weights are required");
    IMX_REQUIRE(n_local > 0 && xin != nullptr && y != nullptr, "ep_forward: every rank brings the same positive number of tokens");
    IMX_REQUIRE(((uintptr_t)xin % 16) == 0 && ((uintptr_t)y % 16) == 0, "ep_forward: x and y must be 16-byte aligned");
    IMX_REQUIRE(x->cfg.shared_intermediate == 0 || w->shared_expert_gate_w != nullptr, "ep_forward: shared_expert_gate weight is required");
    if (workspace == nullptr || ((uintptr_t)workspace % 256) != 0) {
        set_error("ep_forward: workspace must be a 256-byte aligned device pointer");
        return IMX_ERR_WORKSPACE;
    }
    int dev = -1;
    IMX_CHECK_CUDA(cudaGetDevice(&dev));
    IMX_REQUIRE(dev == x->device, "ep_forward: the context was created on device %d, the current device is %d", x->device, dev);
    const int s = pick_schedule(*x, n_local, schedule);
    if (s == IMX_EP_GATHERED) {
        IMX_REQUIRE((long)n_local * x->world * x->cfg.top_k <= (1L << 24), "ep_forward (gathered): batch too large for this schedule");
        return forward_gathered(*x, w, xin, n_local, y, workspace, workspace_bytes, (cudaStream_t)stream, info);
    }
    IMX_REQUIRE(s == IMX_EP_ALL_TO_ALL, "ep_forward: unknown schedule %d", schedule);
    return forward_a2a(*x, w, xin, n_local, y, workspace, workspace_bytes, (cudaStream_t)stream, info, trace);
}

}  // extern "C"
