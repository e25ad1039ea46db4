// Dispatch stage of the MoE block: the host bucketing loop of
// mlx/src/nn/moe.rs:93-104 as a deterministic, stable counting sort on the GPU.
//
// The reference walks tokens in order and slots in order and appends
// (token, token*k+slot) to its expert's list, so the dispatch permutation is
// the STABLE sort of the flat assignment indices by expert id.  Here:
//   rank  each warp ranks 32 ids at a time with __match_any_sync (peers with
//         the same expert, lower lanes first) on top of a per-warp running
//         histogram in shared memory; no order-dependent atomics anywhere
//   scan  per expert, an exclusive scan over warps (and over blocks when the
//         input spans several), then an exclusive scan over experts
//   place perm[offset[e] + block base + warp base + rank] = flat index
// Small inputs (decode) run the three steps in ONE single-block kernel that
// also emits the per-slot gather/scale arrays and the work-unit list of the
// expert kernels; large inputs use three launches.
#include <mutex>

#include "common.cuh"
#include "internal.h"

namespace imx {

namespace {

constexpr int kSortThreads = 1024;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kSortChunk = 4096;   // ids per block in the multi-block path

// Block-wide exclusive scan of one int per thread (all threads must call).
__device__ int block_exclusive_scan(int v, int* s_warp /*[32]*/, int* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int w = (lane < (int)(blockDim.x >> 5)) ? s_warp[lane] : 0;
        int winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int t = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += t;
        }
        s_warp[lane] = winc - w;   // exclusive warp base
        if (lane == 31) s_warp[32] = winc;
    }
    __syncthreads();
    int res = s_warp[warp] + inc - v;
    if (total) *total = s_warp[32];
    __syncthreads();
    return res;
}

// Step 1 for the ids [lo, hi) of this block: block-local stable rank of every
// id among equal ids (written to rank_out) and per-expert totals left in
// s_hist[0][e]..: on return s_tot[e] holds the block's count of expert e.
__device__ void block_rank(const int32_t* __restrict__ ids, int lo, int hi, int E,
                           int* s_hist /*[kSortWarps][E]*/, int* s_tot /*[E]*/,
                           int32_t* __restrict__ rank_out) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int i = tid; i < kSortWarps * E; i += kSortThreads) s_hist[i] = 0;
    __syncthreads();
    const int n = hi - lo;
    int per_warp = ((n + kSortWarps - 1) / kSortWarps + 31) & ~31;
    const int w_lo = lo + warp * per_warp;
    const int w_hi = min(hi, w_lo + per_warp);
    int* my_hist = s_hist + warp * E;
    const unsigned lt = (1u << lane) - 1u;
    for (int base = w_lo; base < w_hi; base += 32) {
        const int i = base + lane;
        int e = (i < w_hi) ? ids[i] : -1;
        if (e < 0 || e >= E) e = -1;                    // moe.rs:100: out-of-range ids are dropped
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        int before = 0;
        if (e >= 0) before = my_hist[e];
        __syncwarp();
        if (e >= 0) {
            const int r = __popc(peers & lt);
            if (r == 0) my_hist[e] = before + __popc(peers);
            rank_out[i] = before + r;
        }
        __syncwarp();
    }
    __syncthreads();
    // exclusive scan over warps, per expert
    for (int e = tid; e < E; e += kSortThreads) {
        int run = 0;
        for (int w = 0; w < kSortWarps; ++w) {
            int t = s_hist[w * E + e];
            s_hist[w * E + e] = run;
            run += t;
        }
        s_tot[e] = run;
    }
    __syncthreads();
    // fold the warp base into the stored ranks
    for (int base = w_lo; base < w_hi; base += 32) {
        const int i = base + lane;
        if (i < w_hi) {
            int e = ids[i];
            if (e >= 0 && e < E) rank_out[i] += my_hist[e];
        }
    }
}

// Exclusive scan of s_tot[0..E) into offsets[0..E] (E <= 1024 = blockDim).
__device__ void scan_experts(const int* s_tot, int E, int32_t* __restrict__ offsets, int* s_off,
                             int* s_warp) {
    const int tid = threadIdx.x;
    int v = tid < E ? s_tot[tid] : 0;
    int total;
    int ex = block_exclusive_scan(v, s_warp, &total);
    if (tid < E) {
        s_off[tid] = ex;
        offsets[tid] = ex;
    }
    if (tid == 0) {
        s_off[E] = total;
        offsets[E] = total;
    }
    __syncthreads();
}

// Units of an expert with `cnt` rows.  Tensor-core tiles (unit sizes of 64 rows and more) cost the same
// whether full or not, so an expert that needs nu of them gets nu even parts (multiples of 16 rows) instead of
// full units and a remainder; very long lists (nu > 8, e.g. the shared expert's) keep the fixed stride.
__device__ __forceinline__ int unit_stride(int cnt, int ur, int nu) {
    if (ur < 64 || nu <= 1 || nu > 8) return ur;
    return (((cnt + nu - 1) / nu) + 15) & ~15;
}

struct SortAux {
    // optional extras emitted by the fused kernel (all may be null)
    const float* topk_w;     // [A] routing weight per flat assignment
    int top_k;
    int32_t* tok_of_slot;    // [A (+N)] token id per sorted slot
    float* w_of_slot;        // [A (+N)] routing weight per sorted slot
    const float* shared_gate;// [N] or null: appended after the A routed slots
    int n_tokens;
    int shared_token0;       // first of the n_tokens tokens the shared expert serves (0 unless tokens are sharded)
    WorkUnit* units;         // work units of `unit_rows` rows
    int32_t* n_units;
    int unit_rows;
    int32_t* sched;          // scheduler words to clear
    int sched_ints;
};

__device__ void emit_aux(const SortAux& aux, const int32_t* __restrict__ perm, const int* s_off,
                         int E, int A, int* s_warp) {
    const int tid = threadIdx.x;
    if (aux.sched != nullptr)
        for (int i = tid; i < aux.sched_ints; i += kSortThreads) aux.sched[i] = 0;
    if (aux.tok_of_slot != nullptr) {
        const int total = s_off[E];
        for (int j = tid; j < total; j += kSortThreads) {
            int f = perm[j];
            aux.tok_of_slot[j] = f / aux.top_k;
            if (aux.w_of_slot) aux.w_of_slot[j] = aux.topk_w ? aux.topk_w[f] : 1.f;
        }
        if (aux.shared_gate != nullptr) {
            for (int t = tid; t < aux.n_tokens; t += kSortThreads) {
                aux.tok_of_slot[A + t] = aux.shared_token0 + t;
                if (aux.w_of_slot) aux.w_of_slot[A + t] = aux.shared_gate[aux.shared_token0 + t];
            }
        }
    }
    if (aux.units != nullptr) {
        const int ur = aux.unit_rows;
        // E routed experts + (optionally) the shared expert as pseudo-expert E
        const bool has_shared = aux.shared_gate != nullptr;
        int cnt = 0, pos0 = 0;
        if (tid < E) {
            cnt = s_off[tid + 1] - s_off[tid];
            pos0 = s_off[tid];
        } else if (tid == E && has_shared) {
            cnt = aux.n_tokens;
            pos0 = A;
        }
        int nu = (cnt + ur - 1) / ur;
        int total;
        int base = block_exclusive_scan(nu, s_warp, &total);
        const int per = unit_stride(cnt, ur, nu);
        for (int c = 0; c < nu; ++c) {
            WorkUnit u;
            u.expert = tid;
            u.slot0 = pos0 + c * per;
            u.rows = min(per, cnt - c * per);
            u.pad = 0;
            aux.units[base + c] = u;
        }
        if (tid == 0) aux.n_units[0] = total;
        if (tid == E) aux.n_units[1] = base;       // units of the routed experts (the extra expert's follow)
    }
}

// One block does everything (A <= kSortChunk).
__global__ void __launch_bounds__(kSortThreads)
sort_fused_kernel(const int32_t* __restrict__ ids, int A, int E, int32_t* __restrict__ counts,
                  int32_t* __restrict__ offsets, int32_t* __restrict__ perm,
                  int32_t* __restrict__ inv_perm, SortAux aux) {
    extern __shared__ int s_mem[];
    int* s_hist = s_mem;                       // [kSortWarps][E]
    int* s_tot = s_hist + kSortWarps * E;      // [E]
    int* s_off = s_tot + E;                    // [E+1]
    int* s_warp = s_off + E + 1;               // [33]
    block_rank(ids, 0, A, E, s_hist, s_tot, inv_perm);
    __syncthreads();
    const int tid = threadIdx.x;
    if (tid < E && counts != nullptr) counts[tid] = s_tot[tid];
    scan_experts(s_tot, E, offsets, s_off, s_warp);
    for (int i = tid; i < A; i += kSortThreads) {
        int e = ids[i];
        if (e >= 0 && e < E) {
            int pos = s_off[e] + inv_perm[i];
            perm[pos] = i;
            inv_perm[i] = pos;
        } else {
            inv_perm[i] = -1;
        }
    }
    __syncthreads();
    emit_aux(aux, perm, s_off, E, A, s_warp);
}

// One block, at most kSmallSortIters ids per thread (A <= kSmallSortIters * kSortThreads, E <=
// kSmallSortExperts): ids are read once, ranks stay in registers, and every output is written once
// (decode-size batches).  A warp owns a contiguous run of ids, so ranks follow the index order.
constexpr int kSmallSortExperts = 256;
constexpr int kSmallSortIters = 4;

__global__ void __launch_bounds__(kSortThreads)
sort_small_kernel(const int32_t* __restrict__ ids, int A, int E, int32_t* __restrict__ counts,
                  int32_t* __restrict__ offsets, int32_t* __restrict__ perm,
                  int32_t* __restrict__ inv_perm, SortAux aux) {
    extern __shared__ int s_mem[];
    int* s_hist = s_mem;                       // [kSortWarps][E]
    int* s_tot = s_hist + kSortWarps * E;      // [E]
    int* s_off = s_tot + E;                    // [E+1]
    int* s_warp = s_off + E + 1;               // [33]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int per_warp = ((A + kSortWarps - 1) / kSortWarps + 31) & ~31;      // <= 32 * kSmallSortIters
    const int w_lo = warp * per_warp, w_hi = min(A, w_lo + per_warp);
    int e[kSmallSortIters], rank[kSmallSortIters];
    float w[kSmallSortIters];
#pragma unroll
    for (int it = 0; it < kSmallSortIters; ++it) {
        const int i = w_lo + it * 32 + lane;
        const bool in = it * 32 < per_warp && i < w_hi;
        int v = in ? ids[i] : -1;
        if (v < 0 || v >= E) v = -1;                      // moe.rs:100: out-of-range ids are dropped
        e[it] = v;
        w[it] = (in && aux.topk_w != nullptr) ? aux.topk_w[i] : 1.f;
        rank[it] = 0;
    }
    for (int i = tid; i < kSortWarps * E; i += kSortThreads) s_hist[i] = 0;
    __syncthreads();
    int* my_hist = s_hist + warp * E;
    const unsigned lt = (1u << lane) - 1u;
#pragma unroll
    for (int it = 0; it < kSmallSortIters; ++it) {
        if (it * 32 < per_warp) {
            // rank among equal ids: those of earlier passes of the warp, then lower lanes of this pass
            const unsigned peers = __match_any_sync(0xffffffffu, e[it]);
            const int before = e[it] >= 0 ? my_hist[e[it]] : 0;
            __syncwarp();
            if (e[it] >= 0) {
                const int r = __popc(peers & lt);
                if (r == 0) my_hist[e[it]] = before + __popc(peers);
                rank[it] = before + r;
            }
            __syncwarp();
        }
    }
    __syncthreads();
    for (int x = tid; x < E; x += kSortThreads) {          // exclusive scan over warps, per expert
        int run = 0;
        for (int v = 0; v < kSortWarps; ++v) {
            const int c = s_hist[v * E + x];
            s_hist[v * E + x] = run;
            run += c;
        }
        s_tot[x] = run;
        if (counts != nullptr) counts[x] = run;
    }
    __syncthreads();
#pragma unroll
    for (int it = 0; it < kSmallSortIters; ++it)
        if (e[it] >= 0) rank[it] += my_hist[e[it]];
    scan_experts(s_tot, E, offsets, s_off, s_warp);
#pragma unroll
    for (int it = 0; it < kSmallSortIters; ++it) {
        const int i = w_lo + it * 32 + lane;
        if (it * 32 < per_warp && i < w_hi) {
            if (e[it] >= 0) {
                const int pos = s_off[e[it]] + rank[it];
                perm[pos] = i;
                inv_perm[i] = pos;
                if (aux.tok_of_slot != nullptr) {
                    aux.tok_of_slot[pos] = i / aux.top_k;
                    if (aux.w_of_slot) aux.w_of_slot[pos] = w[it];
                }
            } else {
                inv_perm[i] = -1;
            }
        }
    }
    if (aux.tok_of_slot != nullptr && aux.shared_gate != nullptr) {
        for (int t = tid; t < aux.n_tokens; t += kSortThreads) {
            aux.tok_of_slot[A + t] = aux.shared_token0 + t;
            if (aux.w_of_slot) aux.w_of_slot[A + t] = aux.shared_gate[aux.shared_token0 + t];
        }
    }
    SortAux rest = aux;
    rest.tok_of_slot = nullptr;                           // written above; what remains: unit list, scheduler reset
    emit_aux(rest, nullptr, s_off, E, A, s_warp);
}

// Multi-block path, launch 1: ranks inside each block + per-block totals.
__global__ void __launch_bounds__(kSortThreads)
sort_rank_kernel(const int32_t* __restrict__ ids, int A, int E, int32_t* __restrict__ rank_tmp,
                 int32_t* __restrict__ block_counts /*[nb][E]*/) {
    extern __shared__ int s_mem[];
    int* s_hist = s_mem;
    int* s_tot = s_hist + kSortWarps * E;
    const int lo = blockIdx.x * kSortChunk;
    const int hi = min(A, lo + kSortChunk);
    block_rank(ids, lo, hi, E, s_hist, s_tot, rank_tmp);
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += kSortThreads) block_counts[(size_t)blockIdx.x * E + e] = s_tot[e];
}

// Launch 2 (one block): scan over blocks per expert, then over experts.
__global__ void __launch_bounds__(kSortThreads)
sort_scan_kernel(int32_t* __restrict__ block_counts, int nb, int E, int32_t* __restrict__ counts,
                 int32_t* __restrict__ offsets, SortAux aux, int A) {
    extern __shared__ int s_mem[];
    int* s_tot = s_mem;             // [E]
    int* s_off = s_tot + E;         // [E+1]
    int* s_warp = s_off + E + 1;    // [33]
    const int tid = threadIdx.x;
    if (tid < E) {
        int run = 0;
        for (int b = 0; b < nb; ++b) {
            int t = block_counts[(size_t)b * E + tid];
            block_counts[(size_t)b * E + tid] = run;
            run += t;
        }
        s_tot[tid] = run;
        if (counts != nullptr) counts[tid] = run;
    }
    __syncthreads();
    scan_experts(s_tot, E, offsets, s_off, s_warp);
    // unit list and scheduler reset only (the per-slot arrays need perm: launch 3)
    SortAux a2 = aux;
    a2.tok_of_slot = nullptr;
    emit_aux(a2, nullptr, s_off, E, A, s_warp);
}

// Launch 3: place.
__global__ void __launch_bounds__(256)
sort_place_kernel(const int32_t* __restrict__ ids, int A, int E, const int32_t* __restrict__ offsets,
                  const int32_t* __restrict__ block_counts, int32_t* __restrict__ perm,
                  int32_t* __restrict__ inv_perm /* holds ranks on entry */, SortAux aux) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < A) {
        int e = ids[i];
        if (e >= 0 && e < E) {
            int b = i / kSortChunk;
            int pos = offsets[e] + block_counts[(size_t)b * E + e] + inv_perm[i];
            perm[pos] = i;
            inv_perm[i] = pos;
            if (aux.tok_of_slot != nullptr) {
                aux.tok_of_slot[pos] = i / aux.top_k;
                if (aux.w_of_slot) aux.w_of_slot[pos] = aux.topk_w ? aux.topk_w[i] : 1.f;
            }
        } else {
            inv_perm[i] = -1;
        }
    }
    if (aux.tok_of_slot != nullptr && aux.shared_gate != nullptr && i < aux.n_tokens) {
        aux.tok_of_slot[A + i] = aux.shared_token0 + i;
        if (aux.w_of_slot) aux.w_of_slot[A + i] = aux.shared_gate[aux.shared_token0 + i];
    }
}

}  // namespace

// Unit list for a caller-given offsets array (stage-level API): one thread per expert, a block scan for
// the positions; also clears the scheduler words.
static __global__ void __launch_bounds__(kSortThreads)
build_units_kernel(const int32_t* __restrict__ offsets, int E, int unit_rows, WorkUnit* __restrict__ units,
                   int32_t* __restrict__ n_units, int32_t* __restrict__ sched, int sched_ints, int extra_from) {
    __shared__ int s_warp[33];
    const int tid = threadIdx.x;
    int cnt = 0, pos0 = 0;
    if (tid < E) {
        pos0 = offsets[tid];
        cnt = offsets[tid + 1] - pos0;
    }
    const int nu = (cnt + unit_rows - 1) / unit_rows;
    int total;
    const int base = block_exclusive_scan(nu, s_warp, &total);
    const int per = unit_stride(cnt, unit_rows, nu);
    for (int c = 0; c < nu; ++c) {
        WorkUnit u;
        u.expert = tid;
        u.slot0 = pos0 + c * per;
        u.rows = min(per, cnt - c * per);
        u.pad = 0;
        units[base + c] = u;
    }
    if (tid == 0) n_units[0] = total;
    // units of the routed experts come first; those of expert `extra_from` (the shared expert, when the caller
    // lists it as the last "expert") follow
    if (extra_from >= 0 ? tid == extra_from : tid == 0) n_units[1] = extra_from >= 0 ? base : total;
    if (sched != nullptr)
        for (int i = tid; i < sched_ints; i += kSortThreads) sched[i] = 0;
}

int launch_build_units(const int32_t* offsets, int E, int unit_rows, WorkUnit* units, int32_t* n_units,
                       int32_t* sched, int sched_ints, cudaStream_t stream, int extra_from) {
    IMX_REQUIRE(E >= 1 && E < kSortThreads, "build_units: num_experts (%d) must be in 1..%d", E, kSortThreads - 1);
    build_units_kernel<<<1, kSortThreads, 0, stream>>>(offsets, E, unit_rows, units, n_units, sched, sched_ints, extra_from); IMX_LAUNCHED();
    IMX_CHECK_CUDA(cudaGetLastError());
    return IMX_OK;
}

// ── allocation-free variant ─────────────────────────────────────────────────
// Scratch of the multi-block path for callers that cannot provide any: a fixed
// array that lives in the library's device image (every GPU that loads the
// library holds these 256 KB until the process exits).
constexpr int kStaticSortMaxAssign = 262144;                                   // ids per call
constexpr int kStaticSortInts = (kStaticSortMaxAssign / kSortChunk) * 1024;    // blocks x experts
static __device__ __align__(256) int32_t g_sort_scratch[kStaticSortInts];

int launch_sort_static(const int32_t* ids, int A, int E, int32_t* counts, int32_t* offsets, int32_t* perm,
                       int32_t* inv_perm, cudaStream_t stream) {
    IMX_REQUIRE(A >= 0 && A <= kStaticSortMaxAssign,
                "sort_static: %d assignments exceed the built-in scratch (maximum %d); use imx_moe_sort with a "
                "caller-provided scratch buffer", A, kStaticSortMaxAssign);
    IMX_REQUIRE(E >= 1 && E <= 1024, "sort_static: num_experts (%d) must be in 1..1024", E);
    // The array's name is only a host-side handle; kernels need its device
    // address, looked up once per device with that device current.
    static std::mutex mu;
    static void* addr[64] = {};
    int dev = 0;
    IMX_CHECK_CUDA(cudaGetDevice(&dev));
    IMX_REQUIRE(dev >= 0 && dev < 64, "sort_static: device ordinal %d not supported", dev);
    void* ptr = nullptr;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (addr[dev] == nullptr) {
            void* p = nullptr;
            IMX_CHECK_CUDA(cudaGetSymbolAddress(&p, g_sort_scratch));
            addr[dev] = p;
        }
        ptr = addr[dev];
    }
    // every (block, expert) count the later passes read is written by the first pass: nothing to clear
    return launch_sort(ids, A, E, counts, offsets, perm, inv_perm, ptr, sizeof(int32_t) * kStaticSortInts, nullptr,
                       stream);
}

size_t sort_scratch_bytes(int n_assign, int E) {
    int nb = ceil_div(n_assign > 0 ? n_assign : 1, kSortChunk);
    return align_up((size_t)nb * E * sizeof(int32_t), 256);
}

int launch_sort(const int32_t* ids, int A, int E, int32_t* counts, int32_t* offsets, int32_t* perm,
                int32_t* inv_perm, void* scratch, size_t scratch_bytes, const SortExtras* ex,
                cudaStream_t stream) {
    IMX_REQUIRE(A >= 0 && E >= 1 && E <= 1024, "sort: num_experts (%d) must be in 1..1024", E);
    IMX_REQUIRE(offsets && perm && inv_perm, "sort: offsets, perm and inv_perm are required");
    SortAux aux = {};
    if (ex != nullptr) {
        aux.topk_w = ex->topk_w;
        aux.top_k = ex->top_k > 0 ? ex->top_k : 1;
        aux.tok_of_slot = ex->tok_of_slot;
        aux.w_of_slot = ex->w_of_slot;
        aux.shared_gate = ex->shared_gate;
        aux.n_tokens = ex->n_tokens;
        aux.shared_token0 = ex->shared_token0;
        aux.units = ex->units;
        aux.n_units = ex->n_units;
        aux.unit_rows = ex->unit_rows > 0 ? ex->unit_rows : 8;
        aux.sched = ex->sched;
        aux.sched_ints = ex->sched_ints;
        IMX_REQUIRE(aux.units == nullptr || E + 1 <= kSortThreads, "sort: too many experts for the unit list");
    }
    const size_t smem_fused = ((size_t)kSortWarps * E + E + E + 1 + 33) * sizeof(int);
    if (A <= kSmallSortIters * kSortThreads && E <= kSmallSortExperts) {
        sort_small_kernel<<<1, kSortThreads, smem_fused, stream>>>(ids, A, E, counts, offsets, perm, inv_perm, aux); IMX_LAUNCHED();
        IMX_CHECK_CUDA(cudaGetLastError());
        return IMX_OK;
    }
    if (A <= kSortChunk) {
        IMX_CHECK_CUDA(cudaFuncSetAttribute(sort_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            (int)smem_fused));
        sort_fused_kernel<<<1, kSortThreads, smem_fused, stream>>>(ids, A, E, counts, offsets, perm,
                                                                   inv_perm, aux); IMX_LAUNCHED();
        IMX_CHECK_CUDA(cudaGetLastError());
        return IMX_OK;
    }
    const int nb = ceil_div(A, kSortChunk);
    IMX_REQUIRE(scratch != nullptr && scratch_bytes >= (size_t)nb * E * sizeof(int32_t),
                "sort: scratch of %zu bytes needed, %zu given", (size_t)nb * E * sizeof(int32_t), scratch_bytes);
    int32_t* block_counts = (int32_t*)scratch;
    const size_t smem_rank = ((size_t)kSortWarps * E + E) * sizeof(int);
    IMX_CHECK_CUDA(cudaFuncSetAttribute(sort_rank_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)smem_rank));
    sort_rank_kernel<<<nb, kSortThreads, smem_rank, stream>>>(ids, A, E, inv_perm, block_counts); IMX_LAUNCHED();
    IMX_CHECK_CUDA(cudaGetLastError());
    const size_t smem_scan = ((size_t)E + E + 1 + 33) * sizeof(int);
    sort_scan_kernel<<<1, kSortThreads, smem_scan, stream>>>(block_counts, nb, E, counts, offsets, aux, A); IMX_LAUNCHED();
    IMX_CHECK_CUDA(cudaGetLastError());
    int place_n = A;
    if (aux.tok_of_slot && aux.shared_gate && aux.n_tokens > place_n) place_n = aux.n_tokens;
    sort_place_kernel<<<ceil_div(place_n, 256), 256, 0, stream>>>(ids, A, E, offsets, block_counts, perm,
                                                                 inv_perm, aux); IMX_LAUNCHED();
    IMX_CHECK_CUDA(cudaGetLastError());
    return IMX_OK;
}

}  // namespace imx
