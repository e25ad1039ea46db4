/* ironmlx_b200 — C ABI of the B200-native mixture-of-experts block.
 *
 * Drop-in boundary for the hot path of ironmlx's Qwen3.5-MoE model: the body
 * of `MoEMLP::forward_with_stream` (mlx/src/nn/moe.rs:55-183) and the two
 * quantized ops it is built from, `ops::quantized_matmul` and
 * `ops::dequantize` (mlx/src/ops.rs:653-727), which the reference reaches
 * through mlx-sys's bindgen of the mlx-c API.  A Rust `-sys` crate next to
 * mlx-sys binds exactly these symbols.
 *
 * Conventions (they follow the mlx-c conventions the reference relies on,
 * mlx/src/ops.rs:12-27, mlx/src/error.rs:17-54):
 *   - every function returns int, 0 = success; on failure a message is kept
 *     per thread and read with imx_last_error(); nothing aborts or exits;
 *   - all pointers are DEVICE pointers unless the name says `host`;
 *   - work is enqueued on the given cudaStream_t (passed as void*) and the
 *     call returns without synchronising, except where stated;
 *   - no call allocates device memory: scratch comes from the caller as a
 *     workspace whose size imx_moe_workspace_bytes() reports; a workspace (and
 *     the scratch of imx_moe_experts) is zero-filled once by the caller before
 *     its first use: its first word is the device status word, which kernels
 *     only ever set (a bounded wait that ran out) and imx_moe_status() reads
 *     and clears;
 *   - one caller thread per workspace (the reference runs one engine thread
 *     per model, ironmlx/src/engine_pool.rs:79-81).
 *
 * Tensor formats (MLX's, see mlx/src/ops.rs:646-652,688-693):
 *   activations  bf16 row-major [N, hidden]
 *   dense weights bf16 row-major [out, in]
 *   quantized     packed uint32 [.., out, in*bits/32] + scales (+ biases)
 *                 [.., out, in/group]; affine: bf16 scales and biases;
 *                 mxfp8: uint8 ue8m0 scales; nvfp4: uint8 e4m3 scales and one
 *                 fp32 scale for the whole tensor.
 */
#ifndef IRONMLX_B200_H
#define IRONMLX_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define IMX_API __attribute__((visibility("default")))
#else
#define IMX_API
#endif

#define IMX_OK 0
#define IMX_ERR_INVALID 1       /* bad argument / unsupported shape          */
#define IMX_ERR_CUDA 2          /* a CUDA runtime call failed                */
#define IMX_ERR_WORKSPACE 3     /* workspace too small or misaligned         */
#define IMX_ERR_DEVICE 4        /* a kernel recorded an error status         */

#define IMX_MODE_AFFINE 0
#define IMX_MODE_MXFP8 1
#define IMX_MODE_NVFP4 2

/* Execution path of the expert products.  AUTO picks by tokens per expert. */
#define IMX_PATH_AUTO 0
#define IMX_PATH_DECODE 1       /* grouped dequant small-N tensor-core kernel */
#define IMX_PATH_PREFILL 2      /* grouped tcgen05/TMEM GEMM fed by TMA       */
#define IMX_PATH_GENERIC 3      /* scalar dequant-GEMV, any format            */
/* (values above 3 select cross-check kernels: ironmlx_b200_testing.h)        */

/* One quantized tensor: the (weight, scales, biases) triple of a
 * `QuantizedLinear` (mlx/src/nn/linear.rs:13-20).  biases is NULL for
 * mxfp8/nvfp4; global_scale is nvfp4's tensor scale (use 1.0 otherwise). */
typedef struct imx_qtensor {
    const void* w;
    const void* scales;
    const void* biases;
    float global_scale;
} imx_qtensor;

/* Parameters of the block: mlx/src/model/config.rs:32-52 (quantization) and
 * :159-170 (num_experts, num_experts_per_tok, moe_intermediate_size,
 * shared_expert_intermediate_size, norm_topk_prob). */
typedef struct imx_moe_config {
    int hidden;               /* H                                           */
    int num_experts;          /* E                                           */
    int top_k;                /* num_experts_per_tok                         */
    int intermediate;         /* I, expert SwiGLU width                      */
    int shared_intermediate;  /* Is, 0 = no shared expert                    */
    int norm_topk_prob;       /* renormalise the k selected probabilities    */
    int mode;                 /* IMX_MODE_*                                  */
    int bits;                 /* affine 2/3/4/5/6/8; mxfp8 8; nvfp4 4        */
    int group_size;           /* affine 32/64/128; mxfp8 32; nvfp4 16        */
    int path;                 /* IMX_PATH_*                                  */
} imx_moe_config;

/* Weights of one `MoEMLP` (mlx/src/nn/moe.rs:39-52) in the fused checkpoint
 * layout that `build_moe_experts` slices (mlx/src/model/qwen35.rs:581-590):
 * gate_up [E, 2I, .] with the gate rows first, down [E, H, .]. */
typedef struct imx_moe_weights {
    const void* router_w;              /* bf16 [E, H]   (moe.rs:41)          */
    const float* router_logit_bias;    /* fp32 [E] or NULL (synthetic skew)  */
    imx_qtensor gate_up;               /* [E, 2I, H..]                       */
    imx_qtensor down;                  /* [E, H, I..]                        */
    imx_qtensor shared_gate_proj;      /* [Is, H..]     (mlp.rs:12-16)       */
    imx_qtensor shared_up_proj;        /* [Is, H..]                          */
    imx_qtensor shared_down_proj;      /* [H, Is..]                          */
    const void* shared_expert_gate_w;  /* bf16 [1, H]   (moe.rs:47)          */
} imx_moe_weights;

/* Optional per-stage outputs for parity checks; any pointer may be NULL. */
typedef struct imx_moe_trace {
    int32_t* topk_idx;     /* [N, k] expert ids, descending probability      */
    float* topk_w;         /* [N, k] routing weights                         */
    int32_t* counts;       /* [E]    assignments per expert                  */
    int32_t* offsets;      /* [E+1]  exclusive scan of counts                */
    int32_t* perm;         /* [N*k]  flat assignment index per sorted slot   */
    int32_t* inv_perm;     /* [N*k]  sorted slot per flat assignment index   */
    float* shared_gate;    /* [N]    sigmoid(x . w_sg)                       */
} imx_moe_trace;

/* Message of the last failure on the calling thread ("" if none). */
IMX_API const char* imx_last_error(void);

/* Library version string. */
IMX_API const char* imx_version(void);

/* Number of kernels the library has launched in this process so far (launches
 * recorded into a stream capture count once, when they are recorded).  For
 * measurement: the difference around a call is the call's launch count. */
IMX_API unsigned long long imx_launch_count(void);

/* ── the block: MoEMLP::forward_with_stream, mlx/src/nn/moe.rs:55-183 ───── */

/* Scratch bytes imx_moe_forward needs for up to n_tokens tokens. */
IMX_API int imx_moe_workspace_bytes(const imx_moe_config* cfg, int n_tokens, size_t* bytes);

/* y[N,H] (bf16) = MoE(x[N,H] (bf16)).  Replaces moe.rs:55-183 (router,
 * softmax, top-k, bucketing, per-expert SwiGLU, weighted combine, gated
 * shared expert) with no host round trip.  workspace: 256-byte aligned
 * device memory of at least imx_moe_workspace_bytes(). */
IMX_API int imx_moe_forward(const imx_moe_config* cfg, const imx_moe_weights* w, const void* x,
                    int n_tokens, void* y, void* workspace, size_t workspace_bytes,
                    void* stream, const imx_moe_trace* trace);

/* The MoE half of a decoder layer, mlx/src/model/qwen35.rs:271-276:
 *   y = h + MoE(rms_norm(h, ln_weight, eps))
 * with the normalisation applied where the router loads h and the residual added
 * where the combine stage rounds its sums, so neither the normalised activations
 * nor the block output make a round trip through memory on their own.
 * h, y: bf16 [N, H]; ln_weight: bf16 [H] or NULL (rms_norm without weight,
 * mlx/src/fast.rs:37-49).  Same workspace as imx_moe_forward. */
IMX_API int imx_moe_forward_residual(const imx_moe_config* cfg, const imx_moe_weights* w, const void* h,
                             const void* ln_weight, float eps, int n_tokens, void* y, void* workspace,
                             size_t workspace_bytes, void* stream, const imx_moe_trace* trace);

/* y[n_rows, hidden] = rms_norm(x, weight, eps) (mlx/src/nn/norm.rs:21-24 ->
 * fast::rms_norm, mlx/src/fast.rs:37-49); bf16 in and out, weight bf16 [hidden] or NULL. */
IMX_API int imx_rms_norm(const void* x, int n_rows, int hidden, const void* weight, float eps, void* y,
                 void* stream);

/* imx_moe_forward with CUDA events recorded on the stream between its stages;
 * synchronises and returns the five stage durations in milliseconds:
 * router, dispatch sort, first expert product (gate/up + SwiGLU), second
 * expert product (down), combine.  For measurement; not on the serving path. */
IMX_API int imx_moe_forward_timed(const imx_moe_config* cfg, const imx_moe_weights* w, const void* x,
                          int n_tokens, void* y, void* workspace, size_t workspace_bytes,
                          void* stream, float* stage_ms);

/* Same with HOST activations: copies x to the device, runs the block, copies
 * y back, and synchronises the stream before returning.  The workspace must
 * be imx_moe_workspace_bytes() + 2*roundup(N*H*2, 256) bytes (the staged x and y). */
IMX_API int imx_moe_forward_host(const imx_moe_config* cfg, const imx_moe_weights* w,
                         const void* x_host, int n_tokens, void* y_host, void* workspace,
                         size_t workspace_bytes, void* stream);

/* Reads (and clears) the device status word of a workspace -- of
 * imx_moe_forward, or the scratch of imx_moe_experts -- after synchronising
 * the stream; IMX_ERR_DEVICE if a kernel recorded an error (a bounded wait
 * ran out: the call's output is incomplete). */
IMX_API int imx_moe_status(void* workspace, void* stream);

/* The expert kernels carry their intermediate rows in fp16 (SwiGLU outputs; on the tensor-core path also
 * the expert rows) and clamp what exceeds its range (+-65504).  A clamp changes the result, so it is counted in
 * the workspace (per value on the decode paths, per thread and tile on the tensor-core path): this reads the
 * count accumulated since the last call, after synchronising the stream, and clears it.  0 = nothing clamped. */
IMX_API int imx_moe_saturations(void* workspace, void* stream, long long* count);

/* ── stages, for expert parallelism and stage-level parity ─────────────── */

/* Router (moe.rs:67-82): logits = x.W_r^T (+bias), fp32 softmax, top-k in
 * descending order (lower expert id first among equal values), optional
 * renormalisation; also the shared-expert gate sigmoid(x.w_sg) (moe.rs:174-177)
 * when w_sg != NULL, and an fp16 copy of x for the expert products. */
IMX_API int imx_moe_route(const void* x, int n_tokens, int hidden, const void* router_w,
                  const float* logit_bias, int num_experts, int top_k, int norm_topk_prob,
                  const void* shared_gate_w, int32_t* topk_idx, float* topk_w,
                  float* shared_gate, void* x_f16, void* stream);

/* The same stage with caller-provided scratch (imx_moe_route_scratch_bytes bytes, 256-byte aligned):
 * batches below 1024 tokens with a multiple of 32 experts then take the split-K
 * tensor-core router, which reads router_w once per 32 tokens instead of once per
 * token.  Results are the same as imx_moe_route's up to the summation order of
 * the logits. */
IMX_API int imx_moe_route_scratch_bytes(int n_tokens, int hidden, int num_experts, size_t* bytes);
IMX_API int imx_moe_route_ws(const void* x, int n_tokens, int hidden, const void* router_w,
                     const float* logit_bias, int num_experts, int top_k, int norm_topk_prob,
                     const void* shared_gate_w, int32_t* topk_idx, float* topk_w,
                     float* shared_gate, void* x_f16, void* scratch, size_t scratch_bytes,
                     void* stream);

/* Bucketing (moe.rs:93-104) as a stable counting sort of the n_assign =
 * N*k expert ids: counts[E], offsets[E+1], perm[n_assign], inv_perm[n_assign].
 * scratch: imx_moe_sort_scratch_bytes(n_assign, E) bytes. */
IMX_API int imx_moe_sort_scratch_bytes(int n_assign, int num_experts, size_t* bytes);
IMX_API int imx_moe_sort(const int32_t* expert_ids, int n_assign, int num_experts, int32_t* counts,
                 int32_t* offsets, int32_t* perm, int32_t* inv_perm, void* scratch,
                 size_t scratch_bytes, void* stream);

/* The same sort for callers that cannot hand over scratch memory or allocate
 * any.  (No counterpart in the reference: it exists for hosts such as an
 * inference engine thread that runs under a framework-owned memory cap, where
 * every device byte must come from that framework's allocator and a stray
 * cudaMalloc is off limits, or code running at a point where allocating is not
 * permitted at all.)  The scratch is a fixed 256 KB array inside the library's
 * device image, so: at most 262144 ids per call (larger inputs are refused with
 * an error: use imx_moe_sort); the FIRST call on each device looks up the
 * array's device address (one cudaGetSymbolAddress with that device current) and
 * should therefore happen before any stream capture begins; all calls on a
 * device share the one array, so two calls whose kernels can overlap on the GPU
 * (different streams) race: serialise them.  Nothing in the array needs
 * clearing between calls.  Calls no cudaMalloc/cudaFree. */
IMX_API int imx_moe_sort_static(const int32_t* expert_ids, int n_assign, int num_experts, int32_t* counts,
                        int32_t* offsets, int32_t* perm, int32_t* inv_perm, void* stream);

/* Grouped SwiGLU experts (moe.rs:117-131 with Expert::forward, moe.rs:26-32),
 * a gather_qmm-style call: for every expert e and every sorted slot
 * j in [offsets[e], offsets[e+1]):
 *   out[j, :] = row_scale[j] * down_e( silu(gate_e(a)) * up_e(a) ),
 *   a = x_f16[row_index[j], :]
 * x_f16: fp16 [.., H]; out: fp32 [n_rows, H]; row_scale may be NULL (= 1).
 * gate_up/down hold num_experts stacked matrices.  scratch:
 * imx_moe_experts_scratch_bytes(). */
IMX_API int imx_moe_experts_scratch_bytes(const imx_moe_config* cfg, int n_rows, size_t* bytes);
IMX_API int imx_moe_experts(const imx_moe_config* cfg, const imx_qtensor* gate_up, const imx_qtensor* down,
                    int num_experts, const void* x_f16, const int32_t* row_index,
                    const int32_t* offsets, int n_rows, int max_rows_per_expert,
                    const float* row_scale, float* out, void* scratch, size_t scratch_bytes,
                    void* stream);

/* Weighted combine (moe.rs:147-181): y[t] = sum over the k slots of token t,
 * in ascending sorted-slot order (the order the reference's expert loop
 * produces them), of rows[inv_perm[t*k+s]] (already weighted) + shared[t]
 * (already gated; may be NULL), rounded once to bf16. */
IMX_API int imx_moe_combine(const float* rows, const int32_t* inv_perm, int n_tokens, int top_k,
                    int hidden, const float* shared_rows, void* y, void* stream);

/* The same combine for rows that arrive UNWEIGHTED (expert parallelism: the
 * rows come back from the ranks that own the experts): every row is first
 * multiplied by row_scale[slot] in fp32 (moe.rs:155-161), then added as above. */
IMX_API int imx_moe_combine_scaled(const float* rows, const float* row_scale, const int32_t* inv_perm,
                           int n_tokens, int top_k, int hidden, const float* shared_rows, void* y,
                           void* stream);

/* The routed part only, left in fp32 and not rounded: y_f32[t] = sum over the
 * slots of token t whose inv_perm entry is >= 0 of row_scale[slot]*rows[slot]
 * (row_scale may be NULL).  A rank that owns a block of the experts produces
 * this partial sum for all tokens; the ranks' partials are added by a
 * reduce-scatter before the shared expert is added and the result rounded. */
IMX_API int imx_moe_combine_partial(const float* rows, const float* row_scale, const int32_t* inv_perm,
                            int n_tokens, int top_k, int hidden, float* y_f32, void* stream);

/* dst[j, :] = src[index[j], :], rows of row_bytes bytes (a multiple of 4): the
 * `take_axis` of moe.rs:124-127, used to pack the dispatch and return buffers
 * of the expert-parallel exchange. */
IMX_API int imx_gather_rows(const void* src, const int32_t* index, int n_rows, size_t row_bytes, void* dst,
                    void* stream);

/* ── expert parallelism (no counterpart in the reference, which has no
 *    distributed code: it shards the expert loop of moe.rs:117-144) ────── */

/* One process per GPU.  Rank r of R owns experts [r*E/R, (r+1)*E/R): its
 * imx_moe_weights holds gate_up / down of THOSE experts only ([E/R, 2I, .] and
 * [E/R, H, .]); router_w covers all E experts, the shared expert and its gate
 * are replicated.  Every rank brings the same number of tokens.  Collectives run
 * on NCCL, which the library loads at run time (the copy already in the
 * process, else libnccl.so.2). */
typedef struct imx_ep_ctx imx_ep_ctx;

#define IMX_EP_UNIQUE_ID_BYTES 128
#define IMX_EP_AUTO 0        /* gathered up to 1023 tokens over all ranks; beyond that the schedule that moves fewer
                                bytes: gathered while 2 * top_k >= 3 * ranks, else all-to-all */
#define IMX_EP_GATHERED 1    /* all-gather tokens, every rank routes all of them and runs its own experts (decode or
                                tensor-core kernels by batch size), reduce-scatter of fp32 partial rows: fixed shapes,
                                no host synchronisation (can be captured in a CUDA graph) */
#define IMX_EP_ALL_TO_ALL 2  /* dispatch / return of fp16 rows by grouped ncclSend / ncclRecv; one host
                                synchronisation per call (the exchange's split sizes); results are bit-identical to
                                imx_moe_forward on one GPU; needs a format/shape the tensor-core kernels take */

typedef struct imx_ep_info {
    int want_timing;                     /* IN: non-zero = all-to-all: record and report phase_ms (synchronises) */
    int schedule;                        /* the schedule that ran                          */
    long long rows_received;             /* all-to-all: rows this rank's experts processed */
    unsigned long long bytes_sent;       /* bytes this rank put on the wire in the call    */
    unsigned long long bytes_received;
    float phase_ms[5];                   /* all-to-all with want_timing: local route/sort/pack, dispatch (count
                                            exchange, host round trip, rows), experts, return, combine */
} imx_ep_info;

/* An NCCL unique id (rank 0 makes one and hands it to the others by whatever means the host has). */
IMX_API int imx_ep_unique_id(void* id128);
/* Collective: builds this rank's context and its own communicator from the id.  cfg describes the whole
 * block (num_experts = E). */
IMX_API int imx_ep_create(const imx_moe_config* cfg, const void* unique_id, int rank, int world, imx_ep_ctx** ctx);
/* The same on a communicator the host already has (an ncclComm_t); it is borrowed, not destroyed. */
IMX_API int imx_ep_create_from_comm(const imx_moe_config* cfg, void* nccl_comm, int rank, int world, imx_ep_ctx** ctx);
/* The context's ncclComm_t (to build further contexts on it with imx_ep_create_from_comm). */
IMX_API void* imx_ep_comm(const imx_ep_ctx* ctx);
/* Frees the context; a communicator the context created itself is destroyed with it: first release every
 * captured CUDA graph that holds its collectives (NCCL can block in its destructor otherwise). */
IMX_API int imx_ep_destroy(imx_ep_ctx* ctx);
/* Scratch bytes for n_local tokens per rank (all-to-all: sized for every assignment of every rank landing here). */
IMX_API int imx_ep_workspace_bytes(const imx_ep_ctx* ctx, int n_local, int schedule, size_t* bytes);
/* y[n_local, H] = MoE(x[n_local, H]) with the experts spread over the ranks.  Collective: every rank calls it
 * with the same n_local and schedule.  workspace: zero-filled once, 256-byte aligned; imx_moe_status() reads its
 * status word.  info and trace may be NULL; trace (all-to-all schedule only) receives the local tokens' routing and
 * their dispatch permutation over the global expert ids, as imx_moe_forward would report them. */
IMX_API int imx_ep_forward(imx_ep_ctx* ctx, const imx_moe_weights* local_weights, const void* x, int n_local, void* y,
                   void* workspace, size_t workspace_bytes, void* stream, int schedule, imx_ep_info* info,
                   const imx_moe_trace* trace);

/* ── the reference's quantized-op surface, mlx/src/ops.rs:630-727 ──────── */

/* out[rows, in] = dequantize(w) (ops.rs:653-686 -> mlx_dequantize).
 * out_dtype: 0 = bf16, 1 = fp32, 2 = fp16. */
IMX_API int imx_dequantize(const imx_qtensor* w, int rows, int in, int group_size, int bits, int mode,
                   int out_dtype, void* out, void* stream);

/* y[m, n_out] = x[m, in] @ dequantize(w[n_out, in])^T when transpose != 0
 * (ops.rs:695-727 -> mlx_quantized_matmul; every layer on the path calls it
 * with transpose = true, mlx/src/nn/linear.rs:51-63); with transpose == 0,
 * y[m, in] = x[m, n_out] @ dequantize(w[n_out, in]).  x, y bf16. */
IMX_API int imx_quantized_matmul(const void* x, int m, const imx_qtensor* w, int n_out, int in,
                         int transpose, int group_size, int bits, int mode, void* y,
                         void* stream);

/* The same product (transpose != 0 form) on the expert kernels: the second expert product is this
 * contraction, so the call runs that kernel alone as a one-expert problem -- the tensor-map decode
 * kernel for few rows, the tcgen05 kernel from 32 rows up -- and falls back to the kernel above for
 * shapes neither takes.  `QuantizedLinear::forward_with_stream` (mlx/src/nn/linear.rs:51-63) with
 * caller-provided scratch (zero-filled once, 256-byte aligned). */
IMX_API int imx_quantized_matmul_scratch_bytes(int m, int n_out, int in, int group_size, int bits, int mode,
                                       size_t* bytes);
IMX_API int imx_quantized_matmul_ws(const void* x, int m, const imx_qtensor* w, int n_out, int in, int group_size,
                            int bits, int mode, void* y, void* scratch, size_t scratch_bytes, void* stream);

/* y[m, hidden] = down( silu(gate(x)) * up(x) ) for ONE expert over all m rows, bf16 in and out:
 * `Expert::forward_with_stream` (mlx/src/nn/moe.rs:26-32) and `MLP::forward_with_stream`
 * (mlx/src/nn/mlp.rs:27-33).  gate_up: [2*intermediate, hidden..] with the gate rows first (one expert of
 * the fused checkpoint tensor, or gate_proj and up_proj stacked); down: [hidden, intermediate..].
 * cfg: hidden, intermediate and the format are read. */
IMX_API int imx_expert_scratch_bytes(const imx_moe_config* cfg, int m, size_t* bytes);
IMX_API int imx_expert_forward(const imx_moe_config* cfg, const imx_qtensor* gate_up, const imx_qtensor* down,
                       const void* x, int m, void* y, void* scratch, size_t scratch_bytes, void* stream);

/* y[m, n_out] = x[m, in] @ w[n_out, in]^T (+ bias[n_out]), all bf16, fp32 accumulation:
 * dense `Linear::forward_with_stream` (mlx/src/nn/linear.rs:170-177); bias may be NULL. */
IMX_API int imx_linear(const void* x, int m, int in, const void* w, int n_out, const void* bias, void* y,
               void* stream);

/* Quantize w[rows, in] (fp32) into packed values, scales and biases
 * (absent from the reference's wrappers, which only consume checkpoints that
 * MLX's `quantize` produced; provided to complete the op surface).  For
 * nvfp4, global_scale is an INPUT (the tensor scale to quantize against). */
IMX_API int imx_quantize(const float* w, int rows, int in, int group_size, int bits, int mode,
                 float global_scale, void* w_packed, void* scales, void* biases, void* stream);

/* gather_qmm: y[j, :] = x[lhs_index[j], :] @ dequantize(w[rhs_index[j]])^T for
 * j < n_rows (bf16 in/out); the per-row form of the grouped expert product
 * the reference spells as take_axis + quantized_matmul per expert
 * (moe.rs:124-130). */
IMX_API int imx_gather_qmm(const void* x, const int32_t* lhs_index, const imx_qtensor* w,
                   const int32_t* rhs_index, int n_rows, int n_out, int in, int group_size,
                   int bits, int mode, void* y, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* IRONMLX_B200_H */
