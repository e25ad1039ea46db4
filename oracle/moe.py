"""The MoE block of mlx/src/nn/moe.rs:55-183, restated stage by stage in numpy.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py; parity unpinned).

Stages and the reference lines they follow:

  route()          moe.rs:67-82   router matmul, softmax, descending top-k,
                                  renormalised top-k weights
  bucket()         moe.rs:93-104  per-expert (token, flat index) lists built
                                  token-major / slot-minor = a stable counting
                                  sort of the N*k assignments by expert
  expert_forward() moe.rs:26-32   down(silu(gate(x)) * up(x)), each product a
                                  `quantized_matmul(transpose=true)`
                                  (linear.rs:51-63); silu = x*sigmoid(x)
                                  (activations.rs:7-10)
  combine          moe.rs:147-170 per token, weighted sum of its expert rows
                                  in the order the expert loop produced them
                                  (ascending expert index)
  shared expert    moe.rs:173-181 MLP(x) * sigmoid(x @ w_sg^T), added

Deliberate deviations from the literal reference, each a named switch:

  * scores are paired with the expert that produced them.  The reference
    takes indices from `argsort(-p)[:, :k]` and values from a separate
    `topk` call and pairs them slot by slot (moe.rs:71-74,141), which is only
    right if `topk` returns descending order.
  * scores are fp32 (the reference reads the score buffer back as f32 without
    a cast, mlx/src/array.rs:143-151) and the combine accumulates in fp32.
  * the shared expert is optional (the reference struct has no Option,
    moe.rs:44-47; "no shared expert" equals zero shared weights).

`bf16_boundaries=True` additionally rounds to bfloat16 wherever the reference
materialises an MLX array in the activation type (every matmul output, silu,
multiply, the weighted rows, the final sum), to show how far the reference's
own bf16 pipeline sits from the fp32-accumulated result that is graded.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np

from . import formats as F


@dataclass
class QLinear:
    """One `QuantizedLinear` (mlx/src/nn/linear.rs:13-49): y = x @ dequant(w)^T."""
    w: np.ndarray                 # uint32 [out, in*bits/32]
    scales: np.ndarray            # bf16 [out, in/g]   (uint8 for mxfp8/nvfp4)
    biases: Optional[np.ndarray]  # bf16 [out, in/g]   (None for mxfp8/nvfp4)
    group_size: int = 64
    bits: int = 4
    mode: str = "affine"
    global_scale: Optional[float] = None

    def dense(self) -> np.ndarray:
        return F.dequantize(self.w, self.scales, self.biases, self.group_size, self.bits,
                            self.mode, self.global_scale)


@dataclass
class MoEParams:
    """Weights of one `MoEMLP` (moe.rs:39-52) in the fused checkpoint layout
    that `build_moe_experts` slices (mlx/src/model/qwen35.rs:581-590):
    gate_up [E, 2I, .] with gate rows first, down [E, H, .]."""
    router_w: np.ndarray                    # bf16 [E, H]
    gate_up: QLinear                        # w [E, 2I, H*b/32]
    down: QLinear                           # w [E, H, I*b/32]
    num_experts_per_tok: int
    norm_topk_prob: bool = True
    shared_gate_proj: Optional[QLinear] = None   # [Is, H]
    shared_up_proj: Optional[QLinear] = None     # [Is, H]
    shared_down_proj: Optional[QLinear] = None   # [H, Is]
    shared_expert_gate_w: Optional[np.ndarray] = None  # bf16 [1, H]
    router_logit_bias: Optional[np.ndarray] = None     # fp32 [E]; synthetic skew only

    @property
    def num_experts(self) -> int:
        return self.router_w.shape[0]


def _f32(a) -> np.ndarray:
    return np.asarray(a).astype(np.float32)


def sigmoid(x):
    x = np.asarray(x, dtype=np.float32)
    return (1.0 / (1.0 + np.exp(-x.astype(np.float64)))).astype(np.float32)


def silu(x):
    """x * sigmoid(x)  (mlx/src/nn/activations.rs:7-10)."""
    return (np.asarray(x, dtype=np.float32) * sigmoid(x)).astype(np.float32)


def router_logits(x, router_w, logit_bias=None) -> np.ndarray:
    """x[N,H] @ W_r[E,H]^T (moe.rs:67, linear.rs:170-177), exact products of
    bf16 inputs accumulated in float64 and rounded once to fp32."""
    z = (_f32(x).astype(np.float64) @ _f32(router_w).astype(np.float64).T)
    if logit_bias is not None:
        z = z + np.asarray(logit_bias, dtype=np.float64)[None, :]
    return z.astype(np.float32)


def softmax_rows(z) -> np.ndarray:
    """Row softmax (moe.rs:68) in fp32 semantics: exp(z - max) / sum."""
    z = np.asarray(z, dtype=np.float32)
    m = z.max(-1, keepdims=True)
    e = np.exp((z - m).astype(np.float64))
    return (e / e.sum(-1, keepdims=True)).astype(np.float32)


def route(x, router_w, k: int, norm_topk_prob: bool = True, logit_bias=None, bf16_logits: bool = False):
    """-> (top_idx int32 [N,k] descending by probability, lower expert index
    first among exact ties; top_w fp32 [N,k]; probs fp32 [N,E]).

    bf16_logits=True follows the reference's dtypes literally: its gate `Linear`
    returns the logits in the activation dtype (bf16, linear.rs:170-177) and
    softmax / argsort / topk run on bf16 arrays (moe.rs:67-74), so logits and
    probabilities are rounded to bf16 before the selection.  The default keeps
    both in fp32, which is what the kernels do; `routing_changes` counts the rows
    where the two differ."""
    z = router_logits(x, router_w, logit_bias)
    if bf16_logits:
        z = _r(z, True)
    probs = softmax_rows(z)
    if bf16_logits:
        probs = _r(probs, True)
    order = np.argsort(-probs, axis=-1, kind="stable")        # moe.rs:71-72
    top_idx = order[:, :k].astype(np.int32)                    # moe.rs:73
    top_w = np.take_along_axis(probs, top_idx, axis=-1)        # moe.rs:74 (paired by expert)
    if norm_topk_prob:                                         # moe.rs:77-82
        top_w = (top_w.astype(np.float64) / top_w.astype(np.float64).sum(-1, keepdims=True))
    return top_idx, top_w.astype(np.float32), probs


def routing_changes(x, router_w, k: int, logit_bias=None) -> dict:
    """How much the bf16 rounding of logits and probabilities (the reference's
    dtypes) changes the routing against fp32: rows whose expert SET differs,
    rows whose ordered list differs, and assignments that go to another expert."""
    a, _, _ = route(x, router_w, k, True, logit_bias, bf16_logits=False)
    b, _, _ = route(x, router_w, k, True, logit_bias, bf16_logits=True)
    set_rows = sum(1 for i in range(a.shape[0]) if set(a[i].tolist()) != set(b[i].tolist()))
    moved = sum(len(set(a[i].tolist()) - set(b[i].tolist())) for i in range(a.shape[0]))
    return {"rows": int(a.shape[0]), "rows_set_differs": int(set_rows),
            "rows_order_differs": int((a != b).any(-1).sum()), "assignments_moved": int(moved)}


def routing_margin(probs: np.ndarray, k: int) -> np.ndarray:
    """Per row, the smallest relative gap between consecutive entries of the
    descending top-(k+1) probabilities.  Rows whose margin is far above fp32
    rounding noise have one and only one correct (ordered) expert list."""
    srt = -np.sort(-probs.astype(np.float64), axis=-1)[:, : k + 1]
    if srt.shape[1] < 2:
        return np.full(probs.shape[0], np.inf)
    gaps = (srt[:, :-1] - srt[:, 1:]) / srt[:, :-1]
    return gaps.min(-1)


def bucket(top_idx: np.ndarray, num_experts: int):
    """The host bucketing loop of moe.rs:93-104 as arrays.

    -> counts int32 [E]; offsets int32 [E+1] (exclusive scan); perm int32
    [N*k]: flat assignment indices t*k+s grouped by expert, token-major
    inside each expert; inv_perm int32 [N*k]: position of flat index in perm.
    """
    n, k = top_idx.shape
    lists = [[] for _ in range(num_experts)]
    flat = top_idx.reshape(-1)
    for f in range(n * k):
        e = int(flat[f])
        if 0 <= e < num_experts:            # moe.rs:100
            lists[e].append(f)
    counts = np.array([len(l) for l in lists], dtype=np.int32)
    offsets = np.zeros(num_experts + 1, dtype=np.int32)
    np.cumsum(counts, out=offsets[1:])
    perm = np.array([f for l in lists for f in l], dtype=np.int32)
    inv = np.full(n * k, -1, dtype=np.int32)           # dropped assignments keep -1
    inv[perm] = np.arange(perm.size, dtype=np.int32)
    return counts, offsets, perm, inv


def bucket_fast(top_idx: np.ndarray, num_experts: int):
    """Same result as `bucket` through a stable argsort (for large N)."""
    n, k = top_idx.shape
    flat = top_idx.reshape(-1).astype(np.int64)
    valid = (flat >= 0) & (flat < num_experts)
    key = np.where(valid, flat, num_experts)
    order = np.argsort(key, kind="stable")
    perm = order[: int(valid.sum())].astype(np.int32)
    counts = np.bincount(flat[valid], minlength=num_experts).astype(np.int32)
    offsets = np.zeros(num_experts + 1, dtype=np.int32)
    np.cumsum(counts, out=offsets[1:])
    inv = np.full(n * k, -1, dtype=np.int32)
    inv[perm] = np.arange(perm.size, dtype=np.int32)
    return counts, offsets, perm, inv


def _r(a, on: bool):
    return F.to_bf16(a) if on else np.asarray(a, dtype=np.float32)


def swiglu_mlp(x, wg, wu, wd, bf16_boundaries=False) -> np.ndarray:
    """down(silu(gate(x)) * up(x)) with dense fp32 weight matrices
    (moe.rs:26-32 / mlp.rs:27-33); float64 accumulation, fp32 results."""
    x64 = _f32(x).astype(np.float64)
    g = _r((x64 @ wg.astype(np.float64).T).astype(np.float32), bf16_boundaries)
    u = _r((x64 @ wu.astype(np.float64).T).astype(np.float32), bf16_boundaries)
    if bf16_boundaries:
        a = _r(_r(silu(g), True) * u, True)       # sigmoid, multiply, multiply: three arrays
    else:
        a = silu(g) * u
    d = (a.astype(np.float64) @ wd.astype(np.float64).T).astype(np.float32)
    return _r(d, bf16_boundaries)


def expert_weights(p: MoEParams, e: int):
    """Dense fp32 (gate, up, down) matrices of expert e: the slices
    `build_moe_experts` takes (qwen35.rs:661-776), dequantized."""
    gu, dn = p.gate_up, p.down
    two_i = gu.w.shape[1]
    half = two_i // 2
    sl = lambda q, rows: F.dequantize(q.w[e][rows], q.scales[e][rows],
                                      None if q.biases is None else q.biases[e][rows],
                                      q.group_size, q.bits, q.mode, q.global_scale)
    return sl(gu, slice(0, half)), sl(gu, slice(half, two_i)), sl(dn, slice(None))


@dataclass
class MoETrace:
    """Everything the parity tests compare, stage by stage."""
    top_idx: np.ndarray
    top_w: np.ndarray
    probs: np.ndarray
    counts: np.ndarray
    offsets: np.ndarray
    perm: np.ndarray
    inv_perm: np.ndarray
    expert_rows: np.ndarray      # fp32 [N*k, H], row j = unweighted output for perm[j]
    routed: np.ndarray           # fp32 [N, H]
    shared: Optional[np.ndarray] # fp32 [N, H] (already gated) or None
    shared_gate: Optional[np.ndarray]  # fp32 [N]
    y: np.ndarray                # fp32 [N, H]
    extras: dict = field(default_factory=dict)


def moe_forward(x, p: MoEParams, bf16_boundaries: bool = False, fast_bucket: bool = False) -> MoETrace:
    """`MoEMLP::forward_with_stream` (moe.rs:55-183) on x[N,H] (bf16 values)."""
    x = _f32(x)
    n, h = x.shape
    k = p.num_experts_per_tok
    e_n = p.num_experts
    top_idx, top_w, probs = route(x, p.router_w, k, p.norm_topk_prob, p.router_logit_bias)
    counts, offsets, perm, inv = (bucket_fast if fast_bucket else bucket)(top_idx, e_n)

    rows = np.zeros((n * k, h), dtype=np.float32)
    for e in range(e_n):                                       # moe.rs:117
        lo, hi = int(offsets[e]), int(offsets[e + 1])
        if lo == hi:
            continue                                           # moe.rs:118-120
        tok = perm[lo:hi] // k                                 # moe.rs:125-127 take_axis
        wg, wu, wd = expert_weights(p, e)
        rows[lo:hi] = swiglu_mlp(x[tok], wg, wu, wd, bf16_boundaries)   # moe.rs:130

    # moe.rs:147-165: per token, rows arrive in ascending expert order
    routed = np.zeros((n, h), dtype=np.float64)
    flat_w = top_w.reshape(-1)
    for j in range(n * k):                                     # perm order == expert-major
        f = int(perm[j])
        t = f // k
        term = rows[j].astype(np.float64) * np.float64(flat_w[f])
        if bf16_boundaries:
            term = F.to_bf16(term).astype(np.float64)
            routed[t] = F.to_bf16(routed[t] + term)
        else:
            routed[t] += term
    routed32 = routed.astype(np.float32)

    shared = gate = None
    y = routed32
    if p.shared_gate_proj is not None:
        so = swiglu_mlp(x, p.shared_gate_proj.dense(), p.shared_up_proj.dense(),
                        p.shared_down_proj.dense(), bf16_boundaries)           # moe.rs:173
        gl = (x.astype(np.float64) @ _f32(p.shared_expert_gate_w).astype(np.float64).T).astype(np.float32)
        gate = sigmoid(_r(gl, bf16_boundaries))[:, 0]                          # moe.rs:174-177
        shared = _r(so * gate[:, None], bf16_boundaries)                       # moe.rs:178
        y = _r(routed32.astype(np.float64) + shared, bf16_boundaries)          # moe.rs:181
    return MoETrace(top_idx, top_w, probs, counts, offsets, perm, inv, rows, routed32, shared,
                    gate, np.asarray(y, dtype=np.float32))


def rel_l2(a, b) -> float:
    """||a-b||_2 / ||b||_2 over all elements, in float64."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    den = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / den) if den > 0 else float(np.linalg.norm(a - b))


def rms_norm(x: np.ndarray, weight: Optional[np.ndarray], eps: float) -> np.ndarray:
    """`fast::rms_norm` (mlx/src/fast.rs:37-49, called by RMSNorm, mlx/src/nn/norm.rs:21-24), as MLX's
    kernels compute it for 16-bit arrays: the sum of squares and the factor in fp32, the normalised
    value rounded to the array type, then multiplied by the weight and rounded again.
    x: bf16-representable [N, H]; returns bf16-representable fp32."""
    xf = np.asarray(x, np.float32)
    inv = (1.0 / np.sqrt((xf.astype(np.float64) ** 2).mean(axis=-1, keepdims=True) + eps)).astype(np.float32)
    t = (xf * inv).astype(F.bf16).astype(np.float32)
    if weight is None:
        return t
    return (np.asarray(weight, np.float32) * t).astype(F.bf16).astype(np.float32)


def decoder_layer_tail(h: np.ndarray, ln_weight: Optional[np.ndarray], eps: float, p: MoEParams):
    """The MoE half of a decoder layer (mlx/src/model/qwen35.rs:271-276):
    `normed = post_attention_layernorm(h); mlp_out = mlp(normed); h + mlp_out`, every array bf16 as the
    reference materialises it.  Returns (y fp32 holding bf16 values, the block's trace)."""
    normed = rms_norm(h, ln_weight, eps)
    tr = moe_forward(normed, p)
    mlp_out = tr.y.astype(F.bf16).astype(np.float32)
    y = (np.asarray(h, np.float32) + mlp_out).astype(F.bf16).astype(np.float32)
    return y, tr, normed
