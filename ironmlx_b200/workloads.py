"""Seeded synthetic workloads for the MoE block (shapes of the five benchmark
configurations; no public dataset is involved).

Every tensor is drawn from its own numpy Philox stream keyed by
(seed, tensor name, block index), so a tensor's values do not depend on the
order in which tensors are generated, and expert e's weights can be produced
alone.  Values are fp32; quantizing them is the caller's business (the CUDA
`quantize` op in the benchmark, the CPU checker in the parity tests).

Distributions: activations ~N(0,1) rounded to bf16; router, shared-gate and
expert weights ~N(0,0.02).  `zipf_s` adds a per-expert router-logit bias so
that expert popularity follows a Zipf law over a seeded permutation.
"""
from __future__ import annotations

import zlib
from dataclasses import dataclass, replace
from typing import Optional

import numpy as np


@dataclass(frozen=True)
class MoEConfig:
    name: str
    tokens: int
    hidden: int
    num_experts: int
    top_k: int
    intermediate: int
    shared_intermediate: int = 0          # 0: no shared expert
    norm_topk_prob: bool = True
    mode: str = "affine"
    bits: int = 4
    group_size: int = 64
    seed: int = 0
    zipf_s: float = 0.0                   # 0: unbiased router
    zipf_hot_share: float = 0.08          # share of assignments of the hottest expert

    def with_(self, **kw) -> "MoEConfig":
        return replace(self, **kw)

    @property
    def assignments(self) -> int:
        return self.tokens * self.top_k


_QWEN = dict(hidden=2048, num_experts=256, top_k=8, intermediate=512, shared_intermediate=512)

CONFIGS = {
    # 32 tokens, 16 experts, top-4, no shared expert, seed 0 (CPU-runnable case)
    "c1": MoEConfig("c1", tokens=32, hidden=512, num_experts=16, top_k=4, intermediate=256, seed=0),
    # Qwen3.5-MoE-shaped decode step
    "c2": MoEConfig("c2", tokens=64, seed=0, **_QWEN),
    # same layer in prefill
    "c3": MoEConfig("c3", tokens=8192, seed=1, **_QWEN),
    # alternative expert quantization, decode and prefill
    "c4-nvfp4-decode": MoEConfig("c4-nvfp4-decode", tokens=256, seed=1, mode="nvfp4", bits=4, group_size=16, **_QWEN),
    "c4-nvfp4-prefill": MoEConfig("c4-nvfp4-prefill", tokens=4096, seed=1, mode="nvfp4", bits=4, group_size=16, **_QWEN),
    "c4-mxfp8-decode": MoEConfig("c4-mxfp8-decode", tokens=256, seed=1, mode="mxfp8", bits=8, group_size=32, **_QWEN),
    "c4-mxfp8-prefill": MoEConfig("c4-mxfp8-prefill", tokens=4096, seed=1, mode="mxfp8", bits=8, group_size=32, **_QWEN),
    # skewed routing stress
    "c5": MoEConfig("c5", tokens=16384, seed=1, zipf_s=1.2, **_QWEN),
    "c5-2bit": MoEConfig("c5-2bit", tokens=16384, seed=1, zipf_s=1.2, bits=2, **_QWEN),
    "c5-8bit": MoEConfig("c5-8bit", tokens=16384, seed=1, zipf_s=1.2, bits=8, **_QWEN),
}


def _rng(seed: int, name: str, block: int = 0) -> np.random.Generator:
    key = (int(seed) & 0xFFFFFFFF) | ((zlib.crc32(name.encode()) & 0xFFFFFFFF) << 32)
    return np.random.Generator(np.random.Philox(key=np.array([key, int(block)], dtype=np.uint64)))


def normal(seed: int, name: str, shape, std: float = 1.0, block: int = 0) -> np.ndarray:
    a = _rng(seed, name, block).standard_normal(shape, dtype=np.float32)
    if std != 1.0:
        a *= np.float32(std)
    return a


def round_bf16(a: np.ndarray) -> np.ndarray:
    """fp32 -> nearest-even bfloat16, returned as fp32 values (pure integer math)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return r.view(np.float32)


def bf16_bits(a: np.ndarray) -> np.ndarray:
    """fp32 values that are exactly representable in bf16 -> their uint16 patterns."""
    return (np.ascontiguousarray(a, dtype=np.float32).view(np.uint32) >> np.uint32(16)).astype(np.uint16)


class Workload:
    """Lazily generated fp32 tensors of one configuration."""

    def __init__(self, cfg: MoEConfig):
        self.cfg = cfg

    def activations(self, tokens: Optional[int] = None, block: int = 0) -> np.ndarray:
        """[N, H] ~N(0,1), bf16-representable.  `block` selects an independent
        batch (another rank's tokens, another step)."""
        n = self.cfg.tokens if tokens is None else tokens
        return round_bf16(normal(self.cfg.seed, "x", (n, self.cfg.hidden), 1.0, block))

    def router_weight(self) -> np.ndarray:
        c = self.cfg
        return round_bf16(normal(c.seed, "router", (c.num_experts, c.hidden), 0.02))

    def shared_gate_weight(self) -> np.ndarray:
        c = self.cfg
        return round_bf16(normal(c.seed, "shared_expert_gate", (1, c.hidden), 0.02))

    def expert_gate_up(self, e: int) -> np.ndarray:
        """[2I, H]: gate rows first, then up rows (the fused checkpoint layout)."""
        c = self.cfg
        return round_bf16(normal(c.seed, "experts.gate_up_proj", (2 * c.intermediate, c.hidden), 0.02, e))

    def expert_down(self, e: int) -> np.ndarray:
        c = self.cfg
        return round_bf16(normal(c.seed, "experts.down_proj", (c.hidden, c.intermediate), 0.02, e))

    def shared(self, which: str) -> np.ndarray:
        """which in gate_proj / up_proj ([Is, H]) / down_proj ([H, Is])."""
        c = self.cfg
        shape = (c.hidden, c.shared_intermediate) if which == "down_proj" else (c.shared_intermediate, c.hidden)
        return round_bf16(normal(c.seed, "shared_expert." + which, shape, 0.02))

    def router_logit_bias(self) -> Optional[np.ndarray]:
        """Per-expert additive logit bias alpha*log(zipf weight) for skewed routing,
        alpha bisected on a fixed sample of tokens so that the hottest expert
        receives `zipf_hot_share` of the assignments; None when unbiased."""
        c = self.cfg
        if c.zipf_s <= 0:
            return None
        rng = _rng(c.seed, "zipf_perm")
        rank = rng.permutation(c.num_experts).astype(np.float64) + 1.0
        logw = -c.zipf_s * np.log(rank)
        logw -= logw.max()
        xs = self.activations(min(c.tokens, 2048)).astype(np.float64)
        z = xs @ self.router_weight().astype(np.float64).T

        def hot_share(alpha: float) -> float:
            top = np.argpartition(-(z + alpha * logw), c.top_k - 1, axis=-1)[:, : c.top_k]
            return np.bincount(top.reshape(-1), minlength=c.num_experts).max() / top.size

        lo, hi = 0.0, 8.0
        for _ in range(40):
            mid = 0.5 * (lo + hi)
            if hot_share(mid) < c.zipf_hot_share:
                lo = mid
            else:
                hi = mid
        return (0.5 * (lo + hi) * logw).astype(np.float32)


def algorithmic_bytes_decode(cfg: MoEConfig, touched_experts: int) -> int:
    """Bytes one decode pass must move: packed weights (+ scales/biases) of the
    experts actually selected and of the shared expert, the dense router and
    shared-gate weights, activations in and out.  Intermediates not counted."""
    c = cfg
    per_w = {"affine": c.bits / 8 + 4 / c.group_size, "mxfp8": 1 + 1 / 32, "nvfp4": 0.5 + 1 / 16}[c.mode]
    expert = 3 * c.intermediate * c.hidden * per_w
    shared = 3 * c.shared_intermediate * c.hidden * per_w
    dense = c.num_experts * c.hidden * 2 + (c.hidden * 2 if c.shared_intermediate else 0)
    act = 2 * c.tokens * c.hidden * 2
    return int(touched_experts * expert + shared + dense + act)


def algorithmic_flops(cfg: MoEConfig, tokens: Optional[int] = None) -> int:
    """Dense-equivalent flops of one pass: expert and shared SwiGLU products,
    router, shared gate.  No padding, no dequantization work."""
    c = cfg
    n = c.tokens if tokens is None else tokens
    f = 6 * n * c.top_k * c.hidden * c.intermediate + 2 * n * c.hidden * c.num_experts
    if c.shared_intermediate:
        f += 6 * n * c.hidden * c.shared_intermediate + 2 * n * c.hidden
    return int(f)
