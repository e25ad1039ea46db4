"""Shared helpers for the tests: build checker-side parameters from a seeded
workload (quantized with the CPU checker's quantizer, so that the CUDA path
and the checker consume byte-identical packed tensors)."""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from ironmlx_b200.workloads import MoEConfig, Workload  # noqa: E402
from oracle import formats as F  # noqa: E402
from oracle import moe as O  # noqa: E402


def quantize_stack(blocks, cfg: MoEConfig) -> O.QLinear:
    """Quantize a list of [out, in] fp32 matrices and stack them on a new axis 0."""
    ws, ss, bs = [], [], []
    gscale = None
    if cfg.mode == "nvfp4":
        # one fp32 scale for the whole tensor: derive it from all blocks together
        amax = max(float(np.abs(b).max()) for b in blocks)
        gscale = np.float32(max(amax, 1e-30) / (F.E2M1_MAX * F.E4M3_MAX))
    for blk in blocks:
        if cfg.mode == "nvfp4":
            p, s = _nvfp4_with_scale(blk, gscale)
            b = None
        else:
            p, s, b, _ = F.quantize(blk, cfg.group_size, cfg.bits, cfg.mode)
        ws.append(p)
        ss.append(s)
        bs.append(b)
    w = np.stack(ws)
    s = np.stack(ss)
    b = None if bs[0] is None else np.stack(bs)
    return O.QLinear(w, s, b, cfg.group_size, cfg.bits, cfg.mode, None if gscale is None else float(gscale))


def _nvfp4_with_scale(blk, t):
    import ml_dtypes
    g = blk.reshape(blk.shape[0], -1, 16)
    amax = np.abs(g).max(-1)
    s8 = np.clip(amax / F.E2M1_MAX / t, 0, F.E4M3_MAX).astype(np.float32).astype(ml_dtypes.float8_e4m3fn)
    sf = s8.astype(np.float32) * t
    sf = np.where(sf == 0, np.float32(1), sf)
    v = np.clip(g / sf[..., None], -F.E2M1_MAX, F.E2M1_MAX).astype(np.float32)
    nib = v.astype(ml_dtypes.float4_e2m1fn).view(np.uint8).reshape(blk.shape) & 0xF
    return F.pack_bits(nib, 4), s8.view(np.uint8)


def squeeze0(q: O.QLinear) -> O.QLinear:
    return O.QLinear(q.w[0], q.scales[0], None if q.biases is None else q.biases[0],
                     q.group_size, q.bits, q.mode, q.global_scale)


def make_params(cfg: MoEConfig):
    """-> (x fp32 [N,H] with bf16 values, oracle.moe.MoEParams)."""
    wl = Workload(cfg)
    x = wl.activations()
    gate_up = quantize_stack([wl.expert_gate_up(e) for e in range(cfg.num_experts)], cfg)
    down = quantize_stack([wl.expert_down(e) for e in range(cfg.num_experts)], cfg)
    p = O.MoEParams(
        router_w=wl.router_weight().astype(F.bf16),
        gate_up=gate_up,
        down=down,
        num_experts_per_tok=cfg.top_k,
        norm_topk_prob=cfg.norm_topk_prob,
        router_logit_bias=wl.router_logit_bias(),
    )
    if cfg.shared_intermediate:
        p.shared_gate_proj = squeeze0(quantize_stack([wl.shared("gate_proj")], cfg))
        p.shared_up_proj = squeeze0(quantize_stack([wl.shared("up_proj")], cfg))
        p.shared_down_proj = squeeze0(quantize_stack([wl.shared("down_proj")], cfg))
        p.shared_expert_gate_w = wl.shared_gate_weight().astype(F.bf16)
    return x, p


TINY = MoEConfig("tiny", tokens=5, hidden=128, num_experts=4, top_k=2, intermediate=128,
                 shared_intermediate=128, seed=3)
SMALL = MoEConfig("small", tokens=48, hidden=256, num_experts=8, top_k=3, intermediate=128,
                  shared_intermediate=128, seed=4)
