"""Builds a device-resident `MoEMLP` from a seeded synthetic workload: fp32
tensors from `workloads.Workload`, quantized on the GPU with the library's own
`quantize` op (expert by expert, so host memory stays bounded)."""
from __future__ import annotations

import numpy as np
import torch

from . import nn, ops
from .workloads import MoEConfig, Workload


def _bf16(a: np.ndarray, device) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).to(device).to(torch.bfloat16)


def nvfp4_tensor_scale(amax: float) -> float:
    return max(float(amax), 1e-30) / (6.0 * 448.0)


def _quantize_stack(blocks_fn, count: int, cfg: MoEConfig, device, gscale=None) -> nn.QuantizedLinear:
    """gscale: nvfp4 tensor scale to quantize against (default: derived from these blocks)."""
    ws, ss, bs = [], [], []
    if cfg.mode == "nvfp4" and gscale is None:
        gscale = nvfp4_tensor_scale(max(float(np.abs(blocks_fn(e)).max()) for e in range(count)))
    for e in range(count):
        w = torch.from_numpy(blocks_fn(e)).to(device)
        out = ops.quantize(w, cfg.group_size, cfg.bits, cfg.mode, global_scale=gscale)
        ws.append(out[0])
        ss.append(out[1])
        bs.append(out[2])
    w = torch.stack(ws)
    s = torch.stack(ss)
    b = None if bs[0] is None else torch.stack(bs)
    return nn.QuantizedLinear(w, s, b, cfg.group_size, cfg.bits, cfg.mode, gscale)


def _single(q: nn.QuantizedLinear) -> nn.QuantizedLinear:
    return nn.QuantizedLinear(q.weight[0], q.scales[0], None if q.biases is None else q.biases[0],
                              q.group_size, q.bits, q.mode, q.global_scale)


def build_moe(cfg: MoEConfig, device="cuda", path: str = "auto") -> nn.MoEMLP:
    """The whole block of a configuration on one device (one rank's share of it: ironmlx_b200.ep.build_local)."""
    wl = Workload(cfg)
    gate_up = _quantize_stack(lambda e: wl.expert_gate_up(e), cfg.num_experts, cfg, device)
    down = _quantize_stack(lambda e: wl.expert_down(e), cfg.num_experts, cfg, device)
    shared = shared_gate = None
    if cfg.shared_intermediate:
        shared = nn.MLP(*(_single(_quantize_stack(lambda e, n=n: wl.shared(n), 1, cfg, device))
                          for n in ("gate_proj", "up_proj", "down_proj")))
        shared_gate = nn.Linear(_bf16(wl.shared_gate_weight(), device))
    bias = wl.router_logit_bias()
    router = nn.Linear(_bf16(wl.router_weight(), device))
    return nn.MoEMLP(router, nn.FusedExperts(gate_up, down), shared, shared_gate, cfg.top_k, cfg.norm_topk_prob,
                     None if bias is None else torch.from_numpy(bias).to(device), path)
