"""Moves checker-side parameters (numpy) onto the GPU as the package's layer
types, byte for byte, so both sides consume identical packed tensors."""
from __future__ import annotations

import numpy as np
import torch

from ironmlx_b200 import nn
from oracle import formats as F
from oracle import moe as O


def t_bf16(a, device) -> torch.Tensor:
    """numpy bf16 (ml_dtypes) or bf16-representable fp32 -> torch bf16 on device."""
    a = np.asarray(a)
    if a.dtype != F.bf16:
        a = a.astype(np.float32).astype(F.bf16)
    return torch.from_numpy(np.ascontiguousarray(a).view(np.uint16).copy()).view(torch.bfloat16).to(device)


def t_words(a, device) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int32).copy()).to(device)


def t_u8(a, device) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a).copy()).to(device)


def q_to_device(q: O.QLinear, device) -> nn.QuantizedLinear:
    scales = t_bf16(q.scales, device) if q.mode == "affine" else t_u8(q.scales, device)
    biases = None if q.biases is None else t_bf16(q.biases, device)
    return nn.QuantizedLinear(t_words(q.w, device), scales, biases, q.group_size, q.bits, q.mode, q.global_scale)


def moe_to_device(p: O.MoEParams, device, path="auto") -> nn.MoEMLP:
    shared = shared_gate = None
    if p.shared_gate_proj is not None:
        shared = nn.MLP(q_to_device(p.shared_gate_proj, device), q_to_device(p.shared_up_proj, device),
                        q_to_device(p.shared_down_proj, device))
        shared_gate = nn.Linear(t_bf16(p.shared_expert_gate_w, device))
    bias = None if p.router_logit_bias is None else torch.from_numpy(p.router_logit_bias).to(device)
    return nn.MoEMLP(nn.Linear(t_bf16(p.router_w, device)),
                     nn.FusedExperts(q_to_device(p.gate_up, device), q_to_device(p.down, device)),
                     shared, shared_gate, p.num_experts_per_tok, p.norm_topk_prob, bias, path)


def bf16_to_np(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def params_from_device(moe: nn.MoEMLP, top_k: int, norm: bool) -> O.MoEParams:
    """Checker-side parameters holding the very bytes a device-built block uses."""
    def q(ql):
        w = ql.weight.cpu().numpy().view(np.uint32)
        if ql.mode == "affine":
            s = ql.scales.view(torch.int16).cpu().numpy().view(F.bf16)
            b = ql.biases.view(torch.int16).cpu().numpy().view(F.bf16)
        else:
            s, b = ql.scales.cpu().numpy(), None
        return O.QLinear(w, s, b, ql.group_size, ql.bits, ql.mode, ql.global_scale)

    p = O.MoEParams(router_w=moe.gate.weight.float().cpu().numpy().astype(F.bf16),
                    gate_up=q(moe._fused.gate_up), down=q(moe._fused.down),
                    num_experts_per_tok=top_k, norm_topk_prob=norm)
    if moe.shared_expert is not None:
        p.shared_gate_proj = q(moe.shared_expert.gate_proj)
        p.shared_up_proj = q(moe.shared_expert.up_proj)
        p.shared_down_proj = q(moe.shared_expert.down_proj)
        p.shared_expert_gate_w = moe.shared_expert_gate.weight.float().cpu().numpy().astype(F.bf16)
    if moe.router_logit_bias is not None:
        p.router_logit_bias = moe.router_logit_bias.cpu().numpy()
    return p
