"""Writes tests/golden/checkpoint/: a tiny synthetic checkpoint in the layout of an mlx-community Qwen3.5-MoE
4-bit checkpoint (config.json + model.safetensors with the key names and fused shapes the reference's builder
reads, mlx/src/model/qwen35.rs:498-522,592-779), quantized with the CPU checker, together with the checker's
output for a seeded input.  No real checkpoint is available offline; this fixture pins the loader's key handling,
dtypes and shapes, not MLX's bit order.

    python tests/golden/make_checkpoint.py
"""
import json
import os
import sys

import numpy as np
import torch
from safetensors.torch import save_file

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
for p in (ROOT, os.path.join(ROOT, "tests")):
    sys.path.insert(0, p)

from ironmlx_b200.workloads import MoEConfig  # noqa: E402
from oracle import formats as F  # noqa: E402
from oracle import moe as O  # noqa: E402
from util import make_params  # noqa: E402

CFG = MoEConfig("ckpt", tokens=12, hidden=256, num_experts=4, top_k=2, intermediate=128, shared_intermediate=128, seed=77)
LAYER = 3


def bf16_t(a):
    return torch.from_numpy(np.ascontiguousarray(np.asarray(a, np.float32).astype(F.bf16)).view(np.uint16).copy()).view(torch.bfloat16)


def u32_t(a):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int32).copy()).view(torch.uint32)


def main():
    out = os.path.join(HERE, "checkpoint")
    os.makedirs(out, exist_ok=True)
    x, p = make_params(CFG)
    pre = f"language_model.model.layers.{LAYER}.mlp"
    t = {f"{pre}.gate.weight": bf16_t(p.router_w), f"{pre}.shared_expert_gate.weight": bf16_t(p.shared_expert_gate_w)}
    for name, q in (("experts.gate_up_proj", p.gate_up), ("experts.down_proj", p.down),
                    ("shared_expert.gate_proj", p.shared_gate_proj), ("shared_expert.up_proj", p.shared_up_proj),
                    ("shared_expert.down_proj", p.shared_down_proj)):
        t[f"{pre}.{name}.weight"] = u32_t(q.w)
        t[f"{pre}.{name}.scales"] = bf16_t(q.scales)
        t[f"{pre}.{name}.biases"] = bf16_t(q.biases)
    save_file(t, os.path.join(out, "model.safetensors"), metadata={"format": "mlx"})
    cfg = {"model_type": "qwen3_5_moe",
           "text_config": {"hidden_size": CFG.hidden, "num_experts": CFG.num_experts, "num_experts_per_tok": CFG.top_k,
                           "moe_intermediate_size": CFG.intermediate, "shared_expert_intermediate_size": CFG.shared_intermediate,
                           "norm_topk_prob": True},
           "quantization": {"group_size": CFG.group_size, "bits": CFG.bits, "mode": "affine"}}
    with open(os.path.join(out, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    ref = O.moe_forward(x, p)
    np.savez(os.path.join(out, "expected.npz"), x=x, y=ref.y, top_idx=ref.top_idx, perm=ref.perm, layer=LAYER)
    print("wrote", out, {k: tuple(v.shape) for k, v in t.items()})


if __name__ == "__main__":
    main()
