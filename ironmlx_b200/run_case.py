"""Runs a few passes of the MoE block on a (possibly reduced) configuration and
exits: the small, self-terminating command that profiler captures wrap.

    python -m ironmlx_b200.run_case --config c2 --experts 96 --steps 3 [--path decode]
"""
from __future__ import annotations

import argparse

import torch

from . import synthetic
from .workloads import CONFIGS, Workload


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="c2")
    ap.add_argument("--experts", type=int, default=0, help="keep only this many experts (0: all)")
    ap.add_argument("--tokens", type=int, default=0)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--path", default="auto")
    a = ap.parse_args()
    cfg = CONFIGS[a.config]
    if a.experts:
        cfg = cfg.with_(num_experts=a.experts)
    if a.tokens:
        cfg = cfg.with_(tokens=a.tokens)
    dev = torch.device("cuda:0")
    moe = synthetic.build_moe(cfg, dev, path=a.path)
    x = torch.from_numpy(Workload(cfg).activations()).to(dev).to(torch.bfloat16)
    for _ in range(a.steps):
        y = moe.forward_with_stream(x)
    torch.cuda.synchronize()
    moe.check_status()
    print(f"{cfg.name}: {a.steps} passes, experts={cfg.num_experts}, tokens={cfg.tokens}, "
          f"|y|={float(y.float().abs().mean()):.4f}")


if __name__ == "__main__":
    main()
