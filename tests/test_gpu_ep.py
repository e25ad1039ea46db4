"""Expert parallelism on GPUs (NCCL): a world of 1 runs everywhere; the 2-rank
case runs when two devices are visible.  Results are compared with the
single-GPU block (same packed weights) and with the CPU checker."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ironmlx_b200 import ep, nn
from ironmlx_b200.workloads import MoEConfig, Workload
from oracle import moe as O
from gpu_util import bf16_to_np, moe_to_device, q_to_device, t_bf16
from util import make_params

pytestmark = pytest.mark.gpu
CFG = MoEConfig("ep-gpu", tokens=24, hidden=256, num_experts=8, top_k=3, intermediate=256,
                shared_intermediate=256, seed=23)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def local_from_params(p, dev, rank, world) -> ep.LocalExperts:
    moe = moe_to_device(p, dev)
    e_loc = p.num_experts // world
    sl = slice(rank * e_loc, (rank + 1) * e_loc)
    f = moe._fused
    cut = lambda q: nn.QuantizedLinear(q.weight[sl].contiguous(), q.scales[sl].contiguous(),
                                       None if q.biases is None else q.biases[sl].contiguous(),
                                       q.group_size, q.bits, q.mode, q.global_scale)
    gu, dn = ep.fuse_shared(moe.shared_expert)
    return ep.LocalExperts(moe.gate.weight, cut(f.gate_up), cut(f.down), gu, dn, moe.shared_expert_gate.weight,
                           moe.router_logit_bias)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        _, p = make_params(CFG)
        x = Workload(CFG).activations(block=rank)
        moe = ep.ExpertParallelMoE(ep.CudaStages(dev), local_from_params(p, dev, rank, world), CFG.num_experts,
                                   CFG.top_k, True, CFG.hidden, CFG.intermediate, CFG.shared_intermediate)
        y = yg = None
        for _ in range(2):
            y = moe.forward(t_bf16(x, dev), mode="a2a")
        perm = moe.last["perm"].cpu().numpy()
        for _ in range(2):
            yg = moe.forward(t_bf16(x, dev), mode="gathered")
        torch.cuda.synchronize()
        single = moe_to_device(p, dev).forward_with_stream(t_bf16(x, dev))
        ref = O.moe_forward(x, p)
        out[rank] = (max(O.rel_l2(bf16_to_np(y), ref.y), O.rel_l2(bf16_to_np(yg), ref.y)),
                     max(O.rel_l2(bf16_to_np(y), bf16_to_np(single)), O.rel_l2(bf16_to_np(yg), bf16_to_np(single))),
                     bool(np.array_equal(perm, ref.perm)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [1, 2])
def test_ep_matches_single_gpu_and_checker(cuda, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    out = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    for rank in range(world):
        err_ref, err_single, perm_ok = out[rank]
        assert perm_ok and err_ref <= 2e-3, (rank, err_ref)
        assert err_single <= 5e-4, (rank, err_single)        # same fp32 sums up to partition order, same bf16 rounding
