"""Expert-parallel bookkeeping on CPU ranks (gloo, world size 2): the exchange
protocol of ironmlx_b200.ep with the stage kernels replaced by the CPU checker,
compared with the single-process checker on every rank's tokens."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ironmlx_b200 import _lib, ep
from ironmlx_b200.workloads import MoEConfig, Workload
from oracle import formats as F
from oracle import moe as O
from util import make_params

CFG = MoEConfig("ep-cpu", tokens=11, hidden=128, num_experts=8, top_k=3, intermediate=128,
                shared_intermediate=128, seed=21)


class NumpyStages:
    """CPU stand-ins for the stage kernels (torch CPU tensors in and out)."""

    def route(self, x, router_w, logit_bias, k, norm, shared_gate_w):
        xf = x.float().numpy()
        idx, w, _ = O.route(xf, router_w, k, norm, logit_bias)
        sg = np.zeros(xf.shape[0], np.float32)
        if shared_gate_w is not None:
            sg = O.sigmoid((xf.astype(np.float64) @ np.asarray(shared_gate_w).astype(np.float32).astype(np.float64).T)
                           .astype(np.float32))[:, 0]
        return (torch.from_numpy(idx), torch.from_numpy(w), torch.from_numpy(sg),
                torch.from_numpy(xf.astype(np.float16)))

    def sort(self, ids, num_experts):
        c, o, p, i = O.bucket_fast(ids.numpy().reshape(-1, 1), num_experts)
        return tuple(torch.from_numpy(a) for a in (c, o, p, i))

    def gather_rows(self, src, index):
        return src.reshape(src.shape[0], -1)[index.long()].clone()

    def experts(self, cfg, gate_up, down, num_experts, x16, row_index, offsets, n_rows, row_scale, key=None):
        x = x16.float().numpy()
        off = offsets.numpy()
        out = np.zeros((n_rows, cfg.hidden), np.float32)
        p = O.MoEParams(router_w=None, gate_up=gate_up, down=down, num_experts_per_tok=1)
        for e in range(num_experts):
            lo, hi = int(off[e]), int(off[e + 1])
            if lo == hi:
                continue
            rows = np.arange(lo, hi) if row_index is None else row_index.numpy()[lo:hi]
            out[lo:hi] = O.swiglu_mlp(x[rows], *O.expert_weights(p, e))
        if row_scale is not None:
            out *= row_scale.numpy()[:, None]
        return torch.from_numpy(out)

    def combine_partial(self, rows, row_scale, inv_perm, n, k, hidden):
        r, s, inv = rows.numpy(), row_scale.numpy(), inv_perm.numpy().reshape(n, k)
        y = np.zeros((n, hidden), np.float64)
        for t in range(n):
            for slot in sorted(v for v in inv[t] if v >= 0):
                y[t] += r[slot].astype(np.float64) * s[slot]
        return torch.from_numpy(y.astype(np.float32))

    def combine(self, rows, inv_perm, n, k, hidden, shared_rows):
        y = rows.numpy()[inv_perm.numpy().reshape(n, k)].astype(np.float64).sum(1)
        if shared_rows is not None:
            y = y + shared_rows.numpy()
        return torch.from_numpy(y.astype(np.float32)).to(torch.bfloat16)

    def combine_scaled(self, rows, row_scale, inv_perm, n, k, hidden, shared_rows):
        r, s, inv = rows.numpy(), row_scale.numpy(), inv_perm.numpy().reshape(n, k)
        y = np.zeros((n, hidden), np.float64)
        for t in range(n):
            for slot in sorted(inv[t]):
                y[t] += r[slot].astype(np.float64) * s[slot]
        if shared_rows is not None:
            y += shared_rows.numpy()
        return torch.from_numpy(y.astype(np.float32)).to(torch.bfloat16)


def local_weights(p: O.MoEParams, rank, world):
    e_loc = p.num_experts // world
    sl = slice(rank * e_loc, (rank + 1) * e_loc)
    cut = lambda q: O.QLinear(q.w[sl], q.scales[sl], None if q.biases is None else q.biases[sl], q.group_size,
                              q.bits, q.mode, q.global_scale)
    cat = lambda a, b: O.QLinear(np.concatenate([a.w, b.w])[None], np.concatenate([a.scales, b.scales])[None],
                                 np.concatenate([a.biases, b.biases])[None], a.group_size, a.bits, a.mode)
    one = lambda q: O.QLinear(q.w[None], q.scales[None], q.biases[None], q.group_size, q.bits, q.mode)
    return ep.LocalExperts(p.router_w, cut(p.gate_up), cut(p.down), cat(p.shared_gate_proj, p.shared_up_proj),
                           one(p.shared_down_proj), p.shared_expert_gate_w, p.router_logit_bias)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        _, p = make_params(CFG)
        x = Workload(CFG).activations(block=rank)            # every rank has its own tokens
        moe = ep.ExpertParallelMoE(NumpyStages(), local_weights(p, rank, world), CFG.num_experts, CFG.top_k, True,
                                   CFG.hidden, CFG.intermediate, CFG.shared_intermediate)
        xt = torch.from_numpy(x).to(torch.bfloat16)
        y = moe.forward(xt, mode="a2a").float().numpy()
        ref = O.moe_forward(x, p)
        perm_ok = bool(np.array_equal(moe.last["perm"].numpy(), ref.perm))
        n_recv = int(moe.last["n_recv"])
        yg = moe.forward(xt, mode="gathered").float().numpy()
        idx_ok = bool(np.array_equal(moe.last["topk_idx"].numpy(), ref.top_idx))
        out[rank] = (max(O.rel_l2(y, ref.y), O.rel_l2(yg, ref.y)), perm_ok and idx_ok, n_recv)
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_ep_two_cpu_ranks_match_single_process():
    world = 2
    out = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert set(out.keys()) == {0, 1}
    for rank in range(world):
        err, perm_ok, _ = out[rank]
        assert perm_ok and err <= 2e-3, (rank, err)
    assert sum(v[2] for v in out.values()) == world * CFG.tokens * CFG.top_k      # every assignment was served once


def test_count_matrix_validation():
    good = torch.tensor([[2, 1], [0, 3]], dtype=torch.int32)
    ep.validate_counts(good, good, 6, 2, 2)
    with pytest.raises(_lib.IronMLXError):
        ep.validate_counts(good, good, 7, 2, 2)                     # a rank lost an assignment
    with pytest.raises(_lib.IronMLXError):
        ep.validate_counts(good[:1], good, 3, 2, 2)                 # truncated matrix
    bad = good.clone()
    bad[0, 0] = -1
    with pytest.raises(_lib.IronMLXError):
        ep.validate_counts(good, bad, 6, 2, 2)
