"""Expert parallelism for the MoE block: one process per GPU, the E experts
split into contiguous blocks of E/R per rank, tokens sharded across ranks, and
one all-to-all each way (dispatch of activation rows to the ranks that own
their experts, return of the expert outputs) over torch.distributed (NCCL on
NVLink).  The reference has no distributed code at all (no collective, no
communicator anywhere in its tree); single-device results are what this has to
reproduce.

Per step and rank (n local tokens, k experts per token):

  1. route + sort locally over the GLOBAL expert ids: because every rank owns
     a contiguous block of experts, the stable sort by expert id is already
     grouped by destination rank, then by expert, then by flat index.
  2. counts: an all-to-all of the [R, E/R] count matrix tells every rank how
     many rows it receives from each source for each of its experts; the two
     count matrices come to the host once per step (the split sizes of the
     all-to-all-v are host values).
  3. dispatch: fp16 activation rows gathered in sorted order -> all-to-all-v.
  4. local experts: received rows are ordered (source, expert); a second stable
     sort by local expert id gives the grouped order the expert kernels want.
  5. return: outputs (fp32, unweighted) put back in received order -> all-to-all-v.
  6. combine on the source rank: rows scaled by their routing weight and added
     per token in ascending expert order, plus the local gated shared expert
     (replicated weights, computed on a side stream under the exchanges).

Decode-size batches use a second schedule with no variable sizes and no host
sync (`forward_gathered`): all-gather the few tokens, route them everywhere
(the router is replicated), run the local experts on the assignments that fall
into the local block (the others are dropped by the sort), form fp32 partial
sums per token, reduce-scatter them back to the token owners, add the local
shared-expert rows and round.  Cross-rank sums are added in the collective's
order, not in ascending expert order; results stay within the block's
tolerance.

The stage kernels come from a `stages` object (the C ABI on CUDA tensors in
production; the tests substitute a CPU implementation to run the bookkeeping
on gloo ranks).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist

from . import _lib, nn, ops
from ._lib import MoEConfig, MoEWeights, check, lib


class CudaStages:
    """The stage-level C ABI calls on torch CUDA tensors."""

    def __init__(self, device):
        self.device = device
        self._scratch = {}

    def _buf(self, key, nbytes):
        b = self._scratch.get(key)
        if b is None or b.numel() < nbytes:
            b = torch.zeros(max(nbytes, 256), dtype=torch.uint8, device=self.device)
            self._scratch[key] = b
        return b

    def route(self, x, router_w, logit_bias, k, norm, shared_gate_w):
        n, h = x.shape
        e = router_w.shape[0]
        idx = torch.empty(n, k, dtype=torch.int32, device=x.device)
        w = torch.empty(n, k, dtype=torch.float32, device=x.device)
        sg = torch.empty(n, dtype=torch.float32, device=x.device)
        x16 = torch.empty(n, h, dtype=torch.float16, device=x.device)
        nb = C.c_size_t(0)
        check(lib().imx_moe_route_scratch_bytes(n, h, e, C.byref(nb)))
        scratch = self._buf("route", nb.value)
        check(lib().imx_moe_route_ws(x.data_ptr(), n, h, router_w.data_ptr(),
                                     None if logit_bias is None else logit_bias.data_ptr(), e, k, int(norm),
                                     None if shared_gate_w is None else shared_gate_w.data_ptr(), idx.data_ptr(),
                                     w.data_ptr(), sg.data_ptr(), x16.data_ptr(), scratch.data_ptr(),
                                     scratch.numel(), ops.stream_ptr()))
        return idx, w, sg, x16

    def sort(self, ids, num_experts):
        a = ids.numel()
        i32 = dict(dtype=torch.int32, device=ids.device)
        counts, offsets = torch.empty(num_experts, **i32), torch.empty(num_experts + 1, **i32)
        # perm is zero-filled: when ids are dropped, its tail stays a valid (unused) index
        perm, inv = torch.zeros(max(a, 1), **i32), torch.empty(max(a, 1), **i32)
        nb = C.c_size_t(0)
        check(lib().imx_moe_sort_scratch_bytes(a, num_experts, C.byref(nb)))
        scratch = self._buf("sort", nb.value)
        check(lib().imx_moe_sort(ids.data_ptr(), a, num_experts, counts.data_ptr(), offsets.data_ptr(),
                                 perm.data_ptr(), inv.data_ptr(), scratch.data_ptr(), scratch.numel(),
                                 ops.stream_ptr()))
        return counts, offsets, perm[:a], inv[:a]

    def gather_rows(self, src, index):
        n = index.numel()
        src2 = src.reshape(src.shape[0], -1)
        out = torch.empty((n,) + tuple(src2.shape[1:]), dtype=src.dtype, device=src.device)
        row_bytes = src2.shape[1] * src.element_size()
        check(lib().imx_gather_rows(src2.data_ptr(), index.data_ptr(), n, row_bytes, out.data_ptr(),
                                    ops.stream_ptr()))
        return out

    def experts(self, cfg: MoEConfig, gate_up: nn.QuantizedLinear, down: nn.QuantizedLinear, num_experts,
                x16, row_index, offsets, n_rows, row_scale, key="experts"):
        out = torch.empty(n_rows, cfg.hidden, dtype=torch.float32, device=x16.device)
        if n_rows == 0:
            return out
        nb = C.c_size_t(0)
        check(lib().imx_moe_experts_scratch_bytes(C.byref(cfg), n_rows, C.byref(nb)))
        scratch = self._buf(key, nb.value)
        g, d = gate_up.qtensor(), down.qtensor()
        check(lib().imx_moe_experts(C.byref(cfg), C.byref(g), C.byref(d), num_experts, x16.data_ptr(),
                                    None if row_index is None else row_index.data_ptr(), offsets.data_ptr(),
                                    n_rows, n_rows, None if row_scale is None else row_scale.data_ptr(),
                                    out.data_ptr(), scratch.data_ptr(), scratch.numel(), ops.stream_ptr()))
        return out

    def combine_partial(self, rows, row_scale, inv_perm, n, k, hidden):
        y = torch.empty(n, hidden, dtype=torch.float32, device=rows.device)
        check(lib().imx_moe_combine_partial(rows.data_ptr(), None if row_scale is None else row_scale.data_ptr(),
                                            inv_perm.data_ptr(), n, k, hidden, y.data_ptr(), ops.stream_ptr()))
        return y

    def combine(self, rows, inv_perm, n, k, hidden, shared_rows):
        y = torch.empty(n, hidden, dtype=torch.bfloat16, device=rows.device)
        check(lib().imx_moe_combine(rows.data_ptr(), inv_perm.data_ptr(), n, k, hidden,
                                    None if shared_rows is None else shared_rows.data_ptr(), y.data_ptr(),
                                    ops.stream_ptr()))
        return y

    def combine_scaled(self, rows, row_scale, inv_perm, n, k, hidden, shared_rows):
        y = torch.empty(n, hidden, dtype=torch.bfloat16, device=rows.device)
        check(lib().imx_moe_combine_scaled(rows.data_ptr(), row_scale.data_ptr(), inv_perm.data_ptr(), n, k, hidden,
                                           None if shared_rows is None else shared_rows.data_ptr(), y.data_ptr(),
                                           ops.stream_ptr()))
        return y


@dataclass
class LocalExperts:
    """The weights one rank holds: its block of routed experts (fused layout)
    and, replicated on every rank, the router, the shared expert (gate and up
    rows fused once into [1, 2*Is, .]) and the shared-expert gate."""
    router_w: torch.Tensor
    gate_up: nn.QuantizedLinear        # [E/R, 2I, .]
    down: nn.QuantizedLinear           # [E/R, H, .]
    shared_gate_up: Optional[nn.QuantizedLinear] = None   # [1, 2Is, .]
    shared_down: Optional[nn.QuantizedLinear] = None      # [1, H, .]
    shared_expert_gate_w: Optional[torch.Tensor] = None
    router_logit_bias: Optional[torch.Tensor] = None
    shared_mlp: Optional[nn.MLP] = None                   # the same shared expert as three separate projections


def fuse_shared(mlp: nn.MLP):
    """gate_proj/up_proj [Is, .] -> one [1, 2Is, .] tensor; down -> [1, H, .]."""
    g, u, d = mlp.gate_proj, mlp.up_proj, mlp.down_proj
    cat = lambda a, b: None if a is None else torch.cat([a, b], 0).unsqueeze(0).contiguous()
    gu = nn.QuantizedLinear(cat(g.weight, u.weight), cat(g.scales, u.scales), cat(g.biases, u.biases),
                            g.group_size, g.bits, g.mode, g.global_scale)
    dn = nn.QuantizedLinear(d.weight.unsqueeze(0).contiguous(), d.scales.unsqueeze(0).contiguous(),
                            None if d.biases is None else d.biases.unsqueeze(0).contiguous(),
                            d.group_size, d.bits, d.mode, d.global_scale)
    return gu, dn


def validate_counts(send_cnt: torch.Tensor, recv_cnt: torch.Tensor, n_assign: int, world: int, e_local: int):
    """Host-side checks on the count matrices before any data moves; a mismatch
    here means a rank disagrees about the exchange and must not reach NCCL."""
    if tuple(send_cnt.shape) != (world, e_local) or tuple(recv_cnt.shape) != (world, e_local):
        raise _lib.IronMLXError(_lib.ERR_INVALID, "expert-parallel count matrix has the wrong shape")
    if int(send_cnt.min()) < 0 or int(recv_cnt.min()) < 0:
        raise _lib.IronMLXError(_lib.ERR_INVALID, "negative count in the expert-parallel exchange")
    if int(send_cnt.sum()) != n_assign:
        raise _lib.IronMLXError(_lib.ERR_INVALID,
                                f"dispatch counts sum to {int(send_cnt.sum())}, expected {n_assign} assignments")


class ExpertParallelMoE:
    def __init__(self, stages, weights: LocalExperts, num_experts: int, top_k: int, norm_topk_prob: bool,
                 hidden: int, intermediate: int, shared_intermediate: int, group=None, path: str = "auto"):
        self.st = stages
        self.w = weights
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if num_experts % self.world:
            raise _lib.IronMLXError(_lib.ERR_INVALID, "num_experts must be divisible by the number of ranks")
        self.E, self.k, self.norm = num_experts, top_k, norm_topk_prob
        self.E_loc = num_experts // self.world
        self.H, self.I, self.Is = hidden, intermediate, shared_intermediate
        q = weights.gate_up
        mk = lambda inter, ne: MoEConfig(hidden, ne, 1, inter, 0, 1, _lib.MODE[q.mode], q.bits, q.group_size,
                                         _lib.PATH[path])
        self.cfg_routed = mk(intermediate, self.E_loc)
        self.cfg_shared = mk(shared_intermediate, 1) if shared_intermediate else None
        # The routed and the shared expert calls run one after the other on the caller's stream: both are
        # stream-K launches whose CTAs hand partial sums to one another and must not share the GPU.
        self.side_stream = None
        self.last = {}
        self._off_cache = {}
        self.gather_limit = 1024         # global tokens up to which the gathered schedule is used

    # -- collectives -----------------------------------------------------------
    def _a2a(self, send, out_rows: int, in_splits: List[int], out_splits: List[int]):
        recv = torch.empty((out_rows,) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
        dist.all_to_all_single(recv, send, output_split_sizes=out_splits, input_split_sizes=in_splits,
                               group=self.group)
        return recv

    def forward(self, x: torch.Tensor, mode: str = "auto") -> torch.Tensor:
        """mode: "a2a" (dispatch/return all-to-all), "gathered" (all-gather + reduce-scatter),
        "auto" (gathered while the global batch is at most `gather_limit` tokens)."""
        if mode == "gathered" or (mode == "auto" and x.shape[0] * self.world <= self.gather_limit):
            return self.forward_gathered(x)
        return self.forward_a2a(x)

    def _offsets_0n(self, n, dev):
        """[0, n] on the device, made once per n (no host-to-device copy inside a step)."""
        t = self._off_cache.get(n)
        if t is None:
            t = torch.tensor([0, n], dtype=torch.int32, device=dev)
            self._off_cache[n] = t
        return t

    def _identity(self, n, dev):
        """arange(n) on the device, made once per n."""
        t = self._off_cache.get(("ident", n))
        if t is None:
            t = torch.arange(n, dtype=torch.int32, device=dev)
            self._off_cache[("ident", n)] = t
        return t

    def _all_gather(self, x):
        out = torch.empty((self.world * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        if dist.get_backend(self.group) == "gloo":
            parts = [torch.empty_like(x) for _ in range(self.world)]
            dist.all_gather(parts, x, group=self.group)
            return torch.cat(parts, 0)
        dist.all_gather_into_tensor(out, x, group=self.group)
        return out

    def _reduce_scatter(self, partial, n):
        if dist.get_backend(self.group) == "gloo":          # gloo has no reduce-scatter: all-reduce and slice
            dist.all_reduce(partial, group=self.group)
            return partial[self.rank * n:(self.rank + 1) * n].contiguous()
        out = torch.empty((n,) + tuple(partial.shape[1:]), dtype=partial.dtype, device=partial.device)
        dist.reduce_scatter_tensor(out, partial, group=self.group)
        return out

    def forward_gathered(self, x: torch.Tensor) -> torch.Tensor:
        st, w = self.st, self.w
        n = x.shape[0]
        dev = x.device
        xg = self._all_gather(x.contiguous())
        n_all = xg.shape[0]
        idx, tw, sg, x16 = st.route(xg, w.router_w, w.router_logit_bias, self.k, self.norm, w.shared_expert_gate_w)
        shared_rows = None
        if self.Is:
            off = self._offsets_0n(n, dev)
            own = slice(self.rank * n, (self.rank + 1) * n)
            run = lambda: st.experts(self.cfg_shared, w.shared_gate_up, w.shared_down, 1, x16[own].contiguous(), None,
                                     off, n, sg[own].contiguous(), key="shared")
            if self.side_stream is not None:
                self.side_stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self.side_stream):
                    shared_rows = run()
            else:
                shared_rows = run()
        # ids outside the local block become out of range and are dropped by the sort (moe.rs:100)
        ids_local = (idx.reshape(-1) - self.rank * self.E_loc).to(torch.int32)
        counts, off2, perm, inv = st.sort(ids_local, self.E_loc)
        a_all = n_all * self.k
        tok = torch.div(perm, self.k, rounding_mode="floor").to(torch.int32)
        out = st.experts(self.cfg_routed, w.gate_up, w.down, self.E_loc, x16, tok, off2, a_all, None)
        w_sorted = st.gather_rows(tw.reshape(-1, 1), perm).reshape(-1)
        partial = st.combine_partial(out, w_sorted, inv, n_all, self.k, self.H)
        mine = self._reduce_scatter(partial, n)
        if self.side_stream is not None and shared_rows is not None:
            torch.cuda.current_stream().wait_stream(self.side_stream)
        y = st.combine(mine, self._identity(n, dev), n, 1, self.H, shared_rows)
        own_idx = idx[self.rank * n:(self.rank + 1) * n]
        self.last = {"topk_idx": own_idx, "topk_w": tw[self.rank * n:(self.rank + 1) * n], "counts": counts,
                     "n_recv": -1, "mode": "gathered",
                     "a2a_bytes": (self.world - 1) * n * self.H * 2 + (self.world - 1) * n * self.H * 4}
        return y

    def forward_a2a(self, x: torch.Tensor) -> torch.Tensor:
        st, w = self.st, self.w
        n = x.shape[0]
        a = n * self.k
        dev = x.device
        idx, tw, sg, x16 = st.route(x, w.router_w, w.router_logit_bias, self.k, self.norm, w.shared_expert_gate_w)

        # shared expert: local tokens, replicated weights, off the critical path
        shared_rows = None
        if self.Is:
            off = self._offsets_0n(n, dev)
            if self.side_stream is not None:
                self.side_stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self.side_stream):
                    shared_rows = st.experts(self.cfg_shared, w.shared_gate_up, w.shared_down, 1, x16, None, off, n,
                                             sg, key="shared")
            else:
                shared_rows = st.experts(self.cfg_shared, w.shared_gate_up, w.shared_down, 1, x16, None, off, n, sg,
                                         key="shared")

        counts, offsets, perm, inv = st.sort(idx.reshape(-1), self.E)
        send_cnt = counts.view(self.world, self.E_loc).contiguous()
        recv_cnt = torch.empty_like(send_cnt)
        dist.all_to_all_single(recv_cnt, send_cnt, group=self.group)
        both = torch.stack([send_cnt, recv_cnt]).cpu()                    # the one host sync of the step
        validate_counts(both[0], both[1], a, self.world, self.E_loc)
        in_splits = both[0].sum(1).tolist()
        out_splits = both[1].sum(1).tolist()
        n_recv = int(sum(out_splits))

        tok = torch.div(perm, self.k, rounding_mode="floor").to(torch.int32)
        send_rows = st.gather_rows(x16, tok)
        recv_rows = self._a2a(send_rows, n_recv, in_splits, out_splits)

        # received rows are ordered (source rank, local expert): regroup by expert
        ids = torch.repeat_interleave(torch.arange(self.E_loc, dtype=torch.int32, device=dev).repeat(self.world),
                                      recv_cnt.reshape(-1).to(torch.int64), output_size=n_recv).to(torch.int32)
        _, off2, perm2, inv2 = st.sort(ids, self.E_loc)
        out_sorted = st.experts(self.cfg_routed, w.gate_up, w.down, self.E_loc, recv_rows, perm2, off2, n_recv, None)
        back = st.gather_rows(out_sorted, inv2) if n_recv else out_sorted
        ret_rows = self._a2a(back, a, out_splits, in_splits)

        w_sorted = st.gather_rows(tw.reshape(-1, 1), perm).reshape(-1)
        if self.side_stream is not None and shared_rows is not None:
            torch.cuda.current_stream().wait_stream(self.side_stream)
        y = st.combine_scaled(ret_rows, w_sorted, inv, n, self.k, self.H, shared_rows)
        self.last = {"topk_idx": idx, "topk_w": tw, "perm": perm, "counts": counts, "n_recv": n_recv, "mode": "a2a",
                     "a2a_bytes": (sum(in_splits) - in_splits[self.rank]) * self.H * 2
                     + (sum(out_splits) - out_splits[self.rank]) * self.H * 4}
        return y


class ExpertParallel:
    """The expert-parallel block behind the C ABI (`imx_ep_*`, csrc/ep.cu): NCCL collectives issued by the
    library itself on its own communicator, the stage kernels enqueued without Python in between.  One
    instance per process / GPU; `forward` is collective.

    `weights` holds this rank's block of experts (`LocalExperts`); the communicator's unique id travels from
    rank 0 through `torch.distributed` (any backend), which is otherwise not used on the data path."""

    def __init__(self, weights: LocalExperts, num_experts: int, top_k: int, norm_topk_prob: bool, hidden: int,
                 intermediate: int, shared_intermediate: int, group=None, path: str = "auto",
                 comm_of: Optional["ExpertParallel"] = None):
        """comm_of: another instance of this process whose communicator is borrowed (one communicator per set
        of ranks is enough; the instance that created it must outlive this one)."""
        self.w = weights
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        q = weights.gate_up
        self.cfg = MoEConfig(hidden, num_experts, top_k, intermediate, shared_intermediate, int(norm_topk_prob),
                             _lib.MODE[q.mode], q.bits, q.group_size, _lib.PATH[path])
        self.hidden = hidden
        dev = weights.router_w.device
        self._ctx = C.c_void_p()
        self._comm_owner = comm_of
        with torch.cuda.device(dev):
            if comm_of is not None:
                check(lib().imx_ep_create_from_comm(C.byref(self.cfg), lib().imx_ep_comm(comm_of._ctx), self.rank,
                                                    self.world, C.byref(self._ctx)))
            else:
                uid = torch.zeros(128, dtype=torch.uint8)
                if self.rank == 0:
                    buf = (C.c_ubyte * 128)()
                    check(lib().imx_ep_unique_id(buf))
                    uid = torch.tensor(list(buf), dtype=torch.uint8)
                uid = uid.to(dev) if dist.get_backend(group) == "nccl" else uid
                dist.broadcast(uid, 0, group=group)
                raw = bytes(uid.cpu().tolist())
                check(lib().imx_ep_create(C.byref(self.cfg), raw, self.rank, self.world, C.byref(self._ctx)))
        self._ws = {}
        self.info = _lib.EpInfo()
        self._weights = self._make_weights()

    def _make_weights(self) -> MoEWeights:
        w, lw = MoEWeights(), self.w
        w.router_w = lw.router_w.data_ptr()
        w.router_logit_bias = None if lw.router_logit_bias is None else lw.router_logit_bias.data_ptr()
        w.gate_up = lw.gate_up.qtensor()
        w.down = lw.down.qtensor()
        if lw.shared_mlp is not None:
            w.shared_gate_proj = lw.shared_mlp.gate_proj.qtensor()
            w.shared_up_proj = lw.shared_mlp.up_proj.qtensor()
            w.shared_down_proj = lw.shared_mlp.down_proj.qtensor()
            w.shared_expert_gate_w = lw.shared_expert_gate_w.data_ptr()
        return w

    def workspace(self, n_local: int, schedule: str, device) -> torch.Tensor:
        key = (n_local, schedule)
        ws = self._ws.get(key)
        if ws is None:
            nb = C.c_size_t(0)
            check(lib().imx_ep_workspace_bytes(self._ctx, n_local, _lib.EP_SCHEDULE[schedule], C.byref(nb)))
            ws = torch.zeros(nb.value, dtype=torch.uint8, device=device)
            self._ws[key] = ws
        return ws

    def forward(self, x: torch.Tensor, schedule: str = "auto", y: Optional[torch.Tensor] = None, timed: bool = False,
                trace: bool = False):
        """Collective.  timed: fill `info.phase_ms` (all-to-all schedule; synchronises).  trace: also return the
        local tokens' routing and dispatch permutation (all-to-all schedule)."""
        if x.dtype != torch.bfloat16 or not x.is_cuda or x.shape[-1] != self.hidden:
            raise _lib.IronMLXError(_lib.ERR_INVALID, "ExpertParallel: x must be a bfloat16 CUDA tensor [n, hidden]")
        x = x.contiguous()
        n = x.numel() // self.hidden
        ws = self.workspace(n, schedule, x.device)
        if y is None:
            y = torch.empty_like(x)
        tr, tensors = None, None
        if trace:
            k, e = self.cfg.top_k, self.cfg.num_experts
            i32 = dict(dtype=torch.int32, device=x.device)
            tensors = {"topk_idx": torch.empty(n, k, **i32), "topk_w": torch.empty(n, k, device=x.device),
                       "counts": torch.empty(e, **i32), "offsets": torch.empty(e + 1, **i32),
                       "perm": torch.empty(n * k, **i32), "inv_perm": torch.empty(n * k, **i32),
                       "shared_gate": torch.empty(n, device=x.device)}
            tr = _lib.MoETrace(**{name: t.data_ptr() for name, t in tensors.items()})
        self.info.want_timing = int(timed)
        check(lib().imx_ep_forward(self._ctx, C.byref(self._weights), x.data_ptr(), n, y.data_ptr(), ws.data_ptr(),
                                   ws.numel(), ops.stream_ptr(), _lib.EP_SCHEDULE[schedule], C.byref(self.info),
                                   None if tr is None else C.byref(tr)))
        self._last_ws = ws
        return (y, tensors) if trace else y

    def check_status(self) -> None:
        ws = getattr(self, "_last_ws", None)
        if ws is not None:
            check(lib().imx_moe_status(ws.data_ptr(), ops.stream_ptr()))

    def close(self) -> None:
        """Frees the context (and the communicator it created).  Release CUDA graphs that captured `forward` first."""
        if self._ctx:
            lib().imx_ep_destroy(self._ctx)
            self._ctx = C.c_void_p()


# ── synthetic construction + the benchmark's runner ──────────────────────────

def build_local(cfg, device, rank: int, world: int) -> LocalExperts:
    """This rank's weights of a seeded synthetic configuration (GPU quantizer)."""
    from . import synthetic
    from .workloads import Workload
    wl = Workload(cfg)
    e_loc = cfg.num_experts // world
    lo = rank * e_loc
    gs_gu = gs_dn = None
    if cfg.mode == "nvfp4":
        # one fp32 scale per stacked tensor, derived from ALL experts so that every rank quantizes its block exactly
        # as the single-GPU block does
        import numpy as np
        gs_gu = synthetic.nvfp4_tensor_scale(max(float(np.abs(wl.expert_gate_up(e)).max()) for e in range(cfg.num_experts)))
        gs_dn = synthetic.nvfp4_tensor_scale(max(float(np.abs(wl.expert_down(e)).max()) for e in range(cfg.num_experts)))
    gate_up = synthetic._quantize_stack(lambda e: wl.expert_gate_up(lo + e), e_loc, cfg, device, gs_gu)
    down = synthetic._quantize_stack(lambda e: wl.expert_down(lo + e), e_loc, cfg, device, gs_dn)
    out = LocalExperts(synthetic._bf16(wl.router_weight(), device), gate_up, down)
    if cfg.shared_intermediate:
        mlp = nn.MLP(*(synthetic._single(synthetic._quantize_stack(lambda e, nm=nm: wl.shared(nm), 1, cfg, device))
                       for nm in ("gate_proj", "up_proj", "down_proj")))
        out.shared_gate_up, out.shared_down = fuse_shared(mlp)
        out.shared_mlp = mlp
        out.shared_expert_gate_w = synthetic._bf16(wl.shared_gate_weight(), device)
    bias = wl.router_logit_bias()
    if bias is not None:
        out.router_logit_bias = torch.from_numpy(bias).to(device)
    return out


class BenchRunner:
    """What bench.py drives at N > 1: `cfg.tokens` tokens per rank (weak scaling),
    experts split across the ranks."""

    # kernels of this library per gathered step: router 2, sort 1, routed and shared experts 5 each (unit list,
    # row permutation, group sums, two products), row gather 1, partial combine 1, final combine 1
    launches_per_step = 16

    def __init__(self, cfg, device, rank, world):
        from .workloads import Workload
        self.cfg = cfg
        self.moe = ExpertParallelMoE(CudaStages(device), build_local(cfg, device, rank, world), cfg.num_experts,
                                     cfg.top_k, cfg.norm_topk_prob, cfg.hidden, cfg.intermediate,
                                     cfg.shared_intermediate)
        x = Workload(cfg).activations(block=rank)
        self.x = torch.from_numpy(x).to(device).to(torch.bfloat16)
        self.xh = self.x.cpu().pin_memory()
        self.yh = torch.empty_like(self.xh).pin_memory()
        self.xd = self.x.clone()

        # The gathered schedule has fixed shapes and no host sync: replay it as a CUDA graph
        # (kernels, the two NCCL collectives and the side stream captured once).
        self.graph = None
        self.y = None
        if self.moe.forward is not None and cfg.tokens * world <= self.moe.gather_limit:
            try:
                for _ in range(3):
                    self.y = self.moe.forward(self.xd_static())
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self.y = self.moe.forward(self.xd)
                self.graph = g
            except Exception as e:            # capture not possible on this stack: run eagerly
                self.graph = None
                self.capture_error = repr(e)
                torch.cuda.synchronize()

    def xd_static(self):
        self.xd.copy_(self.x)
        return self.xd

    def step(self):
        if self.graph is not None:
            self.graph.replay()
            return self.y
        return self.moe.forward(self.xd)

    def step_host(self):
        self.xd.copy_(self.xh, non_blocking=True)
        y = self.step()
        self.yh.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def extra(self):
        return {"ep": {"experts_per_rank": self.moe.E_loc, "tokens_per_rank": self.cfg.tokens,
                       "a2a_bytes_per_rank_per_step": int(self.moe.last.get("a2a_bytes", 0)),
                       "schedule": self.moe.last.get("mode"), "cuda_graph": self.graph is not None,
                       "exchange": "gathered: NCCL all-gather of tokens + reduce-scatter of fp32 partial rows; "
                                   "a2a: NCCL all_to_all_single (fp16 rows out, fp32 rows back) + count all-to-all"}}


def build_bench_runner(cfg, device, rank, world) -> BenchRunner:
    return BenchRunner(cfg, device, rank, world)
