"""Host-side mirror of the layer types on the MoE path of the reference:
`Linear`, `QuantizedLinear`, `LinearLayer` (mlx/src/nn/linear.rs), `MLP`
(mlx/src/nn/mlp.rs), `Expert` and `MoEMLP` (mlx/src/nn/moe.rs:11-52), with
the same field names and `forward_with_stream(x, stream)` entry points, so
model code that builds these structs literally
(mlx/src/model/qwen35.rs:489-531) keeps working.

`MoEMLP.forward_with_stream` is one call into the C ABI (`imx_moe_forward`);
the per-expert host loop, the mid-layer device->host sync and the per-row
graph nodes of the reference (moe.rs:86-170) do not exist here.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional, Sequence, Union

import torch

from . import _lib
from . import ops
from ._lib import IronMLXError, MoEConfig, MoETrace, MoEWeights, QTensor, check, lib


@dataclass
class Linear:
    """Dense `x @ W^T (+ b)` (mlx/src/nn/linear.rs:129-177).  On the MoE path
    only the router and the shared-expert gate are dense, and both are consumed
    inside the fused block; called on its own it is one bf16 tensor-core GEMM."""
    weight: torch.Tensor
    bias: Optional[torch.Tensor] = None

    def forward_with_stream(self, x: torch.Tensor, stream=None) -> torch.Tensor:
        return ops.linear(x, self.weight, self.bias, stream)


@dataclass
class RMSNorm:
    """mlx/src/nn/norm.rs:11-24: weight [H] and eps; forward = `fast::rms_norm`."""
    weight: torch.Tensor
    eps: float = 1e-6

    @classmethod
    def new(cls, weight: torch.Tensor, eps: float) -> "RMSNorm":
        return cls(weight, eps)

    def forward_with_stream(self, x: torch.Tensor, stream=None) -> torch.Tensor:
        return ops.rms_norm(x, self.weight, self.eps, stream)


@dataclass
class QuantizedLinear:
    """mlx/src/nn/linear.rs:13-63: packed weight + per-group scales/biases,
    forward = `quantized_matmul(x, w, scales, biases, transpose=true, ...)`."""
    weight: torch.Tensor
    scales: torch.Tensor
    biases: Optional[torch.Tensor]
    group_size: int = 64
    bits: int = 4
    mode: str = "affine"
    global_scale: Optional[float] = None

    @classmethod
    def new(cls, weight, scales, biases, group_size: int, bits: int) -> "QuantizedLinear":
        return cls(weight, scales, biases, group_size, bits, "affine")

    @classmethod
    def new_with_mode(cls, weight, scales, biases, group_size: int, bits: int, mode: str,
                      global_scale: Optional[float] = None) -> "QuantizedLinear":
        return cls(weight, scales, biases, group_size, bits, mode, global_scale)

    def forward_with_stream(self, x: torch.Tensor, stream=None) -> torch.Tensor:
        return ops.quantized_matmul(x, self.weight, self.scales, self.biases, True, self.group_size,
                                    self.bits, self.mode, stream, self.global_scale)

    def qtensor(self) -> QTensor:
        return ops.qtensor(self.weight, self.scales, self.biases, self.global_scale)


LinearLayer = Union[Linear, QuantizedLinear]


class _SwiGLU:
    """`down(silu(gate(x)) * up(x))` in one call: the gate and up rows as one [2I, .] tensor (a view when they
    are adjacent slices of the fused checkpoint tensor, stacked once otherwise)."""

    def forward_with_stream(self, x: torch.Tensor, stream=None) -> torch.Tensor:
        g, u, d = self.gate_proj, self.up_proj, self.down_proj
        if (g.mode, g.bits, g.group_size) != (u.mode, u.bits, u.group_size) or (g.mode, g.bits, g.group_size) != (d.mode, d.bits, d.group_size):
            raise IronMLXError(_lib.ERR_INVALID, "the three projections of an expert must share one quantization format")
        if g.mode == "nvfp4" and (g.global_scale or 1.0) != (u.global_scale or 1.0):
            raise IronMLXError(_lib.ERR_INVALID, "gate_proj and up_proj carry different nvfp4 tensor scales")
        fused = getattr(self, "_fused_gate_up", None)
        if fused is None:
            def both(a, b):
                if a is None:
                    return None
                step = a.numel() * a.element_size()
                # adjacent slices of ONE tensor (same storage, which also has to hold both): neighbours in
                # memory that belong to two allocations are not a view of anything
                same = (a.untyped_storage().data_ptr() == b.untyped_storage().data_ptr()
                        and a.untyped_storage().nbytes() >= a.storage_offset() * a.element_size() + 2 * step)
                if same and a.is_contiguous() and b.is_contiguous() and b.data_ptr() == a.data_ptr() + step:
                    return a.as_strided((2 * a.shape[0],) + tuple(a.shape[1:]), a.stride(), a.storage_offset())
                return torch.cat([a, b], 0).contiguous()
            fused = (both(g.weight, u.weight), both(g.scales, u.scales), both(g.biases, u.biases))
            self._fused_gate_up = fused
        return ops.expert_forward(x, fused[0], fused[1], fused[2], d.weight, d.scales, d.biases, g.group_size, g.bits,
                                  g.mode, stream, g.global_scale, d.global_scale)


@dataclass
class MLP(_SwiGLU):
    """SwiGLU MLP, `down(silu(gate(x)) * up(x))` (mlx/src/nn/mlp.rs:12-33);
    the shared expert of the block."""
    gate_proj: QuantizedLinear
    up_proj: QuantizedLinear
    down_proj: QuantizedLinear


@dataclass
class Expert(_SwiGLU):
    """One routed expert (mlx/src/nn/moe.rs:11-33).  Its three projections are
    views into the fused [E, 2I, .] / [E, H, .] checkpoint tensors
    (mlx/src/model/qwen35.rs:661-776)."""
    gate_proj: QuantizedLinear
    up_proj: QuantizedLinear
    down_proj: QuantizedLinear


def _stack_or_view(parts: Sequence[torch.Tensor]) -> torch.Tensor:
    """[E] equally shaped tensors -> one contiguous [E, ...] tensor; no copy
    when they already are consecutive slices of one allocation."""
    first = parts[0]
    step = first.numel() * first.element_size()
    if all(p.is_contiguous() and p.data_ptr() == first.data_ptr() + i * step for i, p in enumerate(parts)):
        base = first.as_strided((len(parts),) + tuple(first.shape), (first.numel(),) + tuple(first.stride()))
        return base
    return torch.stack([p.contiguous() for p in parts])


class MoEMLP:
    """Mixture-of-experts MLP with a gated shared expert (mlx/src/nn/moe.rs:39-52).

    Fields keep the reference's names: gate (router), experts, shared_expert,
    shared_expert_gate, num_experts_per_tok, norm_topk_prob.
    """

    def __init__(self, gate: Linear, experts: Union[List[Expert], "FusedExperts"],
                 shared_expert: Optional[MLP], shared_expert_gate: Optional[Linear],
                 num_experts_per_tok: int, norm_topk_prob: bool = True,
                 router_logit_bias: Optional[torch.Tensor] = None, path: str = "auto"):
        self.gate = gate
        self.experts = experts
        self.shared_expert = shared_expert
        self.shared_expert_gate = shared_expert_gate
        self.num_experts_per_tok = int(num_experts_per_tok)
        self.norm_topk_prob = bool(norm_topk_prob)
        self.router_logit_bias = router_logit_bias
        self.path = path
        self._fused = experts if isinstance(experts, FusedExperts) else FusedExperts.from_experts(experts)
        self._workspace = None
        f = self._fused
        self.num_experts = f.gate_up.weight.shape[0]
        self.hidden = gate.weight.shape[1]
        self.intermediate = f.gate_up.weight.shape[1] // 2
        self.shared_intermediate = 0 if shared_expert is None else shared_expert.gate_proj.weight.shape[0]
        if gate.weight.shape[0] != self.num_experts:
            raise IronMLXError(_lib.ERR_INVALID, "router rows must equal the number of experts")
        if (shared_expert is None) != (shared_expert_gate is None):
            raise IronMLXError(_lib.ERR_INVALID, "shared_expert and shared_expert_gate go together")
        if shared_expert is not None:
            q = f.gate_up
            for proj in (shared_expert.gate_proj, shared_expert.up_proj, shared_expert.down_proj):
                if (proj.mode, proj.bits, proj.group_size) != (q.mode, q.bits, q.group_size):
                    raise IronMLXError(_lib.ERR_INVALID, "the shared expert must use the routed experts' quantization format")

    # -- C structs ----------------------------------------------------------
    def config(self, path: Optional[str] = None) -> MoEConfig:
        q = self._fused.gate_up
        return MoEConfig(self.hidden, self.num_experts, self.num_experts_per_tok, self.intermediate,
                         self.shared_intermediate, int(self.norm_topk_prob), _lib.MODE[q.mode], q.bits,
                         q.group_size, _lib.PATH[path or self.path])

    def weights(self) -> MoEWeights:
        w = MoEWeights()
        w.router_w = self.gate.weight.data_ptr()
        w.router_logit_bias = None if self.router_logit_bias is None else self.router_logit_bias.data_ptr()
        w.gate_up = self._fused.gate_up.qtensor()
        w.down = self._fused.down.qtensor()
        if self.shared_expert is not None:
            w.shared_gate_proj = self.shared_expert.gate_proj.qtensor()
            w.shared_up_proj = self.shared_expert.up_proj.qtensor()
            w.shared_down_proj = self.shared_expert.down_proj.qtensor()
            w.shared_expert_gate_w = self.shared_expert_gate.weight.data_ptr()
        return w

    def workspace_bytes(self, n_tokens: int, host_io: bool = False) -> int:
        cfg = self.config()
        out = C.c_size_t(0)
        check(lib().imx_moe_workspace_bytes(C.byref(cfg), n_tokens, C.byref(out)))
        extra = 2 * ((n_tokens * self.hidden * 2 + 255) // 256 * 256) if host_io else 0
        return out.value + extra

    def _ws(self, n_tokens: int, device, host_io: bool = False) -> torch.Tensor:
        need = self.workspace_bytes(n_tokens, host_io)
        if self._workspace is None or self._workspace.numel() < need or self._workspace.device != device:
            self._workspace = torch.zeros(need, dtype=torch.uint8, device=device)
        return self._workspace

    # -- forward ------------------------------------------------------------
    def forward_with_stream(self, x: torch.Tensor, stream=None, trace: bool = False, path: Optional[str] = None):
        """x: bf16 [B, L, H] (or [N, H]) -> same shape (moe.rs:55-183).
        With trace=True also returns the per-stage tensors as a dict."""
        if x.dtype != torch.bfloat16 or not x.is_cuda:
            raise IronMLXError(_lib.ERR_INVALID, "MoEMLP: x must be a bfloat16 CUDA tensor")
        if x.shape[-1] != self.hidden:
            raise IronMLXError(_lib.ERR_INVALID, f"MoEMLP: last dimension {x.shape[-1]} != hidden {self.hidden}")
        x = x.contiguous()
        n = x.numel() // self.hidden
        y = torch.empty_like(x)
        ws = self._ws(n, x.device)
        cfg, w = self.config(path), self.weights()
        tr, tensors = None, None
        if trace:
            k, e = self.num_experts_per_tok, self.num_experts
            i32 = dict(dtype=torch.int32, device=x.device)
            tensors = {
                "topk_idx": torch.empty(n, k, **i32), "topk_w": torch.empty(n, k, device=x.device),
                "counts": torch.empty(e, **i32), "offsets": torch.empty(e + 1, **i32),
                "perm": torch.empty(n * k, **i32), "inv_perm": torch.empty(n * k, **i32),
                "shared_gate": torch.empty(n, device=x.device),
            }
            tr = MoETrace(**{name: t.data_ptr() for name, t in tensors.items()})
        check(lib().imx_moe_forward(C.byref(cfg), C.byref(w), x.data_ptr(), n, y.data_ptr(), ws.data_ptr(),
                                    ws.numel(), ops.stream_ptr(stream), None if tr is None else C.byref(tr)))
        return (y, tensors) if trace else y

    def forward_residual(self, h: torch.Tensor, norm: "RMSNorm", stream=None, trace: bool = False):
        """The MoE half of a decoder layer (mlx/src/model/qwen35.rs:271-276):
        `h + self.forward(norm.forward(h))` in one call, the normalisation fused into
        the router's loads and the residual into the combine stage's rounding."""
        if h.dtype != torch.bfloat16 or not h.is_cuda or h.shape[-1] != self.hidden:
            raise IronMLXError(_lib.ERR_INVALID, "MoEMLP: h must be a bfloat16 CUDA tensor [.., hidden]")
        h = h.contiguous()
        n = h.numel() // self.hidden
        y = torch.empty_like(h)
        ws = self._ws(n, h.device)
        cfg, w = self.config(), self.weights()
        tr, tensors = None, None
        if trace:
            k, e = self.num_experts_per_tok, self.num_experts
            i32 = dict(dtype=torch.int32, device=h.device)
            tensors = {
                "topk_idx": torch.empty(n, k, **i32), "topk_w": torch.empty(n, k, device=h.device),
                "counts": torch.empty(e, **i32), "offsets": torch.empty(e + 1, **i32),
                "perm": torch.empty(n * k, **i32), "inv_perm": torch.empty(n * k, **i32),
                "shared_gate": torch.empty(n, device=h.device),
            }
            tr = MoETrace(**{name: t.data_ptr() for name, t in tensors.items()})
        lw = None if norm.weight is None else norm.weight.data_ptr()
        check(lib().imx_moe_forward_residual(C.byref(cfg), C.byref(w), h.data_ptr(), lw, float(norm.eps), n,
                                             y.data_ptr(), ws.data_ptr(), ws.numel(), ops.stream_ptr(stream),
                                             None if tr is None else C.byref(tr)))
        return (y, tensors) if trace else y

    def capture(self, x: torch.Tensor, x_host: Optional[torch.Tensor] = None,
                y_host: Optional[torch.Tensor] = None) -> "CapturedForward":
        """The block for a fixed input buffer as a CUDA graph: every kernel of
        `forward_with_stream(x)` recorded once and replayed with one launch
        (decode loops call the block with the same shapes every step).  With
        pinned host buffers the graph also holds the copy of `x_host` to the
        device before the block and the copy of the result to `y_host` after it."""
        return CapturedForward(self, x, x_host, y_host)

    def forward_timed(self, x: torch.Tensor, stream=None):
        """-> (y, [router, sort, gate/up, down, combine] milliseconds), measured
        with CUDA events recorded between the stages on the stream."""
        x = x.contiguous()
        n = x.numel() // self.hidden
        y = torch.empty_like(x)
        ws = self._ws(n, x.device)
        cfg, w = self.config(), self.weights()
        ms = (C.c_float * 5)()
        check(lib().imx_moe_forward_timed(C.byref(cfg), C.byref(w), x.data_ptr(), n, y.data_ptr(), ws.data_ptr(),
                                          ws.numel(), ops.stream_ptr(stream), ms))
        return y, list(ms)

    def forward_host(self, x_host: torch.Tensor, y_host: torch.Tensor, stream=None) -> torch.Tensor:
        """Host-resident bf16 activations in and out (pinned memory recommended):
        H2D copy, the block, D2H copy and a stream sync inside one ABI call."""
        n = x_host.numel() // self.hidden
        dev = self.gate.weight.device
        ws = self._ws(n, dev, host_io=True)
        cfg, w = self.config(), self.weights()
        check(lib().imx_moe_forward_host(C.byref(cfg), C.byref(w), x_host.data_ptr(), n, y_host.data_ptr(),
                                         ws.data_ptr(), ws.numel(), ops.stream_ptr(stream)))
        return y_host

    def check_status(self, stream=None) -> None:
        if self._workspace is not None:
            check(lib().imx_moe_status(self._workspace.data_ptr(), ops.stream_ptr(stream)))

    def saturations(self, stream=None) -> int:
        """Values the expert kernels had to clamp to the fp16 range since the last call (0: none)."""
        if self._workspace is None:
            return 0
        n = C.c_longlong(0)
        check(lib().imx_moe_saturations(self._workspace.data_ptr(), ops.stream_ptr(stream), C.byref(n)))
        return int(n.value)


class CapturedForward:
    """CUDA-graph replay of `MoEMLP.forward_with_stream` on static buffers:
    write the step's activations into `x` (or pass them to `__call__`, which
    copies), call, read `y`.  The graph holds the block's workspace, so one
    instance serves one stream of steps at a time."""

    def __init__(self, moe: "MoEMLP", x: torch.Tensor, x_host: Optional[torch.Tensor] = None,
                 y_host: Optional[torch.Tensor] = None):
        self.moe = moe
        self.x = x.contiguous().clone()
        self.x_host, self.y_host = x_host, y_host
        for h in (x_host, y_host):
            if h is not None and not h.is_pinned():
                raise IronMLXError(_lib.ERR_INVALID, "capture: host buffers must be pinned memory")
        side = torch.cuda.Stream(device=x.device)
        side.wait_stream(torch.cuda.current_stream(x.device))
        with torch.cuda.stream(side):                    # warm up off the capture: attributes, workspace
            for _ in range(2):
                moe.forward_with_stream(self.x)
        torch.cuda.current_stream(x.device).wait_stream(side)
        torch.cuda.synchronize(x.device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            if x_host is not None:
                self.x.copy_(x_host.view_as(self.x), non_blocking=True)
            self.y = moe.forward_with_stream(self.x)
            if y_host is not None:
                y_host.view_as(self.y).copy_(self.y, non_blocking=True)

    def __call__(self, x: Optional[torch.Tensor] = None) -> torch.Tensor:
        if x is not None and x.data_ptr() != self.x.data_ptr():
            self.x.copy_(x, non_blocking=True)
        self.graph.replay()
        return self.y

    def run_host(self) -> torch.Tensor:
        """Host buffers in, host buffers out: one replay (copy in, block, copy out) and a stream sync."""
        if self.x_host is None or self.y_host is None:
            raise IronMLXError(_lib.ERR_INVALID, "capture: no host buffers were given")
        self.graph.replay()
        torch.cuda.current_stream(self.x.device).synchronize()
        return self.y_host


@dataclass
class FusedExperts:
    """All routed experts as the two fused checkpoint tensors:
    gate_up [E, 2I, .] (gate rows first) and down [E, H, .]
    (mlx/src/model/qwen35.rs:581-590)."""
    gate_up: QuantizedLinear
    down: QuantizedLinear

    @classmethod
    def from_experts(cls, experts: Sequence[Expert]) -> "FusedExperts":
        if len(experts) == 0:
            raise IronMLXError(_lib.ERR_INVALID, "MoEMLP needs at least one expert")
        e0 = experts[0]
        q = e0.gate_proj
        for e in experts:
            for name, ref in (("gate_proj", e0.gate_proj), ("up_proj", e0.gate_proj), ("down_proj", e0.down_proj)):
                p = getattr(e, name)
                if (p.mode, p.bits, p.group_size) != (q.mode, q.bits, q.group_size):
                    raise IronMLXError(_lib.ERR_INVALID, "experts to be fused must share one quantization format")
                if p.mode == "nvfp4" and (p.global_scale or 1.0) != (ref.global_scale or 1.0):
                    raise IronMLXError(_lib.ERR_INVALID,
                                       "experts to be fused carry different nvfp4 tensor scales: quantize the stacked "
                                       "tensor against one scale (the fused kernels take one per tensor)")

        def fuse(get):
            parts = [get(e) for e in experts]
            return _stack_or_view(parts)

        def gu(attr):
            # per expert, gate rows then up rows; a view when they are adjacent slices
            rows = []
            for e in experts:
                g, u = getattr(e.gate_proj, attr), getattr(e.up_proj, attr)
                if g is None:
                    return None
                step = g.numel() * g.element_size()
                if g.is_contiguous() and u.is_contiguous() and u.data_ptr() == g.data_ptr() + step:
                    rows.append(g.as_strided((2 * g.shape[0],) + tuple(g.shape[1:]), g.stride()))
                else:
                    rows.append(torch.cat([g, u], 0))
            return _stack_or_view(rows)

        gate_up = QuantizedLinear(gu("weight"), gu("scales"), gu("biases"), q.group_size, q.bits, q.mode,
                                  q.global_scale)
        d = e0.down_proj
        down = QuantizedLinear(fuse(lambda e: e.down_proj.weight), fuse(lambda e: e.down_proj.scales),
                               None if d.biases is None else fuse(lambda e: e.down_proj.biases),
                               d.group_size, d.bits, d.mode, d.global_scale)
        return cls(gate_up, down)

    def expert(self, e: int) -> Expert:
        """Expert e as sliced views, the way `build_moe_experts` hands them out."""
        gu, dn = self.gate_up, self.down
        i = gu.weight.shape[1] // 2

        def sl(q: QuantizedLinear, rows) -> QuantizedLinear:
            return QuantizedLinear(q.weight[e][rows], q.scales[e][rows],
                                   None if q.biases is None else q.biases[e][rows],
                                   q.group_size, q.bits, q.mode, q.global_scale)

        return Expert(sl(gu, slice(0, i)), sl(gu, slice(i, 2 * i)), sl(dn, slice(None)))
