"""Weight ingestion for the MoE block: reads a checkpoint directory the way the
reference does (mlx/src/model/loader.rs:13-45: every `*.safetensors` file in
name order into one key -> tensor map) and builds the block of one decoder
layer from the keys `Qwen35Model::from_config_file` consumes
(mlx/src/model/qwen35.rs:498-522 for the router, shared expert and its gate;
`build_moe_experts`, qwen35.rs:592-779, for the fused expert tensors):

    [language_model.model.]layers.{i}.mlp.gate.weight                         [E, H]      bf16
    ...layers.{i}.mlp.experts.gate_up_proj.{weight,scales,biases}             [E, 2I, H*b/32] u32, [E, 2I, H/g]
    ...layers.{i}.mlp.experts.down_proj.{weight,scales,biases}                [E, H, I*b/32]  u32, [E, H, I/g]
    ...layers.{i}.mlp.shared_expert.{gate_proj,up_proj,down_proj}.{weight,scales,biases}
    ...layers.{i}.mlp.shared_expert_gate.weight                               [1, H]      bf16

The packed tensors are used in place (the kernels read the checkpoint layout), so
"repacking" is only needed for checkpoints whose experts are dense
(`gate_up_proj` [E, 2I, H] without `.scales`, the fallback of qwen35.rs:780-843):
those are quantized once on the device with the library's `quantize` and the
result is kept in a cache directory keyed by the source tensors' bytes.

No checkpoint ships with this repository: the parity fixture under tests/golden
is written by tests/golden/make_checkpoint.py with the CPU checker's quantizer.
"""
from __future__ import annotations

import hashlib
import json
import os
from dataclasses import dataclass
from typing import Dict, Optional

import torch

from . import _lib, nn, ops
from ._lib import IronMLXError


@dataclass
class MoELayerConfig:
    """The fields of the reference's config the block reads (mlx/src/model/config.rs:32-52,159-170), with its
    defaults (qwen35.rs:491-496)."""
    hidden_size: int
    num_experts: int
    num_experts_per_tok: int = 8
    moe_intermediate_size: int = 0
    shared_expert_intermediate_size: int = 0
    norm_topk_prob: bool = True
    group_size: int = 64
    bits: int = 4
    mode: str = "affine"


def read_config(directory: str) -> MoELayerConfig:
    """config.json of a checkpoint directory (the text model's fields may sit under `text_config`)."""
    with open(os.path.join(directory, "config.json")) as f:
        raw = json.load(f)
    tc = raw.get("text_config", raw)
    q = raw.get("quantization", raw.get("quantization_config", tc.get("quantization", {}))) or {}
    if "num_experts" not in tc:
        raise IronMLXError(_lib.ERR_INVALID, "config.json: not a mixture-of-experts model (no num_experts)")
    inter = tc.get("moe_intermediate_size") or tc.get("intermediate_size")
    return MoELayerConfig(
        hidden_size=int(tc["hidden_size"]), num_experts=int(tc["num_experts"]),
        num_experts_per_tok=int(tc.get("num_experts_per_tok") or 8), moe_intermediate_size=int(inter),
        shared_expert_intermediate_size=int(tc.get("shared_expert_intermediate_size") or inter),
        norm_topk_prob=bool(tc.get("norm_topk_prob", True)), group_size=int(q.get("group_size", 64)),
        bits=int(q.get("bits", 4)), mode=str(q.get("mode", "affine")))


def load_model_weights(directory: str, device="cpu") -> Dict[str, torch.Tensor]:
    """All `*.safetensors` files of a directory, in file-name order, as one map (later files win, as in the
    reference's loader)."""
    from safetensors.torch import load_file
    files = sorted(f for f in os.listdir(directory) if f.endswith(".safetensors"))
    if not files:
        raise IronMLXError(_lib.ERR_INVALID, "no .safetensors files found")
    out: Dict[str, torch.Tensor] = {}
    for name in files:
        out.update(load_file(os.path.join(directory, name), device=str(device)))
    return out


def _get(weights, name: str) -> Optional[torch.Tensor]:
    """The reference tries the `language_model.model.` prefix first, then the bare key (qwen35.rs:347-361)."""
    t = weights.get("language_model.model." + name)
    return t if t is not None else weights.get(name)


def _need(weights, name: str) -> torch.Tensor:
    t = _get(weights, name)
    if t is None:
        raise IronMLXError(_lib.ERR_INVALID, f"missing weight: {name} (tried prefixed: language_model.model.{name})")
    return t


def _packed(t: torch.Tensor, device) -> torch.Tensor:
    """MLX stores packed codes as uint32: the same bits as int32 for the kernels."""
    if t.dtype not in (torch.uint32, torch.int32):
        raise IronMLXError(_lib.ERR_INVALID, f"packed weight has dtype {t.dtype}, expected uint32")
    return t.contiguous().view(torch.int32).to(device)


def _scales(t: torch.Tensor, mode: str, device) -> torch.Tensor:
    if mode == "affine":
        # affine scales and biases are consumed as bf16 (what 4-bit mlx-community checkpoints of bf16 models hold);
        # float16 ones are converted, which rounds them to 8 significant bits
        return t.to(torch.bfloat16).contiguous().to(device)
    if t.dtype != torch.uint8:
        raise IronMLXError(_lib.ERR_INVALID, f"{mode} scales have dtype {t.dtype}, expected uint8")
    return t.contiguous().to(device)


def _quantized_linear(weights, prefix: str, cfg: MoELayerConfig, device, cache: Optional["RepackCache"]):
    """`LinearLayer::from_weights` (mlx/src/nn/linear.rs:97-126): quantized when `<prefix>.scales` exists."""
    w = _need(weights, prefix + ".weight")
    s = _get(weights, prefix + ".scales")
    if s is None:
        if cache is None:
            raise IronMLXError(_lib.ERR_INVALID,
                               f"{prefix}: dense weights; pass a RepackCache to quantize them once on the device")
        return cache.quantized(prefix, w, cfg, device)
    b = _get(weights, prefix + ".biases")
    if cfg.mode == "affine" and b is None:
        raise IronMLXError(_lib.ERR_INVALID, f"missing weight: {prefix}.biases")
    gs = _get(weights, prefix + ".global_scale")
    return nn.QuantizedLinear(_packed(w, device), _scales(s, cfg.mode, device),
                              None if b is None else _scales(b, cfg.mode, device), cfg.group_size, cfg.bits, cfg.mode,
                              None if gs is None else float(gs.float().item()))


class RepackCache:
    """Quantized copies of dense expert tensors, made once with the device `quantize` op and kept as safetensors
    files in `directory`, keyed by a digest of the source bytes and the target format."""

    def __init__(self, directory: str):
        self.directory = directory
        os.makedirs(directory, exist_ok=True)

    def _path(self, w: torch.Tensor, cfg: MoELayerConfig) -> str:
        h = hashlib.sha256()
        h.update(f"{tuple(w.shape)}|{w.dtype}|{cfg.mode}|{cfg.bits}|{cfg.group_size}".encode())
        flat = w.detach().contiguous().view(torch.uint8).reshape(-1).cpu()
        step = max(1, flat.numel() // (1 << 22))               # a strided sample of at most ~4 M bytes plus the ends
        h.update(flat[::step].numpy().tobytes())
        h.update(flat[-4096:].numpy().tobytes())
        return os.path.join(self.directory, h.hexdigest()[:32] + ".safetensors")

    def quantized(self, name: str, w: torch.Tensor, cfg: MoELayerConfig, device) -> nn.QuantizedLinear:
        from safetensors.torch import load_file, save_file
        path = self._path(w, cfg)
        if os.path.exists(path):
            t = load_file(path, device=str(device))
            gs = t.get("global_scale")
            return nn.QuantizedLinear(t["weight"].view(torch.int32), t["scales"], t.get("biases"), cfg.group_size, cfg.bits,
                                      cfg.mode, None if gs is None else float(gs.item()))
        out = ops.quantize(w.to(device).float(), cfg.group_size, cfg.bits, cfg.mode)
        q = nn.QuantizedLinear(out[0], out[1], out[2], cfg.group_size, cfg.bits, cfg.mode, out[3] if len(out) > 3 else None)
        t = {"weight": q.weight.view(torch.uint32).cpu(), "scales": q.scales.cpu()}
        if q.biases is not None:
            t["biases"] = q.biases.cpu()
        if q.global_scale is not None:
            t["global_scale"] = torch.tensor([q.global_scale], dtype=torch.float32)
        save_file(t, path, metadata={"source": name})
        return q


def moe_layer_from_weights(weights: Dict[str, torch.Tensor], layer: int, cfg: MoELayerConfig, device="cuda",
                           path: str = "auto", cache: Optional[RepackCache] = None) -> nn.MoEMLP:
    """The MoE block of decoder layer `layer` (the `Qwen35MLP::MoE` arm of qwen35.rs:489-531)."""
    lp = f"layers.{layer}"
    gate = nn.Linear(_need(weights, f"{lp}.mlp.gate.weight").to(torch.bfloat16).contiguous().to(device))
    gate_up = _quantized_linear(weights, f"{lp}.mlp.experts.gate_up_proj", cfg, device, cache)
    down = _quantized_linear(weights, f"{lp}.mlp.experts.down_proj", cfg, device, cache)
    e, two_i = gate_up.weight.shape[0], gate_up.weight.shape[1]
    if e != cfg.num_experts or two_i != 2 * cfg.moe_intermediate_size:
        raise IronMLXError(_lib.ERR_INVALID,
                           f"{lp}: experts.gate_up_proj is {tuple(gate_up.weight.shape)}, the config says {cfg.num_experts} "
                           f"experts of intermediate size {cfg.moe_intermediate_size}")
    if tuple(down.weight.shape[:2]) != (e, cfg.hidden_size):
        raise IronMLXError(_lib.ERR_INVALID, f"{lp}: experts.down_proj is {tuple(down.weight.shape)}")
    shared = shared_gate = None
    if _get(weights, f"{lp}.mlp.shared_expert.gate_proj.weight") is not None:
        shared = nn.MLP(*(_quantized_linear(weights, f"{lp}.mlp.shared_expert.{n}", cfg, device, cache)
                          for n in ("gate_proj", "up_proj", "down_proj")))
        shared_gate = nn.Linear(_need(weights, f"{lp}.mlp.shared_expert_gate.weight").to(torch.bfloat16).contiguous().to(device))
    return nn.MoEMLP(gate, nn.FusedExperts(gate_up, down), shared, shared_gate, cfg.num_experts_per_tok, cfg.norm_topk_prob,
                     None, path)


def load_moe_layer(directory: str, layer: int, device="cuda", path: str = "auto",
                   cache: Optional[RepackCache] = None) -> nn.MoEMLP:
    """config.json + safetensors of `directory` -> the MoE block of one decoder layer on `device`."""
    cfg = read_config(directory)
    weights = load_model_weights(directory, "cpu")
    return moe_layer_from_weights(weights, layer, cfg, device, path, cache)
