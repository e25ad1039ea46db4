"""The layer calls of the path on the GPU against the CPU checker: `QuantizedLinear`, `Expert`, `MLP` and dense
`Linear` `forward_with_stream` (mlx/src/nn/linear.rs:51-63,170-177, mlx/src/nn/moe.rs:26-32,
mlx/src/nn/mlp.rs:27-33), each one call into the C ABI."""
import numpy as np
import pytest
import torch

from ironmlx_b200 import _lib, nn
from ironmlx_b200.workloads import MoEConfig, Workload, normal, round_bf16
from oracle import formats as F
from oracle import moe as O
from gpu_util import bf16_to_np, q_to_device, t_bf16
from util import quantize_stack, squeeze0

pytestmark = pytest.mark.gpu
TOL = 2e-3


def _qlinear(out_dim, in_dim, mode, bits, group, seed):
    cfg = MoEConfig("l", 1, in_dim, 1, 1, out_dim, mode=mode, bits=bits, group_size=group, seed=seed)
    w = round_bf16(normal(seed, "w", (out_dim, in_dim), 0.02))
    return squeeze0(quantize_stack([w], cfg))


@pytest.mark.parametrize("mode,bits,group", [("affine", 4, 64), ("affine", 8, 64), ("affine", 2, 64), ("mxfp8", 8, 32),
                                             ("nvfp4", 4, 16)])
@pytest.mark.parametrize("m,in_dim,out_dim", [(1, 2048, 512), (8, 512, 2048), (40, 1024, 1024), (300, 2048, 512),
                                              (70, 512, 20480),        # a vocabulary-sized output on the tensor-core kernel
                                              (5, 192, 320)])          # the last shape: the scalar fallback
def test_quantized_linear_forward(cuda, m, in_dim, out_dim, mode, bits, group):
    if in_dim % group:
        pytest.skip("input dimension not a multiple of the group size")
    q = _qlinear(out_dim, in_dim, mode, bits, group, seed=7)
    x = round_bf16(normal(8, "x", (m, in_dim)))
    ref = F.quantized_matmul(x, q.w, q.scales, q.biases, True, group, bits, mode, global_scale=q.global_scale)
    ql = q_to_device(q, cuda)
    y = bf16_to_np(ql.forward_with_stream(t_bf16(x, cuda)))
    assert y.shape == (m, out_dim)
    assert O.rel_l2(y, ref) <= TOL


@pytest.mark.parametrize("mode,bits,group", [("affine", 4, 64), ("mxfp8", 8, 32)])
@pytest.mark.parametrize("m", [3, 70, 400])
def test_expert_and_mlp_forward(cuda, m, mode, bits, group):
    cfg = MoEConfig("e", m, 1024, 2, 1, 512, 512, mode=mode, bits=bits, group_size=group, seed=11)
    from util import make_params
    x, p = make_params(cfg)
    from gpu_util import moe_to_device
    moe = moe_to_device(p, cuda)
    xd = t_bf16(x, cuda)
    # a routed expert: views into the fused tensors (gate and up rows adjacent)
    e1 = moe._fused.expert(1)
    wg, wu, wd = O.expert_weights(p, 1)
    ref = O.swiglu_mlp(x, wg, wu, wd)
    y = bf16_to_np(e1.forward_with_stream(xd))
    assert O.rel_l2(y, ref) <= TOL
    # the shared expert: three separate tensors
    sg = F.dequantize(p.shared_gate_proj.w, p.shared_gate_proj.scales, p.shared_gate_proj.biases, group, bits, mode,
                      p.shared_gate_proj.global_scale)
    su = F.dequantize(p.shared_up_proj.w, p.shared_up_proj.scales, p.shared_up_proj.biases, group, bits, mode,
                      p.shared_up_proj.global_scale)
    sd = F.dequantize(p.shared_down_proj.w, p.shared_down_proj.scales, p.shared_down_proj.biases, group, bits, mode,
                      p.shared_down_proj.global_scale)
    ref_s = O.swiglu_mlp(x, sg, su, sd)
    ys = bf16_to_np(moe.shared_expert.forward_with_stream(xd))
    assert O.rel_l2(ys, ref_s) <= TOL


@pytest.mark.parametrize("m,in_dim,out_dim,bias", [(1, 2048, 256, False), (70, 512, 1, False), (130, 256, 100, True)])
def test_dense_linear_forward(cuda, m, in_dim, out_dim, bias):
    w = round_bf16(normal(3, "w", (out_dim, in_dim), 0.05))
    b = round_bf16(normal(3, "b", (out_dim,), 0.1)) if bias else None
    x = round_bf16(normal(4, "x", (m, in_dim)))
    ref = x.astype(np.float64) @ w.astype(np.float64).T + (0 if b is None else b.astype(np.float64))
    lin = nn.Linear(t_bf16(w, cuda), None if b is None else t_bf16(b, cuda))
    y = bf16_to_np(lin.forward_with_stream(t_bf16(x, cuda)))
    assert y.shape == (m, out_dim)
    assert O.rel_l2(y, ref) <= TOL
    assert np.abs(y - ref).max() <= 2.0 ** -7 * np.abs(ref).max() + 1e-6


def test_fusing_experts_with_different_tensor_scales_is_refused(cuda):
    q = _qlinear(128, 128, "nvfp4", 4, 16, seed=2)
    a = q_to_device(q, cuda)
    b = q_to_device(q, cuda)
    b.global_scale = (a.global_scale or 1.0) * 2
    with pytest.raises(_lib.IronMLXError):
        nn.FusedExperts.from_experts([nn.Expert(a, a, a), nn.Expert(b, b, b)])
