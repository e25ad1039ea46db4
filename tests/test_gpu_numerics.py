"""Numerics at the edges of the fp16 carriers, and the failure path of a bounded device wait.

Real residual streams have outlier channels; the expert kernels carry activations and intermediate rows in
fp16 and clamp beyond +-65504.  These tests put outlier channels (+-50 .. +-500), small tokens, values near
2^-14 and a deliberately overflowing case through every expert path, and require that the tolerance still holds
and that a clamp is counted, never silent.  (The block's input is the output of the layer's RMSNorm,
mlx/src/model/qwen35.rs:271-273: token rows of unit scale.  Whole rows many octaves below that would underflow
the fp16 SwiGLU rows; that is outside what the path is fed and is not tested as supported.)"""
import numpy as np
import pytest
import torch

from ironmlx_b200 import _lib
from ironmlx_b200.workloads import MoEConfig, round_bf16
from oracle import moe as O
from gpu_util import bf16_to_np, moe_to_device, t_bf16
from util import make_params

pytestmark = pytest.mark.gpu
TOL = 2e-3


def outlier_case(cfg, seed):
    x, p = make_params(cfg)
    rng = np.random.default_rng(seed)
    x = x.copy()
    ch = rng.choice(cfg.hidden, 6, replace=False)
    x[:, ch[:4]] *= rng.choice([50.0, -80.0, 120.0, -200.0], 4)          # a few massive channels in every token
    x[:, ch[4:]] *= 500.0
    x[::5] *= 2.0 ** -4                                                  # every fifth token small as a whole
    tiny = rng.random(x.shape) < 0.05                                    # and values at the bottom of fp16's normal
    x[tiny] = np.sign(x[tiny]) * 2.0 ** -14 * (1 + rng.random(int(tiny.sum())))   # range sprinkled everywhere
    return round_bf16(x), p


@pytest.mark.parametrize("path", ["decode", "prefill", "generic"])
@pytest.mark.parametrize("mode,bits,group", [("affine", 4, 64), ("mxfp8", 8, 32)])
def test_outlier_channels_and_tiny_tokens(cuda, path, mode, bits, group):
    cfg = MoEConfig("outliers", tokens=90, hidden=1024, num_experts=8, top_k=2, intermediate=512, shared_intermediate=512,
                    mode=mode, bits=bits, group_size=group, seed=91)
    x, p = outlier_case(cfg, 1)
    ref = O.moe_forward(x, p)
    moe = moe_to_device(p, cuda, path)
    y = bf16_to_np(moe.forward_with_stream(t_bf16(x, cuda)))
    torch.cuda.synchronize()
    moe.check_status()
    assert moe.saturations() == 0
    assert O.rel_l2(y, ref.y) <= TOL
    # token by token as well: a small token must not drown in a norm taken over the large ones
    num = np.linalg.norm(y - ref.y, axis=1)
    den = np.linalg.norm(ref.y, axis=1)
    assert np.all(num <= 3 * TOL * den + 1e-30)


@pytest.mark.parametrize("path", ["decode", "prefill", "generic"])
def test_a_clamp_is_counted(cuda, path):
    """Expert weights large enough that SwiGLU outputs leave the fp16 range: the kernels clamp, and say so."""
    cfg = MoEConfig("overflow", tokens=40, hidden=512, num_experts=4, top_k=2, intermediate=512, shared_intermediate=0, seed=92)
    x, p = make_params(cfg)
    x = round_bf16(x * 300.0)
    # scale the gate/up weights up through their group scales and biases (bf16 values times a power of two stay exact)
    p.gate_up.scales = (p.gate_up.scales.astype(np.float32) * 64).astype(p.gate_up.scales.dtype)
    p.gate_up.biases = (p.gate_up.biases.astype(np.float32) * 64).astype(p.gate_up.biases.dtype)
    moe = moe_to_device(p, cuda, path)
    moe.forward_with_stream(t_bf16(x, cuda))
    torch.cuda.synchronize()
    moe.check_status()
    assert moe.saturations() > 0
    assert moe.saturations() == 0                       # reading clears the count


def test_expired_handoff_wait_is_reported_and_the_gpu_stays_usable(cuda):
    """A bounded wait that runs out (the partial-sum flags of the decode kernels withheld by a test hook, the spin
    limit cut to 200 iterations): the kernels return, the status word says so, and the next call on the same
    workspace is correct."""
    cfg = MoEConfig("handoff", tokens=24, hidden=512, num_experts=8, top_k=2, intermediate=512, shared_intermediate=512, seed=93)
    x, p = make_params(cfg)
    ref = O.moe_forward(x, p)
    moe = moe_to_device(p, cuda, "decode")
    xd = t_bf16(x, cuda)
    good = moe.forward_with_stream(xd).clone()
    torch.cuda.synchronize()
    moe.check_status()
    lib = _lib.lib()
    try:
        lib.imx_testing_decode_handoff(200, 1)
        moe.forward_with_stream(xd)
        torch.cuda.synchronize()
        with pytest.raises(_lib.IronMLXError) as e:
            moe.check_status()
        assert e.value.code == _lib.ERR_DEVICE and "status 2" in str(e.value)
    finally:
        lib.imx_testing_decode_handoff(0, 0)
    again = moe.forward_with_stream(xd)
    torch.cuda.synchronize()
    moe.check_status()                                   # the status word was cleared when it was read
    assert torch.equal(again, good)
    assert O.rel_l2(bf16_to_np(again), ref.y) <= TOL
