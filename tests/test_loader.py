"""Checkpoint ingestion (mlx/src/model/loader.rs:13-45, mlx/src/model/qwen35.rs:498-522,592-779): the
synthetic fixture under tests/golden/checkpoint (written by tests/golden/make_checkpoint.py) is read key by
key on the CPU; on a GPU the loaded block must reproduce the checker's output for the fixture's input."""
import os
import shutil

import numpy as np
import pytest
import torch

from ironmlx_b200 import _lib, loader
from oracle import formats as F
from oracle import moe as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CKPT = os.path.join(GOLDEN, "checkpoint")
REAL = os.path.join(GOLDEN, "mlx_real")


def test_config_and_keys_are_read_like_the_reference():
    cfg = loader.read_config(CKPT)
    assert (cfg.hidden_size, cfg.num_experts, cfg.num_experts_per_tok, cfg.moe_intermediate_size) == (256, 4, 2, 128)
    assert (cfg.group_size, cfg.bits, cfg.mode, cfg.norm_topk_prob) == (64, 4, "affine", True)
    w = loader.load_model_weights(CKPT)
    exp = np.load(os.path.join(CKPT, "expected.npz"))
    moe = loader.moe_layer_from_weights(w, int(exp["layer"]), cfg, device="cpu")
    assert moe.num_experts == 4 and moe.hidden == 256 and moe.intermediate == 128 and moe.shared_intermediate == 128
    gu = moe._fused.gate_up
    assert gu.weight.dtype == torch.int32 and tuple(gu.weight.shape) == (4, 256, 32)
    assert gu.scales.dtype == torch.bfloat16 and tuple(gu.scales.shape) == (4, 256, 4)
    # the packed bytes are the fixture's, untouched: dequantizing them with the checker gives bf16-exact weights
    wq = F.dequantize(gu.weight.numpy().view(np.uint32), gu.scales.view(torch.int16).numpy().view(F.bf16),
                      gu.biases.view(torch.int16).numpy().view(F.bf16), 64, 4, "affine")
    assert wq.shape == (4, 256, 256) and np.isfinite(wq).all()


def test_missing_keys_and_dense_experts_are_reported(tmp_path):
    cfg = loader.read_config(CKPT)
    w = loader.load_model_weights(CKPT)
    with pytest.raises(_lib.IronMLXError, match="missing weight"):
        loader.moe_layer_from_weights(w, 0, cfg, device="cpu")             # the fixture holds layer 3 only
    bare = {k.replace("language_model.model.", ""): v for k, v in w.items()}
    assert loader.moe_layer_from_weights(bare, 3, cfg, device="cpu").num_experts == 4     # un-prefixed keys are accepted
    dense = dict(w)
    for k in list(dense):
        if "experts.gate_up_proj" in k and not k.endswith(".weight"):
            del dense[k]
    with pytest.raises(_lib.IronMLXError, match="dense"):
        loader.moe_layer_from_weights(dense, 3, cfg, device="cpu")
    d = tmp_path / "empty"
    d.mkdir()
    with pytest.raises(_lib.IronMLXError):
        loader.load_model_weights(str(d))
    shutil.copy(os.path.join(CKPT, "config.json"), d / "config.json")
    assert loader.read_config(str(d)).num_experts == 4


@pytest.mark.gpu
def test_loaded_layer_reproduces_the_checker(cuda):
    exp = np.load(os.path.join(CKPT, "expected.npz"))
    moe = loader.load_moe_layer(CKPT, int(exp["layer"]), cuda)
    x = torch.from_numpy(exp["x"]).to(cuda).to(torch.bfloat16)
    y, tr = moe.forward_with_stream(x, trace=True)
    torch.cuda.synchronize()
    moe.check_status()
    assert np.array_equal(tr["topk_idx"].cpu().numpy(), exp["top_idx"]) and np.array_equal(tr["perm"].cpu().numpy(), exp["perm"])
    assert O.rel_l2(y.float().cpu().numpy(), exp["y"]) <= 2e-3


@pytest.mark.gpu
def test_dense_experts_are_quantized_once_through_the_cache(cuda, tmp_path):
    """Dense expert tensors (the fallback of qwen35.rs:780-843): quantized on the device, kept in the cache, and
    read back from it on the second load."""
    cfg = loader.read_config(CKPT)
    w = loader.load_model_weights(CKPT)
    pre = "language_model.model.layers.3.mlp.experts."
    dense = dict(w)
    for proj in ("gate_up_proj", "down_proj"):
        q = (w[pre + proj + ".weight"], w[pre + proj + ".scales"], w[pre + proj + ".biases"])
        full = F.dequantize(q[0].numpy().view(np.uint32), q[1].view(torch.int16).numpy().view(F.bf16),
                            q[2].view(torch.int16).numpy().view(F.bf16), 64, 4, "affine")
        dense[pre + proj + ".weight"] = torch.from_numpy(full).to(torch.bfloat16)
        del dense[pre + proj + ".scales"], dense[pre + proj + ".biases"]
    cache = loader.RepackCache(str(tmp_path / "cache"))
    exp = np.load(os.path.join(CKPT, "expected.npz"))
    x = torch.from_numpy(exp["x"]).to(cuda).to(torch.bfloat16)
    ys = []
    for _ in range(2):
        moe = loader.moe_layer_from_weights(dense, 3, cfg, cuda, cache=cache)
        ys.append(moe.forward_with_stream(x).float().cpu().numpy())
    assert len(os.listdir(cache.directory)) == 2 and np.array_equal(ys[0], ys[1])
    # against the checker on the very tensors the cache holds (the dense weights were rounded to bf16 and quantized
    # anew, so the fixture's expected output is only a coarse guide: 4-bit noise)
    from gpu_util import params_from_device
    ref = O.moe_forward(exp["x"], params_from_device(moe, cfg.num_experts_per_tok, cfg.norm_topk_prob))
    assert O.rel_l2(ys[0], ref.y) <= 2e-3
    assert O.rel_l2(ys[0], exp["y"]) <= 0.15


@pytest.mark.skipif(not os.path.exists(os.path.join(REAL, "dequantized.npz")),
                    reason="no real mlx-community shard under tests/golden/mlx_real (see its README)")
def test_real_checkpoint_bit_order():
    """Closes the one open question of the format restatement: with one `*.safetensors` shard of an mlx-community
    quantized checkpoint and `mx.dequantize` outputs for some of its tensors in dequantized.npz
    (name -> float32 array), the checker's `dequantize` must reproduce MLX's values exactly."""
    w = loader.load_model_weights(REAL)
    ref = np.load(os.path.join(REAL, "dequantized.npz"))
    cfg = loader.read_config(REAL)
    checked = 0
    for name in ref.files:
        wq, s, b = w[name + ".weight"], w[name + ".scales"], w.get(name + ".biases")
        f16 = lambda t: t.float().numpy().astype(F.bf16) if t.dtype != torch.bfloat16 else t.view(torch.int16).numpy().view(F.bf16)
        got = F.dequantize(wq.contiguous().view(torch.int32).numpy().view(np.uint32), f16(s) if cfg.mode == "affine" else s.numpy(),
                           None if b is None else f16(b), cfg.group_size, cfg.bits, cfg.mode)
        assert np.array_equal(got.astype(np.float32), ref[name].astype(np.float32)), name
        checked += 1
    assert checked > 0
