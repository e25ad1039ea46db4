"""End-to-end parity of the MoE block on the GPU (through the C ABI) against the
CPU checker: bit-exact routing and dispatch on tie-free rows, outputs within
relative L2 2e-3 of the fp32-accumulated result."""
import os

import numpy as np
import pytest
import torch

from ironmlx_b200 import _lib, nn
from ironmlx_b200.workloads import CONFIGS, MoEConfig
from oracle import formats as F
from oracle import moe as O
from gpu_util import bf16_to_np, moe_to_device, params_from_device, t_bf16
from test_gpu_stages import FORMATS, check_routing
from util import SMALL, TINY, make_params

pytestmark = pytest.mark.gpu
TOL = 2e-3          # relative L2 of the bf16 output against the fp32-accumulated checker
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def run(cfg, dev, path="auto", x=None, p=None):
    if p is None:
        x, p = make_params(cfg)
    moe = moe_to_device(p, dev, path)
    y, tr = moe.forward_with_stream(t_bf16(x, dev), trace=True)
    torch.cuda.synchronize()
    moe.check_status()
    return x, p, moe, bf16_to_np(y), {k: v.cpu().numpy() for k, v in tr.items()}


def compare(cfg, x, p, y, tr, fast=False):
    ref = O.moe_forward(x, p, fast_bucket=fast)
    k = cfg.top_k
    clear = check_routing(tr["topk_idx"], tr["topk_w"], x, p, k, cfg.norm_topk_prob, p.router_logit_bias)
    if clear.all():
        assert np.array_equal(tr["counts"], ref.counts) and np.array_equal(tr["offsets"], ref.offsets)
        assert np.array_equal(tr["perm"], ref.perm) and np.array_equal(tr["inv_perm"], ref.inv_perm)
    else:   # the permutation of the GPU's own routing must still be the stable sort
        c, o, pm, inv = O.bucket_fast(tr["topk_idx"], cfg.num_experts)
        assert np.array_equal(tr["perm"], pm) and np.array_equal(tr["offsets"], o)
    err = O.rel_l2(y[clear], ref.y[clear])
    assert err <= TOL, f"{cfg.name}: rel-L2 {err:.3e} > {TOL}"
    assert np.abs(y[clear] - ref.y[clear]).max() <= 2 ** -7 * np.abs(ref.y).max() + 1e-6
    return err


@pytest.mark.parametrize("path", ["generic", "decode", "decode_regs"])
@pytest.mark.parametrize("cfg", [TINY, SMALL, CONFIGS["c1"]], ids=lambda c: c.name)
def test_block_affine4(cuda, cfg, path):
    x, p, _, y, tr = run(cfg, cuda, path)
    compare(cfg, x, p, y, tr)


def test_c1_against_golden_fixture(cuda):
    cfg = CONFIGS["c1"]
    g = np.load(os.path.join(GOLDEN, "c1.npz"))
    x, p, _, y, tr = run(cfg, cuda)
    assert np.array_equal(tr["topk_idx"], g["top_idx"]) and np.array_equal(tr["perm"], g["perm"])
    assert np.array_equal(tr["counts"], g["counts"])
    assert O.rel_l2(y, g["y"]) <= TOL


@pytest.mark.parametrize("mode,bits,group", FORMATS)
def test_block_every_format(cuda, mode, bits, group):
    cfg = SMALL.with_(name=f"small-{mode}{bits}g{group}", mode=mode, bits=bits, group_size=group)
    x, p, _, y, tr = run(cfg, cuda)
    compare(cfg, x, p, y, tr)
    name = f"tiny_{mode}{bits}_g{group}.npz"
    if os.path.exists(os.path.join(GOLDEN, name)):
        g = np.load(os.path.join(GOLDEN, name))
        tcfg = TINY.with_(mode=mode, bits=bits, group_size=group)
        _, _, _, ty, ttr = run(tcfg, cuda)
        assert np.array_equal(ttr["perm"], g["perm"]) and O.rel_l2(ty, g["y"]) <= TOL


@pytest.mark.parametrize("bits,group", [(2, 64), (4, 128), (8, 64), (8, 128)])
def test_decode_path_other_widths(cuda, bits, group):
    cfg = MoEConfig(f"dec{bits}g{group}", tokens=40, hidden=256, num_experts=8, top_k=3, intermediate=128,
                    shared_intermediate=256, bits=bits, group_size=group, seed=9)
    x, p, _, y, tr = run(cfg, cuda, "decode")
    compare(cfg, x, p, y, tr)
    _, _, _, yg, _ = run(cfg, cuda, "generic", x, p)
    assert O.rel_l2(y, yg) < 1e-3                        # both paths round the same fp32 sums to bf16


@pytest.mark.parametrize("cfg", [
    MoEConfig("no-norm", 9, 256, 8, 2, 128, 128, norm_topk_prob=False, seed=12),
    MoEConfig("no-shared", 17, 256, 16, 4, 128, 0, seed=13),
    MoEConfig("k-eq-e", 6, 128, 4, 4, 128, 128, seed=14),
    MoEConfig("one-token", 1, 256, 8, 2, 128, 128, seed=15),
    MoEConfig("one-expert", 5, 128, 1, 1, 128, 0, seed=16),
    MoEConfig("wide-shared", 12, 256, 8, 2, 128, 384, seed=17),
    MoEConfig("crowded", 100, 128, 2, 2, 128, 128, seed=18),      # 100 rows per expert: many units
], ids=lambda c: c.name)
@pytest.mark.parametrize("path", ["generic", "decode", "decode_regs"])
def test_block_edge_shapes(cuda, cfg, path):
    x, p, _, y, tr = run(cfg, cuda, path)
    compare(cfg, x, p, y, tr)


def test_empty_experts_and_skew(cuda):
    cfg = MoEConfig("skew", 64, 256, 32, 4, 128, 128, seed=19, zipf_s=1.2, zipf_hot_share=0.2)
    x, p = make_params(cfg)
    p.router_logit_bias[:8] = -30.0                                      # eight experts never selected
    x, p, _, y, tr = run(cfg, cuda, "decode", x, p)
    assert (tr["counts"][:8] == 0).all() and tr["counts"].max() >= 0.15 * cfg.assignments
    compare(cfg, x, p, y, tr)


def test_zero_tokens_and_errors(cuda):
    x, p = make_params(TINY)
    moe = moe_to_device(p, cuda)
    y = moe.forward_with_stream(torch.empty(0, TINY.hidden, dtype=torch.bfloat16, device=cuda))
    assert y.shape == (0, TINY.hidden)
    with pytest.raises(_lib.IronMLXError):
        moe.forward_with_stream(torch.zeros(2, TINY.hidden + 16, dtype=torch.bfloat16, device=cuda))
    with pytest.raises(_lib.IronMLXError):
        moe.forward_with_stream(torch.zeros(2, TINY.hidden, dtype=torch.float32, device=cuda))
    x3, p3 = make_params(TINY.with_(bits=3, group_size=32))
    with pytest.raises(_lib.IronMLXError):                             # 3-bit has no decode path
        moe_to_device(p3, cuda, "decode").forward_with_stream(t_bf16(x3, cuda))


def test_batch_shape_and_views(cuda):
    """[B, L, H] in and out (moe.rs:56-64,182), experts given as per-expert
    sliced views the way build_moe_experts hands them out (qwen35.rs:661-776)."""
    cfg = SMALL
    x, p = make_params(cfg)
    fused = moe_to_device(p, cuda)
    experts = [fused._fused.expert(e) for e in range(cfg.num_experts)]
    moe = nn.MoEMLP(fused.gate, experts, fused.shared_expert, fused.shared_expert_gate, cfg.top_k, True)
    assert moe._fused.gate_up.weight.data_ptr() == fused._fused.gate_up.weight.data_ptr()   # no copy
    xd = t_bf16(x, cuda).reshape(4, 12, cfg.hidden)
    y3 = moe.forward_with_stream(xd)
    y2 = fused.forward_with_stream(xd.reshape(-1, cfg.hidden))
    assert y3.shape == xd.shape and torch.equal(y3.reshape(-1, cfg.hidden), y2)


def test_reruns_are_bit_identical(cuda):
    x, p = make_params(CONFIGS["c1"])
    moe = moe_to_device(p, cuda)
    xd = t_bf16(x, cuda)
    ys = [moe.forward_with_stream(xd).clone() for _ in range(3)]
    assert torch.equal(ys[0], ys[1]) and torch.equal(ys[0], ys[2])


def test_host_io_entry_point(cuda):
    x, p = make_params(SMALL)
    moe = moe_to_device(p, cuda)
    xh = t_bf16(x, "cpu").pin_memory()
    yh = torch.empty_like(xh).pin_memory()
    moe.forward_host(xh, yh)
    yd = moe.forward_with_stream(xh.to(cuda))
    assert torch.equal(yh.to(cuda), yd)


@pytest.mark.parametrize("cfg", [
    MoEConfig("pf-tiny", 5, 512, 4, 2, 512, 512, seed=31),                       # one ragged tile per expert
    MoEConfig("pf-ragged", 300, 512, 8, 3, 512, 1024, seed=32),                  # tiles of 128 + remainders, wider shared
    MoEConfig("pf-no-shared", 200, 1024, 4, 2, 512, 0, seed=33),
    MoEConfig("pf-g128", 130, 1024, 4, 2, 1024, 1024, group_size=128, seed=34),
    MoEConfig("pf-one-expert", 150, 512, 1, 1, 512, 0, seed=35),
    MoEConfig("pf-empty-experts", 40, 512, 16, 1, 512, 512, seed=36),            # most experts get 0-3 rows
    MoEConfig("pf-no-norm", 129, 512, 4, 2, 512, 512, norm_topk_prob=False, seed=37),
], ids=lambda c: c.name)
def test_prefill_path_shapes(cuda, cfg):
    """The tensor-memory GEMM path (forced) on ragged, empty and odd expert loads; the same kernel with
    its dequantized tile in shared memory instead of tensor memory must agree with it bit for bit (same
    operands, same MMA order)."""
    x, p, _, y, tr = run(cfg, cuda, "prefill")
    compare(cfg, x, p, y, tr)
    _, _, _, yg, _ = run(cfg, cuda, "generic", x, p)
    assert O.rel_l2(y, yg) < 1.5e-3          # fp16 weights and fp16 expert rows on one side, fp32 on the other
    for other in ("prefill_plain", "prefill_smem"):
        _, _, _, ys, _ = run(cfg, cuda, other, x, p)
        assert np.array_equal(y, ys), other


PREFILL_FORMATS = [("affine", 4, 64), ("affine", 4, 32), ("affine", 4, 128), ("affine", 8, 64), ("affine", 8, 128),
                   ("affine", 2, 64), ("affine", 2, 32), ("mxfp8", 8, 32), ("nvfp4", 4, 16)]


@pytest.mark.parametrize("mode,bits,group", PREFILL_FORMATS)
def test_prefill_path_every_format(cuda, mode, bits, group):
    """Every format of the tensor-core prefill path on ragged tiles (a wider shared expert, an expert with
    more than 128 rows), against the checker and against the format-agnostic kernels."""
    inter = 512 if group < 128 else 1024              # a row of scales is whole 16-byte pieces
    cfg = MoEConfig(f"pf-{mode}{bits}g{group}", tokens=210, hidden=1024, num_experts=6, top_k=3, intermediate=inter,
                    shared_intermediate=1024, mode=mode, bits=bits, group_size=group, seed=51)
    x, p, _, y, tr = run(cfg, cuda, "prefill")
    compare(cfg, x, p, y, tr)
    _, _, _, yg, _ = run(cfg, cuda, "generic", x, p)
    assert O.rel_l2(y, yg) < 1.5e-3
    for other in ("prefill_plain", "prefill_smem"):   # same operands, same accumulation order
        _, _, _, ys, _ = run(cfg, cuda, other, x, p)
        assert np.array_equal(y, ys), other


def test_prefill_mxfp8_wide_scale_range(cuda):
    """mxfp8 weight rows whose block scales span many octaves (the kernel scales each block relative to its
    row's largest exponent): rows with magnitudes from 1e-4 to 30."""
    cfg = MoEConfig("pf-mx-range", tokens=140, hidden=512, num_experts=2, top_k=1, intermediate=512,
                    shared_intermediate=0, mode="mxfp8", bits=8, group_size=32, seed=52)
    from ironmlx_b200.workloads import Workload
    from util import quantize_stack
    wl = Workload(cfg)
    rng = np.random.default_rng(3)

    def spread(w):      # per-block magnitudes drawn log-uniformly
        blocks = w.reshape(w.shape[0], -1, 32)
        mag = np.exp(rng.uniform(np.log(1e-4), np.log(30.0), size=blocks.shape[:2])).astype(np.float32)
        return (blocks * mag[..., None]).reshape(w.shape).astype(np.float32)

    x = wl.activations()
    p = O.MoEParams(router_w=wl.router_weight().astype(F.bf16),
                    gate_up=quantize_stack([spread(wl.expert_gate_up(e)) * 0.05 for e in range(2)], cfg),
                    down=quantize_stack([spread(wl.expert_down(e)) * 0.05 for e in range(2)], cfg),
                    num_experts_per_tok=1, norm_topk_prob=True)
    for path in ("prefill", "decode"):
        x, p, _, y, tr = run(cfg, cuda, path, x, p)
        compare(cfg, x, p, y, tr)


@pytest.mark.parametrize("mode,bits,group", [("mxfp8", 8, 32), ("nvfp4", 4, 16)])
@pytest.mark.parametrize("cfg", [
    MoEConfig("fp-base", 40, 256, 8, 3, 128, 256, seed=71),
    MoEConfig("fp-one-token", 1, 512, 8, 2, 256, 128, seed=72),
    MoEConfig("fp-no-shared", 33, 384, 16, 4, 128, 0, seed=73),
    MoEConfig("fp-crowded", 100, 128, 2, 2, 256, 128, seed=74),
], ids=lambda c: c.name)
def test_decode_path_float_formats(cuda, cfg, mode, bits, group):
    """mxfp8 / nvfp4 on their decode kernel, against the checker and the format-agnostic kernels."""
    cfg = cfg.with_(name=f"{cfg.name}-{mode}", mode=mode, bits=bits, group_size=group)
    x, p, _, y, tr = run(cfg, cuda, "decode")
    compare(cfg, x, p, y, tr)
    _, _, _, yg, _ = run(cfg, cuda, "generic", x, p)
    assert O.rel_l2(y, yg) < 1e-3


def test_prefill_path_refuses_unsupported_shapes(cuda):
    x, p = make_params(SMALL)                            # hidden 256: scale rows shorter than 16 bytes
    with pytest.raises(_lib.IronMLXError):
        moe_to_device(p, cuda, "prefill").forward_with_stream(t_bf16(x, cuda))


@pytest.mark.parametrize("group", [64, 128])
def test_prefill_shape_reduced(cuda, group):
    """The prefill layer shape (hidden 2048, intermediate 512, shared expert, top-4 of 16 experts) with
    1024 tokens: 256 rows per expert on average, ragged tiles, the tensor-memory GEMM path by AUTO."""
    cfg = MoEConfig(f"c3-small-g{group}", tokens=1024, hidden=2048, num_experts=16, top_k=4,
                    intermediate=512 if group == 64 else 1024, shared_intermediate=512 if group == 64 else 1024,
                    group_size=group, seed=1)
    x, p, moe, y, tr = run(cfg, cuda)                 # AUTO must pick the prefill path here
    err = compare(cfg, x, p, y, tr, fast=True)
    _, _, _, yd, _ = run(cfg, cuda, "decode", x, p)
    assert O.rel_l2(y, yd) < 1.5e-3
    print(f"{cfg.name} rel-L2 {err:.3e}")


@pytest.mark.parametrize("cfg", [
    MoEConfig("tm-base", 24, 512, 8, 2, 512, 512, seed=31),
    MoEConfig("tm-one-token", 1, 1024, 8, 2, 512, 512, seed=32),
    MoEConfig("tm-no-shared", 33, 512, 16, 4, 1024, 0, seed=33),
    MoEConfig("tm-wide-shared", 12, 1024, 8, 2, 512, 1536, seed=34),
    MoEConfig("tm-crowded", 100, 512, 2, 2, 512, 512, seed=35),          # 100 rows per expert: many units
    MoEConfig("tm-k-eq-e", 9, 512, 4, 4, 512, 1024, seed=36),
    # a long second reduction: its tile pairs go out as chunks of four stages and the chunk that arrives last adds
    # the parts up
    MoEConfig("tm-long-mid", 20, 512, 4, 2, 2048, 2048, seed=38),
    MoEConfig("tm-long-mid-ragged", 37, 1024, 8, 3, 2048, 512, seed=39),
], ids=lambda c: c.name)
def test_decode_tensor_map_kernel(cuda, cfg):
    """Shapes the tensor-map fed decode kernel takes (4-bit, group 64, sizes % 512 == 0): against the
    checker, and against the register-pipelined decode kernel, which shares none of its data movement."""
    x, p, _, y, tr = run(cfg, cuda, "decode")
    compare(cfg, x, p, y, tr)
    _, _, _, yb, _ = run(cfg, cuda, "decode_regs", x, p)
    assert O.rel_l2(y, yb) < 1e-3


def test_decode_tensor_map_skew_and_empty(cuda):
    cfg = MoEConfig("tm-skew", 64, 512, 32, 4, 512, 512, seed=37, zipf_s=1.2, zipf_hot_share=0.2)
    x, p = make_params(cfg)
    p.router_logit_bias[:8] = -30.0
    x, p, _, y, tr = run(cfg, cuda, "decode", x, p)
    assert (tr["counts"][:8] == 0).all()
    compare(cfg, x, p, y, tr)


@pytest.mark.parametrize("cfg", [
    MoEConfig("rt-e32-h192", 31, 192, 32, 4, 128, 128, seed=41),          # K slices of 64
    MoEConfig("rt-e64-h384", 1, 384, 64, 6, 128, 128, seed=42),           # K slices of 128, one token
    MoEConfig("rt-e64-h512", 255, 512, 64, 8, 512, 512, seed=43),         # 8 token blocks, last one ragged
    MoEConfig("rt-e256-h256", 70, 256, 256, 8, 128, 0, seed=44),          # no shared expert
    MoEConfig("rt-e96-nonorm", 33, 512, 96, 5, 512, 512, norm_topk_prob=False, seed=45),
], ids=lambda c: c.name)
def test_split_k_router(cuda, cfg):
    """Batches below 256 tokens with a multiple of 32 experts take the split-K tensor-core router inside
    the fused forward: expert sets, weights, shared gate and the fp16 copy all feed the block output."""
    x, p = make_params(cfg)
    p.router_logit_bias = np.zeros(cfg.num_experts, np.float32)
    p.router_logit_bias[::3] = 0.25
    x, p, moe, y, tr = run(cfg, cuda, "auto", x, p)
    compare(cfg, x, p, y, tr)
    y2, tr2 = moe.forward_with_stream(t_bf16(x, cuda), trace=True)        # same workspace: the counters were left clean
    torch.cuda.synchronize()
    moe.check_status()
    assert np.array_equal(tr["topk_idx"], tr2["topk_idx"].cpu().numpy()) and np.array_equal(y, bf16_to_np(y2))


def test_c2_reduced_experts(cuda):
    """The decode benchmark shape with 32 of the 256 experts (the checker
    finishes in seconds), 64 tokens, top-8, shared expert."""
    cfg = CONFIGS["c2"].with_(name="c2-e32", num_experts=32)
    x, p, _, y, tr = run(cfg, cuda)
    err = compare(cfg, x, p, y, tr)
    print(f"c2-e32 rel-L2 {err:.3e}")


def _full_size(cfg, cuda):
    """A block of the benchmark's full size, built and quantized on the GPU, and the C/OpenMP
    checker's result on the same packed bytes."""
    from ironmlx_b200 import synthetic
    from ironmlx_b200.workloads import Workload
    from oracle import cref
    moe = synthetic.build_moe(cfg, cuda)
    x = Workload(cfg).activations()
    p = params_from_device(moe, cfg.top_k, cfg.norm_topk_prob)
    ref = cref.moe_forward(x, p)
    return moe, x, p, ref


def test_c2_full_size(cuda):
    """The decode benchmark workload itself (256 experts, 453 MB of packed weights): against the C checker,
    and the properties that do not depend on size — same result twice, the CUDA-graph replay equal to the
    eager call bit for bit, and a permutation of the tokens permuting the outputs."""
    cfg = CONFIGS["c2"]
    moe, x, p, ref = _full_size(cfg, cuda)
    xd = t_bf16(x, cuda)
    y, tr = moe.forward_with_stream(xd, trace=True)
    torch.cuda.synchronize()
    moe.check_status()
    yn = bf16_to_np(y)
    clear = check_routing(tr["topk_idx"].cpu().numpy(), tr["topk_w"].cpu().numpy(), x, p, cfg.top_k, cfg.norm_topk_prob)
    err = O.rel_l2(yn[clear], ref["y"][clear])
    assert err <= TOL, f"c2 full size: rel-L2 {err:.3e}"
    if clear.all():
        assert np.array_equal(tr["perm"].cpu().numpy(), ref["perm"]) and np.array_equal(tr["counts"].cpu().numpy(), ref["counts"])
    assert torch.equal(y, moe.forward_with_stream(xd))                        # deterministic
    assert torch.equal(y, moe.capture(xd)().clone())                          # graph replay == eager
    pi = np.random.default_rng(0).permutation(cfg.tokens)
    yp, trp = moe.forward_with_stream(t_bf16(x[pi], cuda), trace=True)
    assert torch.equal(trp["topk_idx"], tr["topk_idx"][torch.from_numpy(pi).to(cuda)])
    assert O.rel_l2(bf16_to_np(yp), yn[pi]) < 2e-4                            # sums regroup across warps, nothing else moves
    print(f"c2 full size rel-L2 {err:.3e}")


def test_c3_full_size(cuda):
    """The prefill benchmark workload (8192 tokens): tensor-memory path against the C checker and against the
    decode kernels on the same input."""
    cfg = CONFIGS["c3"]
    moe, x, p, ref = _full_size(cfg, cuda)
    xd = t_bf16(x, cuda)
    y, tr = moe.forward_with_stream(xd, trace=True)
    torch.cuda.synchronize()
    moe.check_status()
    yn = bf16_to_np(y)
    clear = check_routing(tr["topk_idx"].cpu().numpy(), tr["topk_w"].cpu().numpy(), x, p, cfg.top_k, cfg.norm_topk_prob)
    err = O.rel_l2(yn[clear], ref["y"][clear])
    assert err <= TOL, f"c3 full size: rel-L2 {err:.3e}"
    assert tr["counts"].sum().item() == cfg.tokens * cfg.top_k
    yd = moe.forward_with_stream(xd, path="decode")
    assert O.rel_l2(yn, bf16_to_np(yd)) < 1.5e-3
    print(f"c3 full size rel-L2 {err:.3e}")


def test_rms_norm_op(cuda):
    from ironmlx_b200 import ops
    rng = np.random.default_rng(5)
    x = (rng.standard_normal((37, 512)) * 3).astype(np.float32).astype(F.bf16).astype(np.float32)
    w = (1 + 0.2 * rng.standard_normal(512)).astype(np.float32).astype(F.bf16).astype(np.float32)
    for weight in (w, None):
        y = bf16_to_np(ops.rms_norm(t_bf16(x, cuda), None if weight is None else t_bf16(weight, cuda), 1e-6))
        ref = O.rms_norm(x, weight, 1e-6)
        # the factor's last bit can differ (summation order): at most one bf16 step on a few elements
        assert np.mean(y != ref) < 0.02 and np.abs(y - ref).max() <= 2.0 ** -7 * np.abs(ref).max()


@pytest.mark.parametrize("cfg", [
    MoEConfig("tail-splitk", 48, 512, 32, 4, 512, 512, seed=61),          # router normalises its own tiles
    MoEConfig("tail-cluster", 20, 256, 8, 2, 128, 128, seed=62),          # normalised copy + cluster router
    MoEConfig("tail-noshared", 5, 512, 64, 6, 512, 0, seed=63),
], ids=lambda c: c.name)
def test_decoder_layer_tail(cuda, cfg):
    """y = h + MoE(rms_norm(h)) in one call (qwen35.rs:271-276) against the checker's three-step version."""
    from ironmlx_b200 import nn as inn
    h, p = make_params(cfg)
    h = (2.5 * h).astype(np.float32).astype(F.bf16).astype(np.float32)    # a residual stream that is not unit-variance
    lw = (1 + 0.1 * np.random.default_rng(cfg.seed).standard_normal(cfg.hidden)).astype(np.float32).astype(F.bf16).astype(np.float32)
    yref, tr_ref, normed_ref = O.decoder_layer_tail(h, lw, 1e-6, p)
    moe = moe_to_device(p, cuda)
    norm = inn.RMSNorm(t_bf16(lw, cuda), 1e-6)
    y, tr = moe.forward_residual(t_bf16(h, cuda), norm, trace=True)
    torch.cuda.synchronize()
    moe.check_status()
    yn = bf16_to_np(y)
    # The per-row factor's last bit depends on the order of the sum of squares, which moves a few normalised
    # values by one bf16 step: routing is checked on the GPU's own normalised rows (the fused path must make
    # exactly the choices the unfused one makes), the output against the checker's three-step result.
    normed = bf16_to_np(norm.forward_with_stream(t_bf16(h, cuda)))
    assert np.mean(normed != normed_ref) < 0.02
    clear = check_routing(tr["topk_idx"].cpu().numpy(), tr["topk_w"].cpu().numpy(), normed, p, cfg.top_k, cfg.norm_topk_prob)
    assert O.rel_l2(yn[clear], yref[clear]) <= TOL
    # the block's own contribution, against the unfused calls on the GPU
    y2 = moe.forward_with_stream(norm.forward_with_stream(t_bf16(h, cuda)))
    mlp = bf16_to_np(y2)
    # element by element: one bf16 rounding of the sum plus the rounding the unfused block output carries
    bound = 2.0 ** -8 * np.abs(h + mlp) + 2.0 ** -8 * np.abs(mlp) + 1e-6
    assert np.all(np.abs(yn - (h + mlp)) <= bound)


@pytest.mark.parametrize("name", ["c4-nvfp4-decode", "c4-mxfp8-decode", "c4-nvfp4-prefill", "c4-mxfp8-prefill",
                                  "c5", "c5-2bit", "c5-8bit"])
def test_other_baseline_configs_full_size(cuda, name):
    """The remaining named workloads at their full size against the C checker: block-scaled formats at 256
    tokens (their decode kernel) and 4096 tokens (tensor-core path), and the skewed 16384-token batch at 4-, 2-
    and 8-bit (tensor-core path, ragged experts)."""
    cfg = CONFIGS[name]
    moe, x, p, ref = _full_size(cfg, cuda)
    y, tr = moe.forward_with_stream(t_bf16(x, cuda), trace=True)
    torch.cuda.synchronize()
    moe.check_status()
    clear = check_routing(tr["topk_idx"].cpu().numpy(), tr["topk_w"].cpu().numpy(), x, p, cfg.top_k, cfg.norm_topk_prob,
                          p.router_logit_bias)
    err = O.rel_l2(bf16_to_np(y)[clear], ref["y"][clear])
    assert err <= TOL, f"{name} full size: rel-L2 {err:.3e}"
    counts = tr["counts"].cpu().numpy()
    assert counts.sum() == cfg.tokens * cfg.top_k
    if name.startswith("c5"):
        assert counts.max() >= 0.06 * counts.sum()                         # the hottest expert holds ~8 % of the rows
    print(f"{name} full size rel-L2 {err:.3e}, hottest expert {counts.max() / counts.sum():.3f}")
