"""Stage-level parity of the CUDA path (through the C ABI) against the CPU checker:
router top-k, dispatch sort, quantized ops."""
import ctypes as C

import numpy as np
import pytest
import torch

from ironmlx_b200 import _lib, ops
from ironmlx_b200.workloads import CONFIGS, MoEConfig
from oracle import formats as F
from oracle import moe as O
from gpu_util import bf16_to_np, q_to_device, t_bf16
from util import SMALL, TINY, make_params, quantize_stack, squeeze0

pytestmark = pytest.mark.gpu

FORMATS = [("affine", 2, 64), ("affine", 3, 32), ("affine", 4, 64), ("affine", 4, 128), ("affine", 5, 64),
           ("affine", 6, 128), ("affine", 8, 64), ("affine", 8, 32), ("mxfp8", 8, 32), ("nvfp4", 4, 16)]


def run_route(x, p, k, norm, dev, bias=None, ws=False):
    n, h = x.shape
    e = p.router_w.shape[0]
    xd, wr = t_bf16(x, dev), t_bf16(p.router_w, dev)
    wsg = None if p.shared_expert_gate_w is None else t_bf16(p.shared_expert_gate_w, dev)
    idx = torch.empty(n, k, dtype=torch.int32, device=dev)
    w = torch.empty(n, k, device=dev)
    sg = torch.empty(n, device=dev)
    x16 = torch.empty(n, h, dtype=torch.float16, device=dev)
    bd = None if bias is None else torch.from_numpy(bias).to(dev)
    args = (xd.data_ptr(), n, h, wr.data_ptr(), None if bd is None else bd.data_ptr(), e, k, int(norm),
            None if wsg is None else wsg.data_ptr(), idx.data_ptr(), w.data_ptr(), sg.data_ptr(), x16.data_ptr())
    if ws:      # the entry point with scratch: split-K tensor-core router where it applies
        nb = C.c_size_t(0)
        _lib.check(_lib.lib().imx_moe_route_scratch_bytes(n, h, e, C.byref(nb)))
        scratch = torch.empty(max(nb.value, 256), dtype=torch.uint8, device=dev)
        _lib.check(_lib.lib().imx_moe_route_ws(*args, scratch.data_ptr(), scratch.numel(), ops.stream_ptr()))
    else:
        _lib.check(_lib.lib().imx_moe_route(*args, ops.stream_ptr()))
    torch.cuda.synchronize()
    return idx.cpu().numpy(), w.cpu().numpy(), sg.cpu().numpy(), x16.cpu().numpy()


def check_routing(idx, w, x, p, k, norm, bias=None):
    """Bit-exact ordered expert lists on rows without fp32 near-ties; on the
    rest the choice must still be valid within the tie margin."""
    ridx, rw, probs = O.route(x, p.router_w, k, norm, bias)
    margin = O.routing_margin(probs, k)
    clear = margin > 1e-5
    assert clear.mean() > 0.97
    assert np.array_equal(idx[clear], ridx[clear])
    assert np.allclose(w[clear], rw[clear], rtol=2e-5, atol=1e-8)
    for t in np.nonzero(~clear)[0]:
        kth = np.sort(probs[t])[::-1][k - 1]
        assert len(set(idx[t])) == k and np.all(probs[t, idx[t]] >= kth * (1 - 1e-4))
    return clear


@pytest.mark.parametrize("cfg", [TINY, SMALL, CONFIGS["c1"],
                                 MoEConfig("r64", 64, 2048, 256, 8, 64, 64, seed=0),
                                 MoEConfig("r300", 300, 1024, 128, 6, 64, 0, seed=2),
                                 MoEConfig("odd", 7, 256, 48, 5, 64, 64, norm_topk_prob=False, seed=5),
                                 MoEConfig("one", 1, 128, 4, 4, 64, 0, seed=6)], ids=lambda c: c.name)
@pytest.mark.parametrize("ws", [False, True], ids=["plain", "scratch"])
def test_route_matches_checker(cuda, cfg, ws):
    wl_cfg = cfg.with_(intermediate=64, shared_intermediate=min(cfg.shared_intermediate, 64))
    from ironmlx_b200.workloads import Workload
    wl = Workload(wl_cfg)
    x = wl.activations()
    p = O.MoEParams(router_w=wl.router_weight().astype(F.bf16), gate_up=None, down=None,
                    num_experts_per_tok=cfg.top_k, norm_topk_prob=cfg.norm_topk_prob)
    if cfg.shared_intermediate:
        p.shared_expert_gate_w = wl.shared_gate_weight().astype(F.bf16)
    idx, w, sg, x16 = run_route(x, p, cfg.top_k, cfg.norm_topk_prob, cuda, ws=ws)
    check_routing(idx, w, x, p, cfg.top_k, cfg.norm_topk_prob)
    # the fp16 copy is exact except below fp16's subnormal spacing (2^-24)
    big = np.abs(x) >= 2.0 ** -14
    assert np.array_equal(x16.astype(np.float32)[big], x[big])
    assert np.abs(x16.astype(np.float32) - x).max() <= 2.0 ** -25
    if cfg.shared_intermediate:
        ref = O.sigmoid((x.astype(np.float64) @ p.shared_expert_gate_w.astype(np.float32).astype(np.float64).T)
                        .astype(np.float32))[:, 0]
        assert np.allclose(sg, ref, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("ws", [False, True], ids=["plain", "scratch"])
def test_route_with_logit_bias_and_exact_ties(cuda, ws):
    cfg = MoEConfig("b", 33, 256, 64, 8, 64, 0, seed=8)
    from ironmlx_b200.workloads import Workload
    wl = Workload(cfg)
    x = wl.activations()
    p = O.MoEParams(router_w=wl.router_weight().astype(F.bf16), gate_up=None, down=None, num_experts_per_tok=8)
    bias = np.linspace(-2, 0, 64).astype(np.float32)
    idx, w, _, _ = run_route(x, p, 8, True, cuda, bias, ws=ws)
    check_routing(idx, w, x, p, 8, True, bias)
    # exact ties: all-zero router -> equal probabilities -> experts 0..k-1 in order
    p0 = O.MoEParams(router_w=np.zeros((64, 256), np.float32).astype(F.bf16), gate_up=None, down=None,
                     num_experts_per_tok=8)
    idx, w, _, _ = run_route(x, p0, 8, True, cuda, ws=ws)
    assert np.array_equal(idx, np.tile(np.arange(8, dtype=np.int32), (33, 1))) and np.allclose(w, 0.125)


def run_sort(ids, e, dev):
    a = ids.size
    d = torch.from_numpy(ids.astype(np.int32)).to(dev)
    sb = C.c_size_t(0)
    _lib.check(_lib.lib().imx_moe_sort_scratch_bytes(a, e, C.byref(sb)))
    scratch = torch.zeros(max(sb.value, 256), dtype=torch.uint8, device=dev)
    i32 = dict(dtype=torch.int32, device=dev)
    counts, offsets = torch.empty(e, **i32), torch.empty(e + 1, **i32)
    perm, inv = torch.full((max(a, 1),), -7, **i32), torch.empty(max(a, 1), **i32)
    _lib.check(_lib.lib().imx_moe_sort(d.data_ptr(), a, e, counts.data_ptr(), offsets.data_ptr(), perm.data_ptr(),
                                       inv.data_ptr(), scratch.data_ptr(), scratch.numel(), ops.stream_ptr()))
    torch.cuda.synchronize()
    return counts.cpu().numpy(), offsets.cpu().numpy(), perm.cpu().numpy()[:a], inv.cpu().numpy()[:a]


@pytest.mark.parametrize("n,k,e", [(1, 1, 1), (5, 2, 4), (64, 8, 256), (512, 8, 256), (513, 8, 256),
                                   (8192, 8, 256), (16384, 8, 256), (1000, 3, 1000), (4097, 1, 7)])
def test_sort_bit_exact(cuda, n, k, e):
    rng = np.random.default_rng(n * 31 + e)
    top = rng.integers(0, e, size=(n, k)).astype(np.int32)
    if n >= 64:
        top[: n // 4] = rng.integers(0, max(1, e // 16), size=(n // 4, k))       # skew + empty experts
    rc, ro, rp, ri = O.bucket_fast(top, e)
    for _ in range(2):                                                            # twice: bit-identical reruns
        c, o, p, i = run_sort(top.reshape(-1), e, cuda)
        assert np.array_equal(c, rc) and np.array_equal(o, ro)
        assert np.array_equal(p, rp) and np.array_equal(i, ri)


def test_sort_drops_out_of_range_ids(cuda):
    top = np.array([[0, 9], [1, 0], [-3, 1]], np.int32)
    rc, ro, rp, ri = O.bucket(top, 2)
    c, o, p, i = run_sort(top.reshape(-1), 2, cuda)
    assert np.array_equal(c, rc) and np.array_equal(o, ro)
    assert np.array_equal(p[: ro[-1]], rp) and np.array_equal(i, ri)


@pytest.mark.parametrize("mode,bits,group", FORMATS)
def test_dequantize_bit_exact(cuda, mode, bits, group):
    rng = np.random.default_rng(bits * 7 + group)
    w = (rng.standard_normal((40, 256)) * 0.02).astype(np.float32)
    cfg = TINY.with_(mode=mode, bits=bits, group_size=group)
    q = squeeze0(quantize_stack([w], cfg))
    ref = q.dense()
    qd = q_to_device(q, cuda)
    out = ops.dequantize(qd.weight, qd.scales, qd.biases, group, bits, mode, dtype=torch.float32,
                         global_scale=q.global_scale)
    assert np.array_equal(out.cpu().numpy(), ref)
    out16 = ops.dequantize(qd.weight, qd.scales, qd.biases, group, bits, mode, global_scale=q.global_scale)
    assert np.array_equal(bf16_to_np(out16), F.to_bf16(ref))


@pytest.mark.parametrize("mode,bits,group", FORMATS)
def test_quantize_bit_exact(cuda, mode, bits, group):
    rng = np.random.default_rng(bits * 11 + group)
    w = (rng.standard_normal((24, 256)) * 0.02).astype(np.float32)
    w[3, :group] = 0.0                                   # an all-zero group
    w[4, :group] = np.abs(w[4, :group])                  # an all-positive group
    wd = torch.from_numpy(w).to(cuda)
    if mode == "nvfp4":
        p, s, t = F.nvfp4_quantize(w)
        gp, gs, gb, gt = ops.quantize(wd, group, bits, mode, global_scale=float(t))
        b = None
    else:
        p, s, b, _ = F.quantize(w, group, bits, mode)
        gp, gs, gb = ops.quantize(wd, group, bits, mode)
    assert np.array_equal(gp.cpu().numpy().view(np.uint32), p)
    if mode == "affine":
        assert np.array_equal(gs.view(torch.int16).cpu().numpy().view(np.uint16), s.view(np.uint16))
        assert np.array_equal(gb.view(torch.int16).cpu().numpy().view(np.uint16), b.view(np.uint16))
    else:
        assert np.array_equal(gs.cpu().numpy(), s)


@pytest.mark.parametrize("mode,bits,group", FORMATS)
@pytest.mark.parametrize("transpose", [True, False])
def test_quantized_matmul(cuda, mode, bits, group, transpose):
    rng = np.random.default_rng(bits * 13 + group)
    w = (rng.standard_normal((72, 256)) * 0.02).astype(np.float32)
    q = squeeze0(quantize_stack([w], TINY.with_(mode=mode, bits=bits, group_size=group)))
    x = F.to_bf16(rng.standard_normal((13, 256 if transpose else 72)))
    ref = F.quantized_matmul(x, q.w, q.scales, q.biases, transpose, group, bits, mode, q.global_scale)
    qd = q_to_device(q, cuda)
    y = ops.quantized_matmul(t_bf16(x, cuda), qd.weight, qd.scales, qd.biases, transpose, group, bits, mode,
                             global_scale=q.global_scale)
    got = bf16_to_np(y)
    assert got.shape == ref.shape
    assert O.rel_l2(got, ref) < 2e-3                     # bf16 output rounding only
    assert O.rel_l2(got, F.to_bf16(ref)) < 5e-4


def test_quantized_matmul_errors(cuda):
    q = squeeze0(quantize_stack([np.zeros((8, 128), np.float32)], TINY))
    qd = q_to_device(q, cuda)
    x = torch.zeros(2, 64, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(_lib.IronMLXError):
        ops.quantized_matmul(x, qd.weight, qd.scales, qd.biases)          # wrong inner dimension
    with pytest.raises(_lib.IronMLXError):
        ops.quantized_matmul(x.float(), qd.weight, qd.scales, qd.biases)  # wrong dtype
    with pytest.raises(_lib.IronMLXError):
        ops.dequantize(qd.weight, qd.scales, qd.biases, 64, 7, "affine")  # bad bits
    with pytest.raises(_lib.IronMLXError):
        ops.dequantize(qd.weight, qd.scales, None, 64, 4, "affine")       # affine without biases


@pytest.mark.parametrize("mode,bits,group", [("affine", 4, 64), ("mxfp8", 8, 32), ("nvfp4", 4, 16)])
def test_gather_qmm(cuda, mode, bits, group):
    rng = np.random.default_rng(3)
    blocks = [(rng.standard_normal((48, 128)) * 0.02).astype(np.float32) for _ in range(5)]
    q = quantize_stack(blocks, TINY.with_(mode=mode, bits=bits, group_size=group))
    x = F.to_bf16(rng.standard_normal((9, 128)))
    lhs = rng.integers(0, 9, size=20).astype(np.int32)
    rhs = rng.integers(0, 5, size=20).astype(np.int32)
    dense = q.dense()
    ref = np.stack([x[l].astype(np.float64) @ dense[r].astype(np.float64).T for l, r in zip(lhs, rhs)])
    qd = q_to_device(q, cuda)
    y = ops.gather_qmm(t_bf16(x, cuda), qd.weight, qd.scales, qd.biases, torch.from_numpy(lhs).to(cuda),
                       torch.from_numpy(rhs).to(cuda), group, bits, mode, global_scale=q.global_scale)
    assert O.rel_l2(bf16_to_np(y), ref) < 2e-3
