"""The C/OpenMP restatement (oracle/moe_ref.c) against the numpy checker."""
import numpy as np
import pytest

from ironmlx_b200.workloads import CONFIGS
from oracle import cref
from oracle import moe as O
from util import SMALL, TINY, make_params

FORMATS = [("affine", 2, 64), ("affine", 3, 32), ("affine", 4, 64), ("affine", 5, 64), ("affine", 6, 128),
           ("affine", 8, 64), ("mxfp8", 8, 32), ("nvfp4", 4, 16)]


@pytest.mark.parametrize("mode,bits,group", FORMATS)
def test_c_matches_numpy_every_format(mode, bits, group):
    cfg = TINY.with_(mode=mode, bits=bits, group_size=group)
    x, p = make_params(cfg)
    ref = O.moe_forward(x, p)
    got = cref.moe_forward(x, p)
    assert np.array_equal(got["top_idx"], ref.top_idx) and np.array_equal(got["perm"], ref.perm)
    assert np.array_equal(got["counts"], ref.counts)
    assert np.allclose(got["top_w"], ref.top_w, rtol=1e-6)
    assert O.rel_l2(got["y"], ref.y) < 2e-6


@pytest.mark.parametrize("cfg", [SMALL, CONFIGS["c1"]], ids=lambda c: c.name)
def test_c_matches_numpy_block(cfg):
    x, p = make_params(cfg)
    ref = O.moe_forward(x, p)
    got = cref.moe_forward(x, p)
    assert np.array_equal(got["top_idx"], ref.top_idx) and np.array_equal(got["perm"], ref.perm)
    assert O.rel_l2(got["y"], ref.y) < 2e-6
    assert cref.threads() >= 1


def test_router_in_the_reference_dtypes_both_checkers_agree():
    """The reference's gate Linear returns bf16 logits and softmax / argsort / topk run on bf16 arrays
    (moe.rs:67-74); the kernels and the default checkers keep fp32.  With the switch on, the numpy and the C
    checker still pick the same experts, and the count of rows that differ from the fp32 routing is what the
    design notes quote (c1: none; the rounding moves an assignment in a few per cent of the rows at 256 experts)."""
    cfg = CONFIGS["c1"]
    x, p = make_params(cfg)
    want, _, _ = O.route(x, p.router_w, cfg.top_k, cfg.norm_topk_prob, p.router_logit_bias, bf16_logits=True)
    try:
        cref.set_bf16_logits(True)
        got = cref.moe_forward(x, p)
    finally:
        cref.set_bf16_logits(False)
    assert np.array_equal(got["top_idx"], want)
    ch = O.routing_changes(x, p.router_w, cfg.top_k, p.router_logit_bias)
    assert ch["rows"] == cfg.tokens and ch["rows_set_differs"] == 0
    # a wider router: ties inside one bf16 step appear
    wide = SMALL.with_(num_experts=64, top_k=8, tokens=256, seed=5)
    xw, pw = make_params(wide)
    chw = O.routing_changes(xw, pw.router_w, wide.top_k, pw.router_logit_bias)
    assert chw["rows_order_differs"] >= chw["rows_set_differs"] >= 0
    assert chw["assignments_moved"] <= chw["rows"] * wide.top_k // 10      # a minority of the assignments
    want_w, _, _ = O.route(xw, pw.router_w, wide.top_k, wide.norm_topk_prob, pw.router_logit_bias, bf16_logits=True)
    try:
        cref.set_bf16_logits(True)
        got_w = cref.moe_forward(xw, pw)
    finally:
        cref.set_bf16_logits(False)
    # exact ties after the rounding go to the lower expert id in both checkers
    assert np.array_equal(got_w["top_idx"], want_w)
