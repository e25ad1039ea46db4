"""The CPU checker's MoE block: invariants, hand-checkable cases, golden fixtures."""
import os

import numpy as np
import pytest

from ironmlx_b200.workloads import CONFIGS, MoEConfig
from oracle import formats as F
from oracle import moe as O
from util import SMALL, TINY, make_params

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_route_invariants():
    x, p = make_params(SMALL)
    idx, w, probs = O.route(x, p.router_w, SMALL.top_k, True)
    assert idx.shape == w.shape == (SMALL.tokens, SMALL.top_k)
    assert np.allclose(probs.sum(-1), 1, atol=1e-6) and np.allclose(w.sum(-1), 1, atol=1e-6)
    assert np.all(np.diff(w, axis=-1) <= 0)                       # descending slots (moe.rs:71-73)
    for t in range(SMALL.tokens):
        assert len(set(idx[t])) == SMALL.top_k
        rest = np.delete(probs[t], idx[t])
        assert probs[t, idx[t]].min() >= rest.max()
    idx2, w2, _ = O.route(x, p.router_w, SMALL.top_k, False)
    assert np.array_equal(idx, idx2) and np.allclose(w2, np.take_along_axis(probs, idx, -1))


def test_route_tie_break_lower_index_first():
    x = np.ones((1, 8), np.float32)
    wr = np.zeros((4, 8), np.float32).astype(F.bf16)              # all logits equal
    idx, w, _ = O.route(x, wr, 2, True)
    assert idx.tolist() == [[0, 1]] and np.allclose(w, 0.5)


def test_bucket_is_stable_counting_sort():
    rng = np.random.default_rng(0)
    top = rng.integers(0, 6, size=(37, 3)).astype(np.int32)
    counts, offsets, perm, inv = O.bucket(top, 6)
    c2, o2, p2, i2 = O.bucket_fast(top, 6)
    assert all(np.array_equal(a, b) for a, b in [(counts, c2), (offsets, o2), (perm, p2), (inv, i2)])
    assert counts.sum() == top.size and np.array_equal(np.sort(perm), np.arange(top.size))
    assert np.array_equal(offsets[1:] - offsets[:-1], counts)
    flat = top.reshape(-1)
    for e in range(6):
        seg = perm[offsets[e]:offsets[e + 1]]
        assert np.all(flat[seg] == e) and np.all(np.diff(seg) > 0)   # token-major inside an expert
    assert np.array_equal(perm[inv], np.arange(top.size))


def test_bucket_drops_out_of_range_ids():
    top = np.array([[0, 7], [1, 0]], np.int32)                      # 7 >= num_experts (moe.rs:100)
    counts, offsets, perm, _ = O.bucket(top, 2)
    assert counts.tolist() == [2, 1] and perm.tolist() == [0, 3, 2]


def test_tiny_block_by_hand():
    """Recompute the tiny case with a straight-line restatement of moe.rs."""
    x, p = make_params(TINY)
    tr = O.moe_forward(x, p)
    k = TINY.top_k
    y = np.zeros_like(tr.y, dtype=np.float64)
    for t in range(TINY.tokens):
        for s in range(k):
            e = int(tr.top_idx[t, s])
            wg, wu, wd = O.expert_weights(p, e)
            g = x[t].astype(np.float64) @ wg.T
            u = x[t].astype(np.float64) @ wu.T
            a = g / (1 + np.exp(-g)) * u
            y[t] += tr.top_w[t, s] * (a @ wd.T.astype(np.float64))
        g = x[t].astype(np.float64) @ p.shared_gate_proj.dense().T
        u = x[t].astype(np.float64) @ p.shared_up_proj.dense().T
        so = (g / (1 + np.exp(-g)) * u) @ p.shared_down_proj.dense().T.astype(np.float64)
        gate = 1 / (1 + np.exp(-(x[t].astype(np.float64) @ p.shared_expert_gate_w.astype(np.float32)[0])))
        y[t] += gate * so
    assert O.rel_l2(tr.y, y) < 2e-6


def test_identity_like_combine():
    """With every expert identical, the routed part equals one expert's output
    times the sum of the routing weights (= 1 when renormalised)."""
    cfg = MoEConfig("same", tokens=6, hidden=64, num_experts=4, top_k=2, intermediate=64, seed=11)
    x, p = make_params(cfg)
    for q in (p.gate_up, p.down):
        q.w[:] = q.w[0]
        q.scales[:] = q.scales[0]
        q.biases[:] = q.biases[0]
    tr = O.moe_forward(x, p)
    one = O.swiglu_mlp(x, *O.expert_weights(p, 0))
    assert O.rel_l2(tr.y, one) < 1e-6


def test_bf16_boundary_mode_is_close_but_not_equal():
    x, p = make_params(SMALL)
    a, b = O.moe_forward(x, p), O.moe_forward(x, p, bf16_boundaries=True)
    assert np.array_equal(a.perm, b.perm)
    r = O.rel_l2(b.y, a.y)
    assert 1e-4 < r < 2e-2


@pytest.mark.parametrize("name", ["c1"])
def test_golden_fixture(name):
    """The committed fixture was produced by tests/golden/make_golden.py from
    this same checker; this pins the checker against accidental change."""
    path = os.path.join(GOLDEN, f"{name}.npz")
    g = np.load(path)
    x, p = make_params(CONFIGS[name])
    tr = O.moe_forward(x, p)
    assert np.array_equal(tr.top_idx, g["top_idx"]) and np.array_equal(tr.perm, g["perm"])
    assert np.array_equal(tr.counts, g["counts"])
    assert np.allclose(tr.top_w, g["top_w"], rtol=1e-6, atol=0)
    assert O.rel_l2(tr.y, g["y"].astype(np.float32)) < 1e-6
    assert int(g["gate_up_w_crc"]) == _crc(p.gate_up.w) and int(g["down_w_crc"]) == _crc(p.down.w)


def _crc(a):
    import zlib
    return zlib.crc32(np.ascontiguousarray(a).tobytes())


def test_rms_norm_hand_computed():
    """x = [3, 4] (mean square 12.5), eps = 0: factor 1/sqrt(12.5); the normalised values are rounded to
    bf16 before the weight multiplies them (fast.rs:37-49 through norm.rs:21-24)."""
    x = np.array([[3.0, 4.0]], np.float32)
    inv = np.float32(1.0 / np.sqrt(12.5))
    t = (x * inv).astype(F.bf16).astype(np.float32)
    assert np.array_equal(O.rms_norm(x, None, 0.0), t)
    w = np.array([0.5, 3.0], np.float32)
    assert np.array_equal(O.rms_norm(x, w, 0.0), (w * t).astype(F.bf16).astype(np.float32))
    # eps matters for a zero row and keeps it zero
    assert np.array_equal(O.rms_norm(np.zeros((1, 4), np.float32), np.ones(4, np.float32), 1e-6), np.zeros((1, 4)))


def test_decoder_layer_tail_is_residual_plus_block():
    from util import TINY, make_params
    x, p = make_params(TINY)
    lw = (1.0 + 0.1 * np.arange(TINY.hidden, dtype=np.float32) / TINY.hidden).astype(F.bf16).astype(np.float32)
    y, tr, normed = O.decoder_layer_tail(x, lw, 1e-6, p)
    again = O.moe_forward(normed, p)
    assert np.array_equal(tr.y, again.y)
    assert np.array_equal(y, (x + tr.y.astype(F.bf16).astype(np.float32)).astype(F.bf16).astype(np.float32))
