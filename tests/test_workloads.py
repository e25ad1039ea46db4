import numpy as np

from ironmlx_b200.workloads import CONFIGS, Workload, algorithmic_bytes_decode, algorithmic_flops, round_bf16


def test_tensors_are_order_independent_and_seeded():
    a = Workload(CONFIGS["c1"])
    b = Workload(CONFIGS["c1"])
    _ = b.expert_down(3)
    assert np.array_equal(a.expert_gate_up(5), b.expert_gate_up(5))
    assert not np.array_equal(a.expert_gate_up(5), a.expert_gate_up(6))
    assert not np.array_equal(a.activations(), Workload(CONFIGS["c1"].with_(seed=1)).activations())
    x = a.activations()
    assert x.shape == (32, 512) and abs(float(x.std()) - 1.0) < 0.05
    assert np.array_equal(x, round_bf16(x))
    assert abs(float(a.router_weight().std()) - 0.02) < 0.002


def test_algorithmic_work_matches_stated_figures():
    c2, c3 = CONFIGS["c2"], CONFIGS["c3"]
    per_expert = 3 * 512 * 2048 * (0.5 + 4 / 64)
    assert per_expert == 1769472
    assert abs(algorithmic_bytes_decode(c2, 222) - 397e6) < 2e6
    assert abs(algorithmic_flops(c3) - 4.7248e11) / 4.7248e11 < 1e-3


def test_zipf_bias_hits_the_hot_share():
    cfg = CONFIGS["c5"].with_(tokens=2048)
    wl = Workload(cfg)
    bias = wl.router_logit_bias()
    assert bias.shape == (256,) and bias.max() == 0
    z = wl.activations().astype(np.float64) @ wl.router_weight().astype(np.float64).T + bias
    top = np.argsort(-z, -1)[:, :8]
    share = np.bincount(top.reshape(-1), minlength=256).max() / top.size
    assert abs(share - 0.08) < 0.01
