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
