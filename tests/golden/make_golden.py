"""Regenerates the committed known-answer fixtures from the CPU checker:

    python tests/golden/make_golden.py

c1.npz: the 32-token / 16-expert / top-4 affine-4-bit case (seed 0): routing,
dispatch permutation, fp32 output, and CRCs of the packed expert weights the
seeded generator + quantizer produce.  tiny_*.npz: one small case per weight
format.  The reference's own tests hold no vectors for this path, so these
fixtures pin the checker against itself (and the CUDA path against both).
"""
import os
import sys
import zlib

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from ironmlx_b200.workloads import CONFIGS  # noqa: E402
from oracle import moe as O  # noqa: E402
from util import TINY, make_params  # noqa: E402

FORMATS = [("affine", 2, 64), ("affine", 3, 32), ("affine", 4, 64), ("affine", 5, 64), ("affine", 6, 128),
           ("affine", 8, 64), ("mxfp8", 8, 32), ("nvfp4", 4, 16)]


def crc(a):
    return zlib.crc32(np.ascontiguousarray(a).tobytes())


def dump(name, cfg):
    x, p = make_params(cfg)
    tr = O.moe_forward(x, p)
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"), top_idx=tr.top_idx, top_w=tr.top_w, counts=tr.counts,
        offsets=tr.offsets, perm=tr.perm, y=tr.y.astype(np.float32),
        gate_up_w_crc=np.int64(crc(p.gate_up.w)), down_w_crc=np.int64(crc(p.down.w)))


if __name__ == "__main__":
    dump("c1", CONFIGS["c1"])
    for mode, bits, group in FORMATS:
        dump(f"tiny_{mode}{bits}_g{group}", TINY.with_(mode=mode, bits=bits, group_size=group))
