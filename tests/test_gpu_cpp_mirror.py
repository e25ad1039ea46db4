"""The C++ host mirror (include/ironmlx_b200.hpp) against the ctypes path:
same ABI underneath, so the outputs must be bit-identical."""
import os
import shutil
import subprocess

import numpy as np
import pytest

from ironmlx_b200 import _lib
from ironmlx_b200.workloads import MoEConfig
from oracle import formats as F
from gpu_util import bf16_to_np, moe_to_device, t_bf16, t_words
from util import make_params

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "mirror_main.cpp")


def build_mirror(out_dir):
    exe = os.path.join(out_dir, "mirror_main")
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    lib_dir = os.path.dirname(_lib.LIB_PATH)
    cmd = ["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(cuda, "include"), SRC,
           "-o", exe, "-L", lib_dir, "-l:libironmlx_b200.so", "-L", os.path.join(cuda, "lib64"), "-lcudart",
           f"-Wl,-rpath,{lib_dir}", f"-Wl,-rpath,{os.path.join(cuda, 'lib64')}"]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return exe


def dump(path, a):
    np.ascontiguousarray(a).tofile(path)


def test_cpp_mirror_compiles(tmp_path):
    """The header and the driver compile and link against the built library (no GPU needed)."""
    if shutil.which("g++") is None or not os.path.exists(_lib.LIB_PATH):
        pytest.skip("g++ or the library is missing")
    assert os.path.exists(build_mirror(str(tmp_path)))


@pytest.mark.gpu
def test_cpp_mirror_matches_ctypes_path(cuda, tmp_path):
    cfg = MoEConfig("mirror", tokens=24, hidden=512, num_experts=8, top_k=2, intermediate=512,
                    shared_intermediate=512, seed=51)
    x, p = make_params(cfg)
    d = str(tmp_path)
    exe = build_mirror(d)
    with open(os.path.join(d, "meta.txt"), "w") as f:
        f.write(f"{cfg.tokens} {cfg.hidden} {cfg.num_experts} {cfg.top_k} {cfg.intermediate} "
                f"{cfg.shared_intermediate} {int(cfg.norm_topk_prob)} {cfg.bits} {cfg.group_size}\n")
    bf = lambda a: np.asarray(a, np.float32).astype(F.bf16)
    dump(os.path.join(d, "x.bin"), bf(x))
    dump(os.path.join(d, "router_w.bin"), bf(p.router_w))
    dump(os.path.join(d, "shared_expert_gate.bin"), bf(p.shared_expert_gate_w))
    for name, q in (("gate_up", p.gate_up), ("down", p.down), ("shared_gate", p.shared_gate_proj),
                    ("shared_up", p.shared_up_proj), ("shared_down", p.shared_down_proj)):
        dump(os.path.join(d, f"{name}_w.bin"), q.w)
        dump(os.path.join(d, f"{name}_s.bin"), bf(q.scales))
        dump(os.path.join(d, f"{name}_b.bin"), bf(q.biases))
    lw = bf(1 + 0.1 * np.random.default_rng(4).standard_normal(cfg.hidden))
    dump(os.path.join(d, "ln_w.bin"), lw)
    rng = np.random.default_rng(3)
    xq = bf(rng.standard_normal((cfg.tokens, cfg.intermediate)).astype(np.float32))
    dump(os.path.join(d, "xq.bin"), xq)
    r = subprocess.run([exe, d], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "mirror ok" in r.stdout, r.stderr

    moe = moe_to_device(p, cuda)
    y = bf16_to_np(moe.forward_with_stream(t_bf16(x, cuda)))
    y_cpp = np.fromfile(os.path.join(d, "y.bin"), dtype=F.bf16).astype(np.float32).reshape(y.shape)
    assert np.array_equal(y, y_cpp)

    from ironmlx_b200 import ops
    q = p.down
    yq = ops.quantized_matmul(t_bf16(xq, cuda), t_words(q.w[0], cuda), t_bf16(q.scales[0], cuda),
                              t_bf16(q.biases[0], cuda), True, cfg.group_size, cfg.bits, "affine")
    yq_cpp = np.fromfile(os.path.join(d, "yq.bin"), dtype=F.bf16).astype(np.float32).reshape(cfg.tokens, cfg.hidden)
    assert np.array_equal(bf16_to_np(yq), yq_cpp)

    from ironmlx_b200 import nn as inn
    yt = bf16_to_np(moe.forward_residual(t_bf16(x, cuda), inn.RMSNorm(t_bf16(lw, cuda), 1e-6)))
    yt_cpp = np.fromfile(os.path.join(d, "yt.bin"), dtype=F.bf16).astype(np.float32).reshape(yt.shape)
    assert np.array_equal(yt, yt_cpp)

    ym = bf16_to_np(moe.shared_expert.forward_with_stream(t_bf16(x, cuda)))
    ym_cpp = np.fromfile(os.path.join(d, "ym.bin"), dtype=F.bf16).astype(np.float32).reshape(ym.shape)
    assert np.array_equal(ym, ym_cpp)
    yl = bf16_to_np(moe.gate.forward_with_stream(t_bf16(x, cuda)))
    yl_cpp = np.fromfile(os.path.join(d, "yl.bin"), dtype=F.bf16).astype(np.float32).reshape(yl.shape)
    assert np.array_equal(yl, yl_cpp)
