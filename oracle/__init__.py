"""CPU oracle for the mixture-of-experts block of ironmlx's Qwen3.5-MoE path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package may import this
package; it is the checker that the CUDA path is compared against and the
CPU baseline that the benchmark times beside it.

PARITY UNPINNED.  The arithmetic of the reference's path lives in Apple MLX
core (v0.31.1, named only by a comment in mlx-sys/build.rs:38-39) reached
through mlx-c (vendor/mlx-c, an empty un-vendored submodule).  Neither is in
the reference tree, no Rust toolchain or Python `mlx` module is available to
run it, and the reference's own tests hold no golden vector, fixture or
known-answer test for softmax/top-k routing, `quantized_matmul`,
`dequantize` or the MoE block (mlx/tests/integration.rs only checks that a
softmax row sums to one).  The oracle therefore restates

  * the stage order, slot order, bucketing order and combine order of
    mlx/src/nn/moe.rs:55-183 (the reference's own code), and
  * MLX's published quantized formats (affine 2/3/4/5/6/8-bit, mxfp8, nvfp4)
    from its public documentation,

and is pinned only against hand-computed vectors (tests/test_oracle_formats.py,
tests/test_oracle_moe.py) and the committed fixtures it generated itself
(tests/golden/).
"""
