/* ironmlx_b200 -- values of imx_moe_config.path that select cross-check kernels.
 *
 * Not part of the drop-in boundary (include/ironmlx_b200.h): these exist so that
 * tests can run one input through two independent implementations of the same
 * expert products and compare.  They may change or disappear between versions.
 */
#ifndef IRONMLX_B200_TESTING_H
#define IRONMLX_B200_TESTING_H

#define IMX_PATH_DECODE_REGS 4     /* affine decode kernel, register-pipelined variant (no TMA)        */
#define IMX_PATH_PREFILL_PLAIN 5    /* tcgen05 prefill kernel, one weight tile per stage, streamed activations */
#define IMX_PATH_PREFILL_SMEM 6    /* tcgen05 prefill kernel with the dequantized tile in shared memory */

/* Makes a bounded device wait run out on purpose, without hanging or faulting the GPU: the tensor-map decode
 * kernels' warps hand partial sums to one another through flags; with withhold != 0 the flags are never raised
 * and with a small spin_limit (iterations of about 64 ns) the waiting warps give up at once, record status 2 in
 * the workspace and return.  imx_moe_status() must then report IMX_ERR_DEVICE, and the next call (after
 * imx_testing_decode_handoff(0, 0), which restores the defaults) must be correct again.  Process-wide. */
#ifdef __cplusplus
extern "C"
#endif
__attribute__((visibility("default"))) void imx_testing_decode_handoff(int spin_limit, int withhold);

#endif /* IRONMLX_B200_TESTING_H */
