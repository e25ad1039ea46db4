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

#endif /* IRONMLX_B200_TESTING_H */
