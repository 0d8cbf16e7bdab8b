/*
 * chxq_testing.h - entry points of libchxq.so that exist for measurements and tests only.  Nothing here has a counterpart in
 * the reference, and no product code path depends on any of it: the switches are process-wide and default to "off".
 */
#ifndef CHXQ_TESTING_H_
#define CHXQ_TESTING_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* The tensor-core path has two kernels with identical results: one output tile per step (every epilogue), and grouped
 * tiles whose uint8 outputs leave through shared memory and a TMA store (uint8 requantizing epilogues with 16-byte
 * aligned output rows); the second also has forms for stride-1 convolutions up to 3 x 3 that stage the input halo tile
 * once per tile instead of once per tap.  0 = choose by problem shape (default), 1 = always the first, 2 = the second
 * whenever eligible, 3 = the second with halo tiles (planes of 16-byte rows) whenever eligible, 4 (and 5) = halo tiles stored
 * swizzled.  A third kernel runs dense layers with at least 256 output
 * channels and a 128-byte K tile on CTA pairs (tcgen05.mma.cta_group::2, a 256 x 256 block per pair): 6 = as 0 but never
 * that kernel, 7 = that kernel whenever the problem is eligible, however small.  Packed 3 x 3 depthwise layers over a zero-point-0
 * uint8 map run on the CUDA-core row kernel with TMA-staged rows by default; 2..5 keep them as diagonal blocks on the tensor cores,
 * 1 also takes the plain-load row kernel for maps TMA cannot describe.  Process-wide; meant for measurements and tests. */
int chxq_tc_variant(int32_t variant);

/* The bounded device-side waits of the tensor-core kernels give up after wait_limit_ns without progress (default 2 s; 1 ms ..
 * 10 s here), set the device status word (chxq_device_status -> CHXQ_ERR_DEVICE_TIMEOUT), and the CTA tears down in order:
 * nothing traps or spins on.  skip_weight_load_kb >= 0 makes the one-tile kernel's producer leave out the weight load of that K
 * block, so that its stage never fills: the way a test makes a wait run out.  (-1: off, the default.)  Process-wide. */
int chxq_tc_test_hooks(int64_t wait_limit_ns, int32_t skip_weight_load_kb);

/* Number of CTA pairs (clusters of two) of the paired tensor-core kernel that the current device keeps resident at once
 * (cudaOccupancyMaxActiveClusters): the kernel's grid is twice this, or smaller for small problems. */
int chxq_tc_pair_slots(int32_t* slots);


#ifdef __cplusplus
}
#endif
#endif /* CHXQ_TESTING_H_ */
