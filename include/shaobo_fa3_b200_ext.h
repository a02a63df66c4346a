/*
 * Extensions of this library that have no counterpart in the reference
 * project's headers.  A caller that only knows the reference ABI never needs
 * them.
 */
#ifndef SHAOBO_FA3_B200_EXT_H_
#define SHAOBO_FA3_B200_EXT_H_

#include "shaobo_fa3_api.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Device-side error flag.  Every wait inside the tensor-core kernels is
 * bounded; a wait that runs out makes the kernel stop cleanly and raise this
 * flag instead of hanging.  Returns 0 (no error), 1 (a bounded wait timed
 * out), 2 (dynamic shared memory was not 1 KiB aligned), or -1 if the flag
 * could not be read.  Synchronises the current device.  clear != 0 resets the
 * flag after reading it.  (No counterpart in the reference.) */
int shaobo_fa3_b200_device_error(int clear);

/* Per-stage device timing of shaobo_fa3_bwd_v2, for benchmarking.
 * enable != 0: create four CUDA events on the current device; every later v2
 * call records them around its three launches.  enable == 0: stop and destroy
 * them.  Off by default.  (No counterpart in the reference.) */
int shaobo_fa3_b200_stage_timing(int enable);

/* Milliseconds of the three stages of the last timed v2 call; waits for that
 * call.  Fused path: {delta, five-GEMM kernel, dQ convert}; deterministic
 * path: {delta, dK/dV kernel, dQ kernel}.  INVALID_VALUE when timing is off or
 * no call was timed.  (No counterpart in the reference.) */
int shaobo_fa3_b200_last_stage_ms(float* ms3);

#ifdef __cplusplus
}
#endif

#endif  /* SHAOBO_FA3_B200_EXT_H_ */
