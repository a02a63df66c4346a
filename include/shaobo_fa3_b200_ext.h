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

/* Size of the scratch array built into the library for
 * shaobo_fa3_b200_bwd_v2_noalloc: 32 MiB on every GPU that loads the library,
 * held until the process exits. */
#define SHAOBO_FA3_B200_STATIC_SCRATCH_BYTES (32u << 20)

/* shaobo_fa3_bwd_v2 for callers that cannot allocate device memory.  (No
 * counterpart in the reference.)
 *
 * Who needs it: code that runs where cudaMalloc is off limits - a plugin
 * living inside a host framework's fixed memory arena, a latency-critical loop
 * that must not allocate after start-up, a job whose device memory was sized
 * by its launcher.  Such a caller can pass inputs and outputs but has no
 * workspace to offer, and shaobo_fa3_bwd_v2 needs one.
 *
 * What it does: the same computation as shaobo_fa3_bwd_v2, same arguments and
 * results, except that params->workspace and params->workspace_bytes are
 * ignored: the scratch is a fixed array of
 * SHAOBO_FA3_B200_STATIC_SCRATCH_BYTES inside the library.  It holds what the
 * workspace of shaobo_fa3_bwd_v2 holds: the fp32 dQ accumulator
 * (4*B*Hq*Sq*D bytes), on small problems whose key tiles are split over
 * several thread blocks the partial dK/dV sums of those blocks (512*D bytes
 * per block for fp16 inputs, 1024*D for bf16 inputs, up to 148 blocks), delta
 * and the packed sidecar (16 bytes per query row).  The call performs no cudaMalloc, no cudaFree and no other
 * allocating runtime or library call.
 *
 * Limit: the problem must satisfy
 *     shaobo_fa3_bwd_v2_workspace_bytes(params) <= SHAOBO_FA3_B200_STATIC_SCRATCH_BYTES
 * (ask that function; e.g. B=1,H=4,S=2048,D=128 fp16 needs 13 MiB and
 * B=1,H=15,S=4096,D=128 31 MiB, B=2,H=16,S=2048,D=128 does not fit).  A larger
 * problem returns SHAOBO_FA3_STATUS_UNSUPPORTED and launches nothing.  Status
 * codes otherwise follow shaobo_fa3_bwd_v2 in the same order: parameter
 * validation first, then NULL tensor pointers (INVALID_VALUE), then this limit.
 *
 * First call: the first call on each device looks up the device address of the
 * array (one runtime query, with that device current).  Make that first call
 * outside any stream capture.
 *
 * Sharing: every call on a device uses the same array, which still holds what
 * the previous call left there; the part that must start at zero (the dQ
 * accumulator) is cleared by the call itself.  Two calls that overlap in time
 * on one GPU (different streams, or different host threads) race on the array
 * and give wrong results: run them one after the other. */
int shaobo_fa3_b200_bwd_v2_noalloc(const void* dout,
                                   const void* q,
                                   const void* k,
                                   const void* v,
                                   const void* out,
                                   const void* softmax_lse,
                                   void* dq,
                                   void* dk,
                                   void* dv,
                                   void* softmax_d,
                                   const ShaoboFa3Params* params);

/* shaobo_fa3_bwd_v2 for tensors that live in HOST memory (pinned for full
 * speed): dout, q, k, v, out, softmax_lse are read from and dq, dk, dv written
 * to host buffers; [B,H,S,D] layout, fixed lengths (other parameter blocks
 * return UNSUPPORTED).  No counterpart in the reference.
 *
 * The call copies the inputs to the GPU, runs the backward and copies the
 * gradients back, cut into (batch, KV head) shards that are pipelined over
 * three internal streams so that copies in both directions and kernels overlap
 * (over PCIe the copies bound such a call).  `staging` is device memory owned
 * by the caller, at least shaobo_fa3_b200_bwd_v2_host_staging_bytes(params)
 * bytes; params->workspace is ignored.  The work is enqueued behind the
 * caller's stream (params->reserved_ptr[7], NULL = default stream), which is
 * made to wait for it: the host outputs are valid once that stream has been
 * synchronised, or on return with sync_after_launch = 1.  The internal streams
 * and events are created on the first call per device (outside stream
 * capture) and kept; calls that overlap in time must use different staging. */
size_t shaobo_fa3_b200_bwd_v2_host_staging_bytes(const ShaoboFa3Params* params);
int shaobo_fa3_b200_bwd_v2_host(const void* dout,
                                const void* q,
                                const void* k,
                                const void* v,
                                const void* out,
                                const void* softmax_lse,
                                void* dq,
                                void* dk,
                                void* dv,
                                void* staging,
                                size_t staging_bytes,
                                const ShaoboFa3Params* params);

/* Attention forward: out = softmax(q k^T * scale) v and softmax_lse = the
 * natural-log log-sum-exp of every row, i.e. the two tensors shaobo_fa3_bwd_v2
 * takes next to q, k, v.  No counterpart in the reference, which is a backward
 * only and expects them from the caller's forward
 * (reference docs/tridao_fa3_bwd_api.md:48-55).
 *
 * Same parameter block, validation and status codes as shaobo_fa3_bwd_v2 (all
 * layouts, lengths, windows and packed sequences it accepts); `deterministic`
 * and the workspace fields are ignored, nothing is allocated.  out has the
 * shape, dtype and layout of q; softmax_lse is fp32 [B,Hq,Sq] ([Hq,total_q]
 * for packed sequences).  A query that sees no key gets out = 0 and
 * softmax_lse = -inf. */
int shaobo_fa3_b200_fwd(const void* q,
                        const void* k,
                        const void* v,
                        void* out,
                        void* softmax_lse,
                        const ShaoboFa3Params* params);

#ifdef __cplusplus
}
#endif

#endif  /* SHAOBO_FA3_B200_EXT_H_ */
