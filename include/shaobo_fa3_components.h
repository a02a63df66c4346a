/*
 * Stage-level entry points of the FlashAttention-3 backward: the pieces that
 * shaobo_fa3_bwd_v2 chains, exported one by one so that a harness or a
 * profiler can run a single stage.  Names, argument order and status codes
 * follow the reference project's include/shaobo_fa3_components.h (lines
 * 10-58); each declaration below cites the reference definition it replaces.
 *
 * Shared conventions
 *   - all pointers are device pointers owned by the caller; BHSD contiguous;
 *   - the packed sidecar is fp32 [B,Hq,S,3] = {m, r, delta} per query row with
 *     P = exp2(s*scale*log2e - m) * r.  In LSE mode m = lse*log2e and r = 1;
 *     in SMAX_SSUM mode m = rowmax*scale*log2e and r = 1/rowsum (0 if the sum
 *     is 0) (reference src/dot_do_o_kernel.cpp:49-62);
 *   - launches are asynchronous unless params->sync_after_launch is 1.
 */
#ifndef SHAOBO_FA3_COMPONENTS_H_
#define SHAOBO_FA3_COMPONENTS_H_

#include "shaobo_fa3_api.h"

#ifdef __cplusplus
extern "C" {
#endif

/* delta[r] = sum_d dout[r,d]*out[r,d] (fp32) and the packed sidecar.
 * scores_max is the LSE in LSE mode (scores_sum may then be NULL).
 * UNSUPPORTED for a dtype / head_dim / layout / aux mode outside the
 * capability set, INVALID_VALUE for a NULL tensor.
 * Replaces reference src/dot_do_o_kernel.cpp:78-125. */
int shaobo_fa3_bwd_dot_do_o(const void* dout,
                            const void* out,
                            const void* scores_max,
                            const void* scores_sum,
                            void* delta,
                            void* packed_sidecar,
                            const ShaoboFa3Params* params);

/* Workspace of the fused five-GEMM stage: one fp32 dQ accumulator
 * [B,Hq,S,D], rounded up to 256 bytes; 0 for parameters it cannot run.
 * Replaces reference src/fused_bwd_dq_reduce.cpp:154-202,281-284. */
size_t shaobo_fa3_bwd_fused5_workspace_bytes(const ShaoboFa3Params* params);

/* Fused five-GEMM backward from a packed sidecar: S, dP, dV, dK, dQ in one
 * kernel, GQA groups reduced inside it, then the dQ accumulator is scaled and
 * converted.  dq, dk, dv are written in the input dtype.  The stage clears its
 * workspace itself.  Replaces reference src/fused_bwd_kernel.cpp:1673-1764
 * together with the two reductions of src/fused_bwd_dq_reduce.cpp:225-279. */
int shaobo_fa3_bwd_fused5(const void* dout,
                          const void* q,
                          const void* k,
                          const void* v,
                          const void* packed_sidecar,
                          void* dq,
                          void* dk,
                          void* dv,
                          const ShaoboFa3Params* params);

/* Split path, dK/dV half (four GEMMs, no atomics, bitwise reproducible).
 * dkv_path selects SHAOBO_FA3_DKV_PATH_CANONICAL (tensor-core kernel; the
 * sidecar is passed in reserved_ptr[SHAOBO_FA3_RESERVED_PTR_SIDECAR]; dk and
 * dv are fp32 [B,Hkv,S,D]; no workspace).  SHAOBO_FA3_DKV_PATH_REFERENCE (the
 * reference's naive fp32 debug kernels, src/dkv_kernel.cpp:1086-1266) is not
 * built: NOT_IMPLEMENTED, and the size function reports the workspace that
 * path would need.  out, softmax_aux0/1 and dq are ignored, as in the
 * reference.
 * Replaces reference src/dkv_kernel.cpp:1288-1421. */
size_t shaobo_fa3_bwd_dkv_workspace_bytes(const ShaoboFa3Params* params);

int shaobo_fa3_bwd_dkv(const void* dout,
                       const void* q,
                       const void* k,
                       const void* v,
                       const void* out,
                       const void* softmax_aux0,
                       const void* softmax_aux1,
                       void* dq,
                       void* dk,
                       void* dv,
                       const ShaoboFa3Params* params);

/* Split path, dQ half (three GEMMs, no atomics, no workspace, bitwise
 * reproducible); dq is fp32 [B,Hq,S,D]; out, dk and dv are ignored.
 * dq_path must be SHAOBO_FA3_DQ_PATH_CANONICAL (the tensor-core kernel).
 * The row statistics are taken, in this order of preference, from
 *   (a) the reference's convention (src/dq_kernel.cpp:1515-1549):
 *       softmax_aux0 / softmax_aux1 = row maximum of the unscaled scores and
 *       row sum, [B,Hq,S] fp32 each (or the log-sum-exp and NULL when
 *       softmax_aux_mode is SHAOBO_FA3_SOFTMAX_AUX_LSE), with delta [B,Hq,S]
 *       in reserved_ptr[SHAOBO_FA3_RESERVED_PTR_DELTA]; used when all of
 *       them are non-NULL;
 *   (b) the packed sidecar of shaobo_fa3_bwd_dot_do_o in
 *       reserved_ptr[SHAOBO_FA3_RESERVED_PTR_SIDECAR], as for the dK/dV half.
 * INVALID_VALUE when neither form is complete.
 * SHAOBO_FA3_DQ_PATH_REFERENCE (the reference's naive fp32 debug kernels,
 * src/dq_kernel.cpp:955-1130) is not built: NOT_IMPLEMENTED, and its
 * workspace size function reports what that path would need.
 * Replaces reference src/dq_kernel.cpp:1486-1630. */
size_t shaobo_fa3_bwd_dq_workspace_bytes(const ShaoboFa3Params* params);

int shaobo_fa3_bwd_dq(const void* dout,
                      const void* q,
                      const void* k,
                      const void* v,
                      const void* out,
                      const void* softmax_aux0,
                      const void* softmax_aux1,
                      void* dq,
                      void* dk,
                      void* dv,
                      const ShaoboFa3Params* params);

#ifdef __cplusplus
}  /* extern "C" */
#endif

#endif  /* SHAOBO_FA3_COMPONENTS_H_ */
