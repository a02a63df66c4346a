/*
 * Public C ABI of the B200-native FlashAttention-3 backward.
 *
 * This header is the drop-in boundary: a caller that was written against the
 * reference project's include/shaobo_fa3_api.h (reference file, lines 13-147)
 * compiles and links against this library unchanged.  Every enumerator value,
 * every field offset of ShaoboFa3Params (296 bytes on LP64) and every function
 * signature is the same as there; what differs is the capability set that
 * shaobo_fa3_bwd_get_capabilities reports and shaobo_fa3_bwd_v2_validate
 * accepts (BF16, head_dim 64, the [B,S,H,D] layout, sequence lengths that are
 * not multiples of 128 or differ between queries and keys, sliding windows,
 * packed sequences and softcap are supported here; the reference rejects all
 * of them: reference src/shaobo_fa3_bwd_api.cpp:53-68,109-118).
 *
 * Ownership: the library never allocates device memory in the entry points
 * declared here.  All tensors and the workspace are device pointers owned by
 * the caller.  Tensors are contiguous in the layout params->layout names:
 * [B,H,S,D] (SHAOBO_FA3_LAYOUT_BHSD, the reference's only layout) or
 * [B,S,H,D]; packed sequences are [total, H, D].
 *
 * Stream: launches go to the legacy default stream of the current device,
 * like the reference (which has no stream argument).  As a compatible
 * extension, a non-null reserved_ptr[SHAOBO_FA3_RESERVED_PTR_STREAM] is used
 * as the cudaStream_t of every launch of that call.
 */
#ifndef SHAOBO_FA3_API_H_
#define SHAOBO_FA3_API_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* reference include/shaobo_fa3_api.h:11 */
#define SHAOBO_FA3_API_VERSION 2u

/* Return codes (reference include/shaobo_fa3_api.h:13-19).  Value 4 keeps the
 * reference's name; here it reports a CUDA runtime / driver error. */
typedef enum ShaoboFa3Status {
    SHAOBO_FA3_STATUS_SUCCESS = 0,
    SHAOBO_FA3_STATUS_INVALID_VALUE = 1,
    SHAOBO_FA3_STATUS_UNSUPPORTED = 2,
    SHAOBO_FA3_STATUS_NOT_IMPLEMENTED = 3,
    SHAOBO_FA3_STATUS_HIP_ERROR = 4
} ShaoboFa3Status;
#define SHAOBO_FA3_STATUS_CUDA_ERROR SHAOBO_FA3_STATUS_HIP_ERROR

/* reference include/shaobo_fa3_api.h:21-25 */
typedef enum ShaoboFa3DType {
    SHAOBO_FA3_DTYPE_FP16 = 0,
    SHAOBO_FA3_DTYPE_BF16 = 1,
    SHAOBO_FA3_DTYPE_FP8 = 2
} ShaoboFa3DType;

/* reference include/shaobo_fa3_api.h:27-30 */
typedef enum ShaoboFa3Layout {
    SHAOBO_FA3_LAYOUT_BHSD = 0,
    SHAOBO_FA3_LAYOUT_BSHD = 1
} ShaoboFa3Layout;

/* reference include/shaobo_fa3_api.h:32-35.  SMAX_SSUM: aux0 = unscaled row
 * maximum of Q.K^T, aux1 = row sum of exp2((s-max)*scale*log2e).  LSE: aux0 =
 * natural-log log-sum-exp of the scaled scores. */
typedef enum ShaoboFa3SoftmaxAuxMode {
    SHAOBO_FA3_SOFTMAX_AUX_SMAX_SSUM = 0,
    SHAOBO_FA3_SOFTMAX_AUX_LSE = 1
} ShaoboFa3SoftmaxAuxMode;

/* Feature bits (reference include/shaobo_fa3_api.h:37-51). */
typedef uint64_t ShaoboFa3BwdFeatureMask;
#define SHAOBO_FA3_BWD_FEATURE_FIXED_LENGTH   (UINT64_C(1) << 0)
#define SHAOBO_FA3_BWD_FEATURE_VARLEN         (UINT64_C(1) << 1)
#define SHAOBO_FA3_BWD_FEATURE_FP16           (UINT64_C(1) << 2)
#define SHAOBO_FA3_BWD_FEATURE_BF16           (UINT64_C(1) << 3)
#define SHAOBO_FA3_BWD_FEATURE_CAUSAL         (UINT64_C(1) << 4)
#define SHAOBO_FA3_BWD_FEATURE_LOCAL_WINDOW   (UINT64_C(1) << 5)
#define SHAOBO_FA3_BWD_FEATURE_GQA            (UINT64_C(1) << 6)
#define SHAOBO_FA3_BWD_FEATURE_SOFTCAP        (UINT64_C(1) << 7)
#define SHAOBO_FA3_BWD_FEATURE_DETERMINISTIC  (UINT64_C(1) << 8)
#define SHAOBO_FA3_BWD_FEATURE_SOFTMAX_LSE    (UINT64_C(1) << 9)
#define SHAOBO_FA3_BWD_FEATURE_BSHD           (UINT64_C(1) << 10)
#define SHAOBO_FA3_BWD_FEATURE_BHSD           (UINT64_C(1) << 11)
#define SHAOBO_FA3_BWD_FEATURE_FULL_ATTENTION (UINT64_C(1) << 12)

/* Uses of the reserved slots.  Slots 0 and 3 of reserved_ptr and slots 0 and 1
 * of reserved_i32 carry the meaning the reference's split path gives them
 * (reference src/dq_kernel.cpp:1522-1547, src/dkv_kernel.cpp:1393-1406). */
#define SHAOBO_FA3_RESERVED_PTR_DELTA   0 /* shaobo_fa3_bwd_dq: fp32 delta [B,Hq,S] */
#define SHAOBO_FA3_RESERVED_PTR_SIDECAR 3 /* shaobo_fa3_bwd_dkv: packed sidecar [B,Hq,S,3] */
#define SHAOBO_FA3_RESERVED_PTR_STREAM  7 /* extension: cudaStream_t, NULL = default stream */

/* Values of dkv_path / dq_path understood by the component entry points
 * (reference include/dkv_contract.h:7-8, include/dq_contract.h:7-8). */
#define SHAOBO_FA3_DKV_PATH_REFERENCE 1
#define SHAOBO_FA3_DKV_PATH_CANONICAL 5
#define SHAOBO_FA3_DQ_PATH_REFERENCE  1
#define SHAOBO_FA3_DQ_PATH_CANONICAL  6

/* Parameter block (reference include/shaobo_fa3_api.h:53-99).  Byte offsets on
 * LP64 are given at the right; the tail after reserved_ptr was appended for
 * Tri Dao FA3 compatibility and is covered by struct_size. */
typedef struct ShaoboFa3Params {
    uint32_t struct_size;          /*   0  sizeof(ShaoboFa3Params) of the caller */

    int32_t batch;                 /*   4 */
    int32_t seqlen_q;              /*   8 */
    int32_t seqlen_k;              /*  12 */
    int32_t num_heads_q;           /*  16 */
    int32_t num_heads_kv;          /*  20 */
    int32_t head_dim_qk;           /*  24 */
    int32_t head_dim_v;            /*  28 */

    int32_t causal;                /*  32  0 or 1 */
    int32_t window_left;           /*  36  -1 = unbounded */
    int32_t window_right;          /*  40  -1 = unbounded */
    float softmax_scale;           /*  44  used when softmax_scale_is_set != 0 */
    float dropout_p;               /*  48  must be 0 */

    int32_t dtype;                 /*  52  ShaoboFa3DType */
    int32_t layout;                /*  56  ShaoboFa3Layout */
    int32_t softmax_aux_mode;      /*  60  ShaoboFa3SoftmaxAuxMode (components) */
    int32_t dkv_path;              /*  64  component selector */
    int32_t dq_path;               /*  68  component selector */
    int32_t block_threads;         /*  72  ignored */
    int32_t sync_after_launch;     /*  76  0 or 1 */

    const int32_t* cu_seqlens_q;   /*  80  packed sequences: device array of batch+1 offsets, or NULL */
    const int32_t* cu_seqlens_k;   /*  88 */
    int32_t max_seqlen_q;          /*  96 */
    int32_t max_seqlen_k;          /* 100 */

    void* workspace;               /* 104  device scratch owned by the caller */
    size_t workspace_bytes;        /* 112 */

    int32_t reserved_i32[16];      /* 120 */
    void* reserved_ptr[8];         /* 184 */

    const int32_t* seqused_q;      /* 248 */
    const int32_t* seqused_k;      /* 256 */
    int64_t total_q;               /* 264 */
    int64_t total_k;               /* 272 */
    float softcap;                 /* 280  0 = off; > 0: scores capped with softcap*tanh(x/softcap) */
    int32_t deterministic;         /* 284  0 or 1; 1 selects the atomic-free split path */
    int32_t sm_margin;             /* 288  must be 0 */
    int32_t softmax_scale_is_set;  /* 292  0 -> scale = 1/sqrt(head_dim_qk) */
} ShaoboFa3Params;

/* reference include/shaobo_fa3_api.h:101-109 */
typedef struct ShaoboFa3BwdCapabilities {
    uint32_t struct_size;
    uint32_t api_version;
    ShaoboFa3BwdFeatureMask feature_mask;
    int32_t min_head_dim;
    int32_t max_head_dim;
    int32_t head_dim_alignment;
    int32_t sequence_alignment;
} ShaoboFa3BwdCapabilities;

/* Zero-fill, set struct_size, window -1/-1, FP16, BHSD, AUX_LSE.
 * Replaces reference src/shaobo_fa3_bwd_api.cpp:160-171. */
void shaobo_fa3_params_init(ShaoboFa3Params* params);

/* The caller sets capabilities->struct_size first; too small a value returns
 * INVALID_VALUE.  Replaces reference src/shaobo_fa3_bwd_api.cpp:173-193. */
int shaobo_fa3_bwd_get_capabilities(ShaoboFa3BwdCapabilities* capabilities);

/* Capability validation, host only, no launch.  INVALID_VALUE checks come
 * before UNSUPPORTED checks.  Replaces reference
 * src/shaobo_fa3_bwd_api.cpp:70-120,195-198. */
int shaobo_fa3_bwd_v2_validate(const ShaoboFa3Params* params);

/* Bytes of params->workspace that shaobo_fa3_bwd_v2 needs; 0 when the
 * parameters are invalid or unsupported.  Replaces reference
 * src/shaobo_fa3_bwd_api.cpp:122-156,200-204.  The formula is this library's
 * own: one fp32 dQ accumulator [B,Hq,S,D] + delta + packed sidecar, instead of
 * the reference's per-K-tile dQ partials. */
size_t shaobo_fa3_bwd_v2_workspace_bytes(const ShaoboFa3Params* params);

/* Attention backward.  softmax_lse is the natural-log LSE of the forward,
 * fp32 [B,Hq,Sq]; softmax_d is optional (may be NULL) and receives
 * delta = rowsum(dout * out) in fp32 [B,Hq,Sq].  dq, dk, dv are written in the
 * input dtype.  Replaces reference src/shaobo_fa3_bwd_api.cpp:206-260.
 *
 * Wider than the reference (which returns UNSUPPORTED for all of these,
 * src/shaobo_fa3_bwd_api.cpp:53-68,109-118):
 *  - params->layout = BSHD: q, out, dout, dq are [B,Sq,Hq,D] and k, v, dk, dv
 *    are [B,Sk,Hkv,D], contiguous; softmax_lse and softmax_d stay [B,Hq,Sq].
 *  - seqlen_q and seqlen_k need not be multiples of 128.
 *  - seqlen_q != seqlen_k; with causal = 1 the diagonal is aligned to the
 *    bottom-right corner: query i sees key j iff j <= i + seqlen_k - seqlen_q.
 *    A query that sees no key (softmax_lse = -inf) gets a zero gradient.
 *  - window_left / window_right >= 0: sliding window, query i sees keys
 *    i + off - window_left .. i + off + window_right (off = seqlen_k - seqlen_q);
 *    a negative side is unbounded and causal = 1 forces window_right = 0.
 *  - cu_seqlens_q and cu_seqlens_k non-NULL (device arrays of batch+1 int32 row
 *    offsets): packed sequences.  q, out, dout, dq are [total_q, Hq, D], k, v,
 *    dk, dv are [total_k, Hkv, D], softmax_lse and softmax_d are [Hq, total_q];
 *    batch is the number of sequences; max_seqlen_q/k, total_q/k must be set
 *    and seqlen_q/k hold the maxima; layout is ignored.  Rows of dq/dk/dv
 *    outside every sequence are not part of the contract.
 *  - seqused_q / seqused_k non-NULL (device arrays of batch int32): only the
 *    first seqused[b] rows of batch entry b take part (with fixed-length
 *    batches and with packed sequences); the rows of dq/dk/dv behind them, up
 *    to the end of the entry, are written as zero.
 *  - softcap > 0: the scaled scores go through softcap * tanh(x / softcap)
 *    before the softmax (softmax_lse must come from such a forward).
 *
 * The call only enqueues work on the stream (params->reserved_ptr[7], NULL =
 * default stream) unless sync_after_launch is set.  The first call on a host
 * thread, and the first call that uses a given kernel variant on a device, do
 * one-time set-up through the runtime: make them outside stream capture. */
int shaobo_fa3_bwd_v2(const void* dout,
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

/* "success" | "invalid_value" | "unsupported" | "not_implemented" |
 * "hip_error" | "unknown".  Replaces reference src/dkv_kernel.cpp:1271-1286. */
const char* shaobo_fa3_status_string(int status);

/* Legacy names.  In the reference's standalone dKV build these forward to
 * shaobo_fa3_bwd_dkv_workspace_bytes / shaobo_fa3_bwd_dkv (reference
 * src/dkv_kernel.cpp:1423-1443); they do the same here. */
size_t shaobo_fa3_bwd_workspace_bytes(const ShaoboFa3Params* params);

int shaobo_fa3_bwd(const void* dout,
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

static_assert(sizeof(ShaoboFa3Params) == 296 || sizeof(void*) != 8,
              "ShaoboFa3Params must stay 296 bytes on LP64");
#endif

#endif  /* SHAOBO_FA3_API_H_ */
