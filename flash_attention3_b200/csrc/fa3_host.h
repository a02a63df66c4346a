// Host-side helpers shared by the validation layer (fa3_api.cpp, plain C++)
// and the launch layer (fa3_launch.cu).  Nothing here touches CUDA.
#pragma once

#include <cstddef>
#include <cstdint>

#include "geometry.h"
#include "shaobo_fa3_api.h"

namespace fa3b200 {

constexpr size_t kWorkspaceAlignment = 256;  // same as reference src/shaobo_fa3_bwd_api.cpp:16
constexpr int kSequenceAlignment = 128;      // K/Q tile edge; reference :18 (lengths need not be multiples)
constexpr int kMinHeadDim = 64;
constexpr int kMaxHeadDim = 128;
constexpr int kSidecarFields = 3;            // {m, r, delta}; reference src/dot_do_o_kernel.cpp:11

// Overflow-checked size arithmetic (role of reference
// src/shaobo_fa3_bwd_api.cpp:28-51).
bool mul_ok(size_t a, size_t b, size_t* out);
bool add_ok(size_t a, size_t b, size_t* out);
bool round_up_256(size_t bytes, size_t* out);

inline bool head_dim_supported(int d) { return d == 64 || d == 128; }
inline bool layout_supported(int l) {
    return l == SHAOBO_FA3_LAYOUT_BHSD || l == SHAOBO_FA3_LAYOUT_BSHD;
}
inline bool dtype_supported(int t) {
    return t == SHAOBO_FA3_DTYPE_FP16 || t == SHAOBO_FA3_DTYPE_BF16;
}

// Packed ("varlen") sequences: q, out, dout, dq are [total_q, Hq, D] and k, v, dk, dv are
// [total_k, Hkv, D]; sequence b owns rows cu_seqlens[b] .. cu_seqlens[b+1]-1 (device arrays of
// batch+1 int32).  softmax_lse, delta and the sidecar are [Hq, total_q].  max_seqlen_q / max_seqlen_k
// bound the per-sequence lengths and size the launch.
inline bool is_varlen(const ShaoboFa3Params* p) {
    return p->cu_seqlens_q != nullptr || p->cu_seqlens_k != nullptr;
}
// seqused_q / seqused_k (device arrays of batch int32): only the first seqused[b] rows of batch entry
// b take part; works with fixed-length batches and with packed sequences.
inline bool has_seqused(const ShaoboFa3Params* p) {
    return p->seqused_q != nullptr || p->seqused_k != nullptr;
}
// Length the launch is planned for: the sequence length, or the longest sequence when packed.
inline int plan_seqlen_q(const ShaoboFa3Params* p) { return is_varlen(p) ? p->max_seqlen_q : p->seqlen_q; }
inline int plan_seqlen_k(const ShaoboFa3Params* p) { return is_varlen(p) ? p->max_seqlen_k : p->seqlen_k; }

// The visible band of a parameter block (window_left / window_right: negative = unbounded; causal
// forces right = 0, as reference src/shaobo_fa3_bwd_api.cpp:53-68 normalises it).
inline Band band_of(const ShaoboFa3Params* p) {
    return make_band(plan_seqlen_q(p), plan_seqlen_k(p), p->causal != 0, p->window_left, p->window_right);
}

// Public validation used by every v2 entry.
int validate_v2(const ShaoboFa3Params* p);

// Shape test shared by the fused stage and its workspace formula: positive
// dims, Hq % Hkv == 0, D in {64,128}, Dqk == Dv.
bool fused_shape_ok(const ShaoboFa3Params* p);

// Bytes of the fp32 dQ accumulator [B,Hq,S,D] rounded up to 256; 0 on
// overflow or unsupported shape.
size_t dq_accum_bytes(const ShaoboFa3Params* p);

// Splitting of key tiles on small problems.  Shapes with fewer (batch x KV head x key tile) units
// than a B200 has SMs would leave most of the chip idle, so the query steps of every key tile are
// cut into chunks of `chunk_steps` steps, one CTA per chunk; every CTA writes its dK/dV partial sums
// to its own fp32 slab and the convert kernel adds the slabs of a tile in chunk order.  The chunk
// size is the one with the smallest modelled makespan when the CTAs, longest first, are handed to
// 148 SMs as they free up (a CTA costs a fixed part worth 3.5 steps plus its steps); that may be
// more CTAs than SMs: the overflow are the shortest ones and run on the SMs that free up first.
// The decision depends on the parameters only, so the workspace formula and the launch always
// agree.  The deterministic path never splits.
constexpr int kSplitSmCount = 148;
struct SplitPlan {
    int chunk_steps = 0;      // 0 = no splitting
    int chunks_per_head = 0;  // CTAs per (batch, KV head)
};
SplitPlan split_plan(const ShaoboFa3Params* p);

// Bytes of the per-CTA partial-sum slabs of split tiles (one dK and one dV slab of [128][D] per CTA,
// fp16 for fp16 inputs and fp32 for bf16 inputs); 0 when tiles are not split.
size_t dkv_accum_bytes(const ShaoboFa3Params* p);

// Carving of the caller's workspace by shaobo_fa3_bwd_v2:
//   [0, dq_accum)                fp32 dQ accumulator
//   [dq_accum, +dkv_accum)       fp32 dK / dV partial-sum slabs (only when tiles are split)
//   [delta_offset, +rows*4)      delta, used when softmax_d is NULL
//   [sidecar_offset, +rows*12)   packed sidecar
// Each region starts on a 256-byte boundary.
struct V2Workspace {
    size_t dq_accum_bytes = 0;
    size_t dkv_accum_bytes = 0;
    size_t delta_offset = 0;
    size_t sidecar_offset = 0;
    size_t total_bytes = 0;
    bool valid = false;
};
V2Workspace v2_workspace(const ShaoboFa3Params* p);

// Workspace of the naive fp32 device reference used by dkv_path/dq_path == 1:
// prob[rows,Sk] + dp[rows,Sk] + row_max + row_sum + delta
// (reference src/dkv_kernel.cpp:88-97).
size_t naive_reference_bytes(const ShaoboFa3Params* p);

}  // namespace fa3b200
