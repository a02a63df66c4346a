// Attention forward for sm_100a: O = softmax(Q K^T * scale) V and the log-sum-exp of every row, the
// two tensors the backward needs next to Q, K, V.  Same tile geometry, masks, layouts and packed
// sequences as the backward kernels (geometry.h).
//
// One CTA owns one (batch, query head) and TWO neighbouring 128-row query tiles, A and B.  Both Q tiles
// stay in shared memory, K and V tiles stream through two-stage rings and are used by both query
// tiles, and each query tile has its own softmax warpgroup, score buffer and output accumulator in
// tensor memory.  Per key tile and query tile:
//
//     S  = Q K^T          [query i on TMEM lanes, key j on columns]           SS MMA
//     m  = max(m, rowmax S),  P = exp2((S - m) * scale*log2e),  l = l*alpha + rowsum P
//          (thread i owns query row i: no shuffles; P is written over S as 16-bit pairs)
//     O += P V            A = P from TMEM, B = V (MN-major)                   TS MMA
//
// The two query tiles alternate on the tensor pipe: while the softmax warpgroup of tile A works on
// S_A(t), the pipe computes S_B(t) and P_B V, and the other way round.
// The running maximum is updated lazily: a row keeps its reference maximum until the new maximum
// exceeds it by more than 2^8, so P stays below 256 and the accumulator only has to be rescaled
// (tensor memory -> registers -> tensor memory) on the rare steps where some row of a warp moves
// its reference.  The result is exact: O and l carry the same factor, which cancels in O / l.
//
// Tensor-memory ledger: S_A [0,128)  S_B [128,256)  O_A [256,256+D)  O_B [256+D,256+2D).
// Shared-memory ledger: Q_A, Q_B resident (2 x D*256), K and V two stages each (4 x D*256),
// mbarriers 256: 196,864 bytes at D=128, 98,560 at D=64.
#pragma once

#include <cuda.h>

#include <type_traits>

#include "fused_bwd_kernel.cuh"
#include "geometry.h"
#include "ptx.cuh"

namespace fa3b200 {

struct FwdArgs {
    void* out;                // [B,Hq,Sq,D] or [B,Sq,Hq,D] (or [total_q,Hq,D]), see o_strides
    float* lse;               // [B,Hq,Sq] natural log ([Hq,total_q] when packed)
    TensorStrides o_strides;  // element strides of out
    int batch;
    int heads_q;
    int heads_kv;
    Band band;                // sequence lengths and the visible band; maxima when packed
    const int* cu_seqlens_q;  // non-null: packed sequences, see FusedArgs
    const int* cu_seqlens_k;
    const int* seqused_q;     // non-null: used lengths per batch entry, see FusedArgs; rows behind them
    const int* seqused_k;     // get out = 0 and lse = -inf
    int lse_rows;             // rows per head of lse (seqlen_q, or total_q when packed)
    float scale_log2;         // softmax scale * log2(e)
    float softcap_pre;        // softcap variant: scores become softcap_post * tanh(score * softcap_pre),
    float softcap_post;       // with softcap_pre = scale / softcap and softcap_post = softcap * log2(e)
};

template <int D>
struct FwdCfg {
    static constexpr int kTile = 128;
    static constexpr int kThreads = 384;
    static constexpr int kBoxBytes = 128 * 128;
    static constexpr int kBoxes = D / 64;
    static constexpr int kOperandBytes = kBoxes * kBoxBytes;
    static constexpr int kStages = 2;
    static constexpr int kOffQ = 0;                                  // two query tiles
    static constexpr int kOffK = 2 * kOperandBytes;
    static constexpr int kOffV = kOffK + kStages * kOperandBytes;
    static constexpr int kOffBar = kOffV + kStages * kOperandBytes;
    static constexpr int kSmemBytes = kOffBar + 256;
    static_assert(kSmemBytes <= 232448, "shared-memory ledger exceeds 227 KiB");
    static constexpr int kTmemCols = 512;
    static constexpr int kColS = 0;     // + 128 per query tile
    static constexpr int kColO = 256;   // + D per query tile
    static_assert(kColO + 2 * D <= kTmemCols, "tensor-memory ledger exceeds 512 columns");
    static constexpr float kRescaleThreshold = 8.0f;  // log2 units
    // setmaxnreg split: the kernel starts with 168 registers per thread (384 threads); the producer /
    // MMA warpgroup gives most of its share to the two softmax warpgroups, which hold a whole score
    // row (128 values) in registers
    static constexpr int kRegsControl = 64;
    static constexpr int kRegsSoftmax = 216;
    static_assert(kRegsControl + 2 * kRegsSoftmax <= 504, "more registers than the CTA was launched with (168 x 384)");
};

enum FwdBar : int {
    kFwdQFull = 0,    // per query tile
    kFwdKFull = 2,    // 2 stages
    kFwdKEmpty = 4,   // 2 stages
    kFwdVFull = 6,    // 2 stages
    kFwdVEmpty = 8,   // 2 stages
    kFwdSFull = 10,   // per query tile
    kFwdPReady = 12,  // per query tile
    kFwdPvDone = 14,  // per query tile
    kFwdNum = 16,
};

// kSoftcap: the scaled scores go through softcap * tanh(x / softcap) before the softmax.
template <typename T, int D, bool kMasked, bool kSoftcap = false>
__global__ void __launch_bounds__(384, 1)
fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
           const __grid_constant__ CUtensorMap tm_v, const FwdArgs a) {
    using C = FwdCfg<D>;
    constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = ptx::smem_u32(smem);
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    auto bar = [&](int i) -> uint32_t { return sbase + C::kOffBar + 8 * i; };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + C::kOffBar + 8 * kFwdNum);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int n_pairs = (tiles_of(a.band.seqlen_q) + 1) / 2;  // of the longest sequence
    const int bh_count = a.batch * a.heads_q;
    // heaviest query tiles (most visible keys) are launched first
    const int pair = kMasked ? n_pairs - 1 - int(blockIdx.x) / bh_count : int(blockIdx.x) / bh_count;
    const int bhi = int(blockIdx.x) % bh_count;
    const int b = bhi / a.heads_q;
    const int hq = bhi % a.heads_q;
    const int kvh = hq / (a.heads_q / a.heads_kv);
    // packed sequences: this batch entry's own lengths and first rows
    Band band = a.band;
    int q_base = 0, k_base = 0, b_coord = b;
    if (a.cu_seqlens_q != nullptr) {
        q_base = a.cu_seqlens_q[b];
        k_base = a.cu_seqlens_k[b];
        band.seqlen_q = a.cu_seqlens_q[b + 1] - q_base;
        band.seqlen_k = a.cu_seqlens_k[b + 1] - k_base;
        band.off = band.seqlen_k - band.seqlen_q;
        b_coord = 0;
    }
    const int slot_q = band.seqlen_q;  // rows of out this batch entry owns
    if (a.seqused_q != nullptr || a.seqused_k != nullptr) {
        if (a.seqused_q != nullptr) band.seqlen_q = max(0, min(band.seqlen_q, a.seqused_q[b]));
        if (a.seqused_k != nullptr) band.seqlen_k = max(0, min(band.seqlen_k, a.seqused_k[b]));
        band.off = band.seqlen_k - band.seqlen_q;
    }
    // Query tile x (0 = A, 1 = B) visits key tiles first[x] .. first[x] + count[x] - 1; count is 0 when
    // no key is visible or the tile lies past the end of this sequence.  The CTA walks the union.
    int first[2], count[2];
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        const int qt = 2 * pair + x;
        first[x] = first_k_tile(qt, band);
        count[x] = qt * C::kTile < band.seqlen_q ? k_tiles_of_q_tile(qt, band) : 0;
    }
    int t_begin = 0, t_end = -1;  // inclusive range of key tiles
    if (count[0] > 0 && count[1] > 0) {
        t_begin = min(first[0], first[1]);
        t_end = max(first[0] + count[0], first[1] + count[1]) - 1;
    } else if (count[0] > 0) {
        t_begin = first[0];
        t_end = first[0] + count[0] - 1;
    } else if (count[1] > 0) {
        t_begin = first[1];
        t_end = first[1] + count[1] - 1;
    }
    const int n_iter = t_end - t_begin + 1;
    auto active = [&](int x, int t) { return t >= first[x] && t < first[x] + count[x]; };
    const bool misaligned = (sbase & 1023u) != 0;

    if (threadIdx.x == 0) {
        if (misaligned) atomicCAS(&g_device_error, kDevOk, kDevSmemMisaligned);
        for (int s = 0; s < 2; ++s) {
            ptx::mbar_init(bar(kFwdQFull + s), 1);
            ptx::mbar_init(bar(kFwdKFull + s), 1);
            ptx::mbar_init(bar(kFwdKEmpty + s), 1);
            ptx::mbar_init(bar(kFwdVFull + s), 1);
            ptx::mbar_init(bar(kFwdVEmpty + s), 1);
            ptx::mbar_init(bar(kFwdSFull + s), 1);
            ptx::mbar_init(bar(kFwdPReady + s), 128);
            ptx::mbar_init(bar(kFwdPvDone + s), 1);
        }
        *abort_flag = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), C::kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    // (each role changes its register budget at the top of its own branch, where the compiler can see
    // which code runs under which budget)
    if (warp < 4) {
        ptx::setmaxnreg_dec<C::kRegsControl>();
        if (misaligned) {
            // nothing to do
        } else if (warp == 0) {
            if (lane == 0 && n_iter > 0) {
                ptx::prefetch_tensormap(&tm_q);
                ptx::prefetch_tensormap(&tm_k);
                ptx::prefetch_tensormap(&tm_v);
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    if (count[x] == 0) continue;  // nothing is loaded for a tile that sees no key
                    ptx::mbar_arrive_expect_tx(bar(kFwdQFull + x), C::kOperandBytes);
#pragma unroll
                    for (int bx = 0; bx < C::kBoxes; ++bx) {
                        ptx::tma_load_4d(sbase + C::kOffQ + x * C::kOperandBytes + bx * C::kBoxBytes, &tm_q,
                                         bar(kFwdQFull + x), bx * 64, q_base + (2 * pair + x) * C::kTile, hq, b_coord);
                    }
                }
#pragma unroll 1
                for (int it = 0; it < n_iter; ++it) {
                    const int s = it & 1;
                    const uint32_t wait_parity = ((it >> 1) & 1) ^ 1;
                    const int kv_row = k_base + (t_begin + it) * C::kTile;
                    if (!bounded_wait(bar(kFwdKEmpty + s), wait_parity, abort_flag)) break;
                    ptx::mbar_arrive_expect_tx(bar(kFwdKFull + s), C::kOperandBytes);
#pragma unroll
                    for (int bx = 0; bx < C::kBoxes; ++bx) {
                        ptx::tma_load_4d(sbase + C::kOffK + s * C::kOperandBytes + bx * C::kBoxBytes, &tm_k,
                                         bar(kFwdKFull + s), bx * 64, kv_row, kvh, b_coord);
                    }
                    if (!bounded_wait(bar(kFwdVEmpty + s), wait_parity, abort_flag)) break;
                    ptx::mbar_arrive_expect_tx(bar(kFwdVFull + s), C::kOperandBytes);
#pragma unroll
                    for (int bx = 0; bx < C::kBoxes; ++bx) {
                        ptx::tma_load_4d(sbase + C::kOffV + s * C::kOperandBytes + bx * C::kBoxBytes, &tm_v,
                                         bar(kFwdVFull + s), bx * 64, kv_row, kvh, b_coord);
                    }
                }
            }
        } else if (warp == 1) {
            // MMA issuer: the whole warp runs the role converged; the lean issue forms and the commits
            // elect their lane inside the asm.
            constexpr uint32_t kIdS = ptx::instr_desc_f16(kBf16, 128, 128, false, false);
            constexpr uint32_t kIdO = ptx::instr_desc_f16(kBf16, 128, D, false, true);
            constexpr uint32_t kHi = ptx::kDescHiSw128;
            constexpr uint32_t kBoxStep = C::kBoxBytes >> 4;
            auto k_step = [](int kk) -> uint32_t { return uint32_t(kk >> 2) * kBoxStep + uint32_t(kk & 3) * 2u; };
            auto mn_step = [](int kk) -> uint32_t { return uint32_t(kk) * 128u; };
            // S of query tile x against the key tile in ring slot `it`
            auto issue_s = [&](int x, int it) {
                const uint32_t loQ = ptx::desc_lo_k_major(sbase + C::kOffQ + x * C::kOperandBytes);
                const uint32_t loK = ptx::desc_lo_k_major(sbase + C::kOffK + (it & 1) * C::kOperandBytes);
                const uint32_t dst = tmem + C::kColS + x * 128;
                ptx::mma_ss_lean<false>(dst, loQ, loK, kHi, kIdS);
#pragma unroll
                for (int kk = 1; kk < D / 16; ++kk)
                    ptx::mma_ss_lean<true>(dst, loQ + k_step(kk), loK + k_step(kk), kHi, kIdS);
                ptx::tc_commit_elect(bar(kFwdSFull + x));
            };
            auto issue_pv = [&](int x, int it, bool accumulate) {
                const uint32_t loV = ptx::desc_lo_mn_major(sbase + C::kOffV + (it & 1) * C::kOperandBytes, C::kBoxBytes);
                const uint32_t p_cols = tmem + C::kColS + x * 128;
                const uint32_t o_cols = tmem + C::kColO + x * D;
                ptx::mma_ts_lean_rt(o_cols, p_cols, loV, kHi, kIdO, accumulate ? 1u : 0u);
#pragma unroll
                for (int kk = 1; kk < 8; ++kk)
                    ptx::mma_ts_lean<true>(o_cols, p_cols + kk * 8, loV + mn_step(kk), kHi, kIdO);
                ptx::tc_commit_elect(bar(kFwdPvDone + x));
            };
            bool ok = n_iter > 0;
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                if (ok && count[x] > 0) ok = warp_wait<false>(bar(kFwdQFull + x), 0, abort_flag);
            }
            if (ok) ok = warp_wait<false>(bar(kFwdKFull + 0), 0, abort_flag);
            if (ok) {
                ptx::tc_fence_after();
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    if (active(x, t_begin)) issue_s(x, 0);
                }
                ptx::tc_commit_elect(bar(kFwdKEmpty + 0));
            }
            int done[2] = {0, 0};  // local step counters of the two query tiles
#pragma unroll 1
            for (int it = 0; ok && it < n_iter; ++it) {
                const int t = t_begin + it;
                const bool more = it + 1 < n_iter;
                bool v_ready = false, k_ready = false;
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    if (active(x, t)) {
                        if (!(ok = warp_wait<false>(bar(kFwdPReady + x), done[x] & 1, abort_flag))) break;
                        if (!v_ready) {
                            if (!(ok = warp_wait<false>(bar(kFwdVFull + (it & 1)), (it >> 1) & 1, abort_flag))) break;
                            v_ready = true;
                        }
                        ptx::tc_fence_after();
                        issue_pv(x, it, done[x] > 0);
                        ++done[x];
                    }
                    // S of the next key tile goes over P of this one: it follows P V in the pipe
                    if (more && active(x, t + 1)) {
                        if (!k_ready) {
                            if (!(ok = warp_wait<false>(bar(kFwdKFull + ((it + 1) & 1)), ((it + 1) >> 1) & 1, abort_flag))) break;
                            k_ready = true;
                        }
                        ptx::tc_fence_after();
                        issue_s(x, it + 1);
                    }
                }
                if (!ok) break;
                if (more) ptx::tc_commit_elect(bar(kFwdKEmpty + ((it + 1) & 1)));
                ptx::tc_commit_elect(bar(kFwdVEmpty + (it & 1)));
            }
        }
    } else {
        ptx::setmaxnreg_inc<C::kRegsSoftmax>();
        if (!misaligned) {
            const int x = (warp - 4) >> 2;      // which query tile
            const int i = threadIdx.x & 127;    // query row inside the tile == TMEM lane
            const int qt = 2 * pair + x;
            const int n_steps = x == 0 ? count[0] : count[1];  // (selects, not indexing: no local array)
            const int k_begin = x == 0 ? first[0] : first[1];
            const uint32_t tl = tmem + (uint32_t((warp & 3) * 32) << 16);
            const uint32_t s_cols = tl + C::kColS + x * 128;
            const uint32_t o_cols = tl + C::kColO + x * D;
            const int qi = qt * C::kTile + i;  // query row inside the head
            const bool q_valid = qi < band.seqlen_q;
            float m_ref = -INFINITY;  // reference maximum (raw scores) the exponentials are taken against
            float l = 0.0f;           // sum of the exponentials, in units of exp2(m_ref * scale_log2)
            const float sl = kSoftcap ? 1.0f : a.scale_log2;  // log2 units per unit of (transformed) score
            bool ok = true;
#pragma unroll 1
            for (int u = 0; u < n_steps; ++u) {
                if (!(ok = warp_wait(bar(kFwdSFull + x), u & 1, abort_flag))) break;
                ptx::tc_fence_after();
                // key j of this tile survives for query i iff mask_from <= j <= mask_to
                const bool diagonal = kMasked && tile_needs_mask(k_begin + u, qt, band);
                int mask_from = 0, mask_to = 0;
                if (diagonal) key_range_of_query(qi, (k_begin + u) * C::kTile, band, &mask_from, &mask_to);
                // ---- the whole score row of this tile goes to registers in one round trip
                uint32_t r[4][32];
#pragma unroll
                for (int c = 0; c < 4; ++c) ptx::tmem_ld32(s_cols + c * 32, r[c]);
                ptx::tmem_ld_wait();
                if (kSoftcap) {
                    // capped scores, already in log2 units: from here on they are used with a scale of 1
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
#pragma unroll
                        for (int e = 0; e < 32; ++e) {
                            r[c][e] = __float_as_uint(a.softcap_post *
                                                      ptx::tanh_approx(__uint_as_float(r[c][e]) * a.softcap_pre));
                        }
                    }
                }
                float mt = -INFINITY;
                if (diagonal) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
#pragma unroll
                        for (int e = 0; e < 32; ++e) {
                            const int j = c * 32 + e;
                            if (j >= mask_from && j <= mask_to) mt = fmaxf(mt, __uint_as_float(r[c][e]));
                        }
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
#pragma unroll
                        for (int e = 0; e < 32; ++e) mt = fmaxf(mt, __uint_as_float(r[c][e]));
                    }
                }
                // ---- move the reference maximum only when it is more than 2^8 too small
                float alpha = 1.0f;
                const bool move = (mt - m_ref) * sl > C::kRescaleThreshold;  // also -inf -> finite
                if (move) {
                    alpha = ptx::ex2_approx((m_ref - mt) * sl);  // exp2(-inf) = 0 on the first move
                    m_ref = mt;
                    l *= alpha;
                }
                if (u > 0 && __any_sync(0xffffffffu, move)) {
                    // O carries the old reference: wait for P V of step u-1, then rescale these 32 rows
                    if (!(ok = warp_wait(bar(kFwdPvDone + x), (u - 1) & 1, abort_flag))) break;
                    ptx::tc_fence_after();
                    // (16 columns at a time: the score row is still held in registers)
#pragma unroll 1
                    for (int c = 0; c < D / 16; ++c) {
                        uint32_t acc[16];
                        ptx::tmem_ld16(o_cols + c * 16, acc);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int e = 0; e < 16; ++e) acc[e] = __float_as_uint(__uint_as_float(acc[e]) * alpha);
                        ptx::tmem_st16(o_cols + c * 16, acc);
                    }
                    ptx::tmem_st_wait();
                }
                // ---- P = exp2((S - m_ref) * scale_log2), written over S as 16-bit pairs (every column of
                // S has been read by now)
                const float neg = m_ref == -INFINITY ? 0.0f : -m_ref * sl;
                float sum = 0.0f;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t o[16];
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        float p0 = ptx::ex2_approx(fmaf(__uint_as_float(r[c][e + 0]), sl, neg));
                        float p1 = ptx::ex2_approx(fmaf(__uint_as_float(r[c][e + 1]), sl, neg));
                        if (diagonal) {
                            const int j = c * 32 + e;
                            p0 = (j + 0 >= mask_from && j + 0 <= mask_to) ? p0 : 0.0f;
                            p1 = (j + 1 >= mask_from && j + 1 <= mask_to) ? p1 : 0.0f;
                        }
                        sum += p0 + p1;
                        o[e / 2] = ptx::Pack2<T>::pack(p0, p1);
                    }
                    ptx::tmem_st16(s_cols + c * 16, o);
                }
                l += sum;
                ptx::tmem_st_wait();
                ptx::tc_fence_before();
                ptx::mbar_arrive(bar(kFwdPReady + x));
            }
            if (ok && n_steps > 0) ok = warp_wait(bar(kFwdPvDone + x), (n_steps - 1) & 1, abort_flag);
            T* dst = reinterpret_cast<T*>(a.out) + b_coord * a.o_strides.batch + hq * a.o_strides.head +
                     int64_t(q_base + qi) * a.o_strides.row;
            float* lse_dst = a.lse + int64_t(b_coord * a.heads_q + hq) * a.lse_rows + q_base + qi;
            if (ok && ((q_valid && n_steps == 0) || (!q_valid && qi < slot_q))) {
                // no visible key at all, or a row behind the used length: O = 0, lse = -inf
                uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
                for (int e = 0; e < D / 8; ++e) d4[e] = make_uint4(0u, 0u, 0u, 0u);
                *lse_dst = -INFINITY;
            }
            __syncwarp();
            if (ok && n_steps > 0) {
                // (tensor-memory loads are warp-wide: every lane runs them, only the stores of query rows
                // past the end of the sequence are skipped)
                ptx::tc_fence_after();
                const float inv = l > 0.0f ? 1.0f / l : 0.0f;
                if (q_valid) {
                    // ln(sum exp(s*scale)) = (m_ref*scale_log2 + log2 l) * ln 2
                    *lse_dst = l > 0.0f ? (m_ref * sl + __log2f(l)) * 0.69314718055994531f : -INFINITY;
                }
#pragma unroll
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t r[32];
                    ptx::tmem_ld32(o_cols + c * 32, r);
                    ptx::tmem_ld_wait();
                    if (q_valid) {
                        uint4* d4 = reinterpret_cast<uint4*>(dst + c * 32);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            uint4 o;
                            o.x = ptx::Pack2<T>::pack(__uint_as_float(r[8 * e + 0]) * inv, __uint_as_float(r[8 * e + 1]) * inv);
                            o.y = ptx::Pack2<T>::pack(__uint_as_float(r[8 * e + 2]) * inv, __uint_as_float(r[8 * e + 3]) * inv);
                            o.z = ptx::Pack2<T>::pack(__uint_as_float(r[8 * e + 4]) * inv, __uint_as_float(r[8 * e + 5]) * inv);
                            o.w = ptx::Pack2<T>::pack(__uint_as_float(r[8 * e + 6]) * inv, __uint_as_float(r[8 * e + 7]) * inv);
                            d4[e] = o;
                        }
                    }
                    __syncwarp();  // reconverge before the next warp-wide load
                }
            }
        }
    }

    __syncwarp();
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem, C::kTmemCols);
    }
}

}  // namespace fa3b200
