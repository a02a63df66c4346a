// Three-GEMM dQ kernel for sm_100a: the dQ half of the atomic-free split path.
//
// One CTA owns one (batch, query head, 128-row query tile): Q and dO stay in
// shared memory, K and V tiles stream through a two-stage ring, and dQ is
// accumulated in tensor memory over all key tiles in a fixed order, so the
// result is bitwise reproducible and needs no workspace.  Per key tile:
//
//     S  = Q K^T      [query i on TMEM lanes, key j on columns]        SS MMA
//     dP = dO V^T                                                       SS MMA
//     dS = exp2(S*scale*log2e - m_i) * r_i * (dP - delta_i)  -> TMEM b16
//          (row statistics live in registers: thread i owns query row i)
//     dQ += dS K      A = dS from TMEM, B = K (MN-major)                TS MMA
//
// Tensor-memory ledger: S [0,128)  dP, then dS in place [128,256)  dQ [256,256+D).
// Shared-memory ledger: Q, dO resident (2 x D*256), K and V two stages each
// (4 x D*256), mbarriers 128: 196,736 bytes at D=128, 98,432 at D=64.
//
// Same math as reference src/dq_kernel.cpp:546-596 (S, dP, dS, dQ per K/V
// page with a resident Q/dO tile), restated for tcgen05.
#pragma once

#include <cuda.h>

#include <type_traits>

#include "fused_bwd_kernel.cuh"
#include "ptx.cuh"

namespace fa3b200 {

struct DqArgs {
    // Row statistics: the packed sidecar [B,Hq,Sq,3] = {m, r, delta}, or, when it is null, the three
    // arrays of the reference's calling convention (reference src/dq_kernel.cpp:1515-1549): aux0 and
    // aux1 = row maximum of the unscaled scores and row sum (or aux0 = log-sum-exp and aux1 = null),
    // and delta, each [B,Hq,Sq].
    const float* sidecar;
    const float* aux0;
    const float* aux1;
    const float* delta;
    void* dq;              // [B,Hq,Sq,D] or [B,Sq,Hq,D], see q_strides
    TensorStrides q_strides;  // element strides of dq
    int batch;
    int heads_q;
    int heads_kv;
    Band band;                // sequence lengths and the visible band (geometry.h); maxima when packed
    const int* cu_seqlens_q;  // non-null: packed sequences, see FusedArgs
    const int* cu_seqlens_k;
    const int* seqused_q;     // non-null: used lengths per batch entry, see FusedArgs
    const int* seqused_k;
    int sidecar_rows;         // rows per head of the sidecar (seqlen_q, or total_q when packed)
    float scale;
    float scale_log2;
    float softcap_pre;        // softcap variant, see FusedArgs
    float softcap_post;
};

template <int D>
struct DqCfg {
    static constexpr int kTile = 128;
    static constexpr int kThreads = 256;
    static constexpr int kBoxBytes = 128 * 128;
    static constexpr int kBoxes = D / 64;
    static constexpr int kOperandBytes = kBoxes * kBoxBytes;
    static constexpr int kStages = 2;
    static constexpr int kOffQ = 0;
    static constexpr int kOffDO = kOperandBytes;
    static constexpr int kOffK = 2 * kOperandBytes;
    static constexpr int kOffV = kOffK + kStages * kOperandBytes;
    static constexpr int kOffBar = kOffV + kStages * kOperandBytes;
    static constexpr int kSmemBytes = kOffBar + 128;
    static constexpr int kTmemCols = 512;
    static constexpr int kColS = 0;
    static constexpr int kColDP = 128;
    static constexpr int kColDQ = 256;
};

enum DqBar : int {
    kDqbQFull = 0,
    kDqbKvFull = 1,   // 2 stages
    kDqbKvEmpty = 3,  // 2 stages
    kDqbSFull = 5,
    kDqbDpFull = 6,
    kDqbSFree = 7,
    kDqbDsReady = 8,
    kDqbDone = 9,
    kDqbNum = 10,
};

template <typename T, int D, bool kCausal, typename TOut, bool kSoftcap = false>
__global__ void __launch_bounds__(256, 1)
dq_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
              const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
              const DqArgs a) {
    using C = DqCfg<D>;
    constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = ptx::smem_u32(smem);
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    auto bar = [&](int i) -> uint32_t { return sbase + C::kOffBar + 8 * i; };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + C::kOffBar + 8 * kDqbNum);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int n_q_tiles = tiles_of(a.band.seqlen_q);  // of the longest sequence
    const int bh_count = a.batch * a.heads_q;
    // heaviest query tiles (most visible keys) are launched first
    const int qt = kCausal ? n_q_tiles - 1 - int(blockIdx.x) / bh_count : int(blockIdx.x) / bh_count;
    const int bhi = int(blockIdx.x) % bh_count;
    const int b = bhi / a.heads_q;
    const int hq = bhi % a.heads_q;
    const int kvh = hq / (a.heads_q / a.heads_kv);
    // packed sequences: this batch entry's own lengths and first rows (see the five-GEMM kernel)
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
    const int slot_q = band.seqlen_q;  // rows of dQ this batch entry owns
    if (a.seqused_q != nullptr || a.seqused_k != nullptr) {
        if (a.seqused_q != nullptr) band.seqlen_q = max(0, min(band.seqlen_q, a.seqused_q[b]));
        if (a.seqused_k != nullptr) band.seqlen_k = max(0, min(band.seqlen_k, a.seqused_k[b]));
        band.off = band.seqlen_k - band.seqlen_q;
    }
    // key tiles k_begin .. k_begin + n_steps - 1 in ascending order; none when no key is visible or
    // the query tile lies past the end of this sequence
    const int k_begin = first_k_tile(qt, band);
    const int n_steps = qt * C::kTile < band.seqlen_q ? k_tiles_of_q_tile(qt, band) : 0;
    const bool misaligned = (sbase & 1023u) != 0;

    if (threadIdx.x == 0) {
        if (misaligned) atomicCAS(&g_device_error, kDevOk, kDevSmemMisaligned);
        ptx::mbar_init(bar(kDqbQFull), 1);
        for (int s = 0; s < 2; ++s) {
            ptx::mbar_init(bar(kDqbKvFull + s), 1);
            ptx::mbar_init(bar(kDqbKvEmpty + s), 1);
        }
        ptx::mbar_init(bar(kDqbSFull), 1);
        ptx::mbar_init(bar(kDqbDpFull), 1);
        ptx::mbar_init(bar(kDqbSFree), 128);
        ptx::mbar_init(bar(kDqbDsReady), 128);
        ptx::mbar_init(bar(kDqbDone), 1);
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
    const int q_row = qt * C::kTile;  // row inside the head

    if (!misaligned) {
        if (warp == 0) {
            if (lane == 0 && n_steps > 0) {  // nothing is loaded for a tile that sees no key
                ptx::prefetch_tensormap(&tm_q);
                ptx::prefetch_tensormap(&tm_k);
                ptx::prefetch_tensormap(&tm_v);
                ptx::prefetch_tensormap(&tm_do);
                ptx::mbar_arrive_expect_tx(bar(kDqbQFull), 2 * C::kOperandBytes);
#pragma unroll
                for (int bx = 0; bx < C::kBoxes; ++bx) {
                    ptx::tma_load_4d(sbase + C::kOffQ + bx * C::kBoxBytes, &tm_q, bar(kDqbQFull), bx * 64, q_base + q_row, hq, b_coord);
                    ptx::tma_load_4d(sbase + C::kOffDO + bx * C::kBoxBytes, &tm_do, bar(kDqbQFull), bx * 64, q_base + q_row, hq, b_coord);
                }
#pragma unroll 1
                for (int t = 0; t < n_steps; ++t) {
                    const int s = t & 1;
                    const int kv_row = k_base + (k_begin + t) * C::kTile;
                    if (!bounded_wait(bar(kDqbKvEmpty + s), ((t >> 1) & 1) ^ 1, abort_flag)) break;
                    ptx::mbar_arrive_expect_tx(bar(kDqbKvFull + s), 2 * C::kOperandBytes);
#pragma unroll
                    for (int bx = 0; bx < C::kBoxes; ++bx) {
                        ptx::tma_load_4d(sbase + C::kOffK + s * C::kOperandBytes + bx * C::kBoxBytes, &tm_k,
                                         bar(kDqbKvFull + s), bx * 64, kv_row, kvh, b_coord);
                        ptx::tma_load_4d(sbase + C::kOffV + s * C::kOperandBytes + bx * C::kBoxBytes, &tm_v,
                                         bar(kDqbKvFull + s), bx * 64, kv_row, kvh, b_coord);
                    }
                }
            }
        } else if (warp == 1) {
            // MMA issuer: the whole warp runs the role converged; the lean issue forms and the commits
            // elect their lane inside the asm (a lone divergent lane is starved by the math warps).
            {
                constexpr uint32_t kIdSdP = ptx::instr_desc_f16(kBf16, 128, 128, false, false);
                constexpr uint32_t kIdDq = ptx::instr_desc_f16(kBf16, 128, D, false, true);
                constexpr uint32_t kHi = ptx::kDescHiSw128;
                constexpr uint32_t kBoxStep = C::kBoxBytes >> 4;
                auto k_step = [](int kk) -> uint32_t { return uint32_t(kk >> 2) * kBoxStep + uint32_t(kk & 3) * 2u; };
                auto mn_step = [](int kk) -> uint32_t { return uint32_t(kk) * 128u; };
                const uint32_t loQ = ptx::desc_lo_k_major(sbase + C::kOffQ);
                const uint32_t loDO = ptx::desc_lo_k_major(sbase + C::kOffDO);
                auto sK = [&](int t) { return sbase + C::kOffK + (t & 1) * C::kOperandBytes; };
                auto sV = [&](int t) { return sbase + C::kOffV + (t & 1) * C::kOperandBytes; };
                auto issue_s = [&](int t) {
                    const uint32_t loK = ptx::desc_lo_k_major(sK(t));
                    ptx::mma_ss_lean<false>(tmem + C::kColS, loQ, loK, kHi, kIdSdP);
#pragma unroll
                    for (int kk = 1; kk < D / 16; ++kk)
                        ptx::mma_ss_lean<true>(tmem + C::kColS, loQ + k_step(kk), loK + k_step(kk), kHi, kIdSdP);
                    ptx::tc_commit_elect(bar(kDqbSFull));
                };
                auto issue_dp = [&](int t) {
                    const uint32_t loV = ptx::desc_lo_k_major(sV(t));
                    ptx::mma_ss_lean<false>(tmem + C::kColDP, loDO, loV, kHi, kIdSdP);
#pragma unroll
                    for (int kk = 1; kk < D / 16; ++kk)
                        ptx::mma_ss_lean<true>(tmem + C::kColDP, loDO + k_step(kk), loV + k_step(kk), kHi, kIdSdP);
                    ptx::tc_commit_elect(bar(kDqbDpFull));
                };
                bool ok = n_steps > 0 && warp_wait<false>(bar(kDqbQFull), 0, abort_flag) &&
                          warp_wait<false>(bar(kDqbKvFull + 0), 0, abort_flag);
                if (ok) {
                    ptx::tc_fence_after();
                    issue_s(0);
                    issue_dp(0);
                }
#pragma unroll 1
                for (int t = 0; ok && t < n_steps; ++t) {
                    const bool more = t + 1 < n_steps;
                    if (more) {
                        // S(t) is in registers: S(t+1) may overwrite it
                        if (!(ok = warp_wait<false>(bar(kDqbSFree), t & 1, abort_flag))) break;
                        if (!(ok = warp_wait<false>(bar(kDqbKvFull + ((t + 1) & 1)), ((t + 1) >> 1) & 1, abort_flag))) break;
                        ptx::tc_fence_after();
                        issue_s(t + 1);
                    }
                    if (!(ok = warp_wait<false>(bar(kDqbDsReady), t & 1, abort_flag))) break;
                    ptx::tc_fence_after();
                    {
                        const uint32_t loK = ptx::desc_lo_mn_major(sK(t), C::kBoxBytes);
                        ptx::mma_ts_lean_rt(tmem + C::kColDQ, tmem + C::kColDP, loK, kHi, kIdDq, t > 0 ? 1u : 0u);
#pragma unroll
                        for (int kk = 1; kk < 8; ++kk)
                            ptx::mma_ts_lean<true>(tmem + C::kColDQ, tmem + C::kColDP + kk * 8, loK + mn_step(kk), kHi, kIdDq);
                    }
                    if (more) issue_dp(t + 1);  // after dQ(t) in issue order: dS(t) is consumed first
                    ptx::tc_commit_elect(bar(kDqbKvEmpty + (t & 1)));
                }
                if (ok) ptx::tc_commit_elect(bar(kDqbDone));  // never reached without steps: nobody waits then
            }
        } else if (warp >= 4) {
            const int i = threadIdx.x - 128;  // query row inside the tile == TMEM lane
            const uint32_t tl = tmem + (uint32_t((warp & 3) * 32) << 16);
            const int qi = q_row + i;  // query row inside the head
            const bool q_valid = qi < band.seqlen_q;
            // rows past the end of the sequence: P = exp2(-inf) = 0
            // P = exp2(x - m) * r = exp2(x + (log2 r - m)); a row that saw no key (m = -inf or r = 0) gets -inf
            const int64_t stat_row = int64_t(b_coord * a.heads_q + hq) * a.sidecar_rows + q_base + (q_valid ? qi : 0);
            float neg = -INFINITY, delta = 0.0f;
            if (q_valid) {
                if (a.sidecar != nullptr) {
                    const float* side = a.sidecar + stat_row * 3;
                    neg = __log2f(side[1]) - side[0];
                    delta = side[2];
                } else {
                    const float x = a.aux0[stat_row];
                    if (a.aux1 == nullptr) {
                        neg = x == -INFINITY ? -INFINITY : -x * 1.44269504088896340736f;
                    } else {
                        const float sum = a.aux1[stat_row];
                        neg = (x == -INFINITY || sum == 0.0f) ? -INFINITY : -__log2f(sum) - x * a.scale_log2;
                    }
                    delta = a.delta[stat_row];
                }
            }
            uint32_t ppk[64];
            bool ok = true;
#pragma unroll 1
            for (int t = 0; t < n_steps; ++t) {
                if (!(ok = warp_wait(bar(kDqbSFull), t & 1, abort_flag))) break;
                ptx::tc_fence_after();
                // element (query i, key j) survives iff mask_from <= j <= mask_to (band edges, end of keys)
                const bool diagonal = kCausal && tile_needs_mask(k_begin + t, qt, band);
                int mask_from, mask_to;
                key_range_of_query(qi, (k_begin + t) * C::kTile, band, &mask_from, &mask_to);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t r[32];
                    ptx::tmem_ld32(tl + C::kColS + c * 32, r);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        float p0, p1;
                        if (kSoftcap) {
                            p0 = ptx::ex2_approx(fmaf(a.softcap_post, ptx::tanh_approx(__uint_as_float(r[e + 0]) * a.softcap_pre), neg));
                            p1 = ptx::ex2_approx(fmaf(a.softcap_post, ptx::tanh_approx(__uint_as_float(r[e + 1]) * a.softcap_pre), neg));
                        } else {
                            p0 = ptx::ex2_approx(fmaf(__uint_as_float(r[e + 0]), a.scale_log2, neg));
                            p1 = ptx::ex2_approx(fmaf(__uint_as_float(r[e + 1]), a.scale_log2, neg));
                        }
                        if (diagonal) {
                            const int j = c * 32 + e;
                            p0 = (j + 0 >= mask_from && j + 0 <= mask_to) ? p0 : 0.0f;
                            p1 = (j + 1 >= mask_from && j + 1 <= mask_to) ? p1 : 0.0f;
                        }
                        ppk[c * 16 + e / 2] = ptx::Pack2<T>::pack(p0, p1);
                    }
                }
                ptx::tc_fence_before();
                ptx::mbar_arrive(bar(kDqbSFree));
                if (!(ok = warp_wait(bar(kDqbDpFull), t & 1, abort_flag))) break;
                ptx::tc_fence_after();
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t r[32];
                    ptx::tmem_ld32(tl + C::kColDP + c * 32, r);
                    ptx::tmem_ld_wait();
                    uint32_t o[16];
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        const float2 p = ptx::Pack2<T>::unpack(ppk[c * 16 + e / 2]);
                        float ds0 = p.x * (__uint_as_float(r[e + 0]) - delta);
                        float ds1 = p.y * (__uint_as_float(r[e + 1]) - delta);
                        if (kSoftcap) {
                            // slope 1 - tanh^2 of the cap, with tanh recovered from P and the row's reference
                            const float inv_post = 1.0f / a.softcap_post;
                            const float t0 = (__log2f(p.x) - neg) * inv_post, t1 = (__log2f(p.y) - neg) * inv_post;
                            ds0 = p.x > 0.0f ? ds0 * fmaxf(1.0f - t0 * t0, 0.0f) : 0.0f;
                            ds1 = p.y > 0.0f ? ds1 * fmaxf(1.0f - t1 * t1, 0.0f) : 0.0f;
                        }
                        o[e / 2] = ptx::Pack2<T>::pack(ds0, ds1);
                    }
                    // dS chunk c lands on columns [16c, 16c+16) of the dP region,
                    // all of which were read by chunk loads <= c
                    ptx::tmem_st16(tl + C::kColDP + c * 16, o);
                }
                ptx::tmem_st_wait();
                ptx::tc_fence_before();
                ptx::mbar_arrive(bar(kDqbDsReady));
            }
            if (ok && n_steps > 0) ok = warp_wait(bar(kDqbDone), 0, abort_flag);
            TOut* dst = reinterpret_cast<TOut*>(a.dq) + b_coord * a.q_strides.batch + hq * a.q_strides.head +
                        int64_t(q_base + qi) * a.q_strides.row;
            if (ok && ((q_valid && n_steps == 0) || (!q_valid && qi < slot_q))) {
                // no visible key at all, or a row behind the used length: the gradient is zero
                uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
                for (int e = 0; e < int(D * sizeof(TOut) / 16); ++e) d4[e] = make_uint4(0u, 0u, 0u, 0u);
            }
            __syncwarp();
            if (ok && n_steps > 0) {
                // (tensor-memory loads are warp-wide: every lane runs them, only the stores of query
                // rows past the end of the sequence are skipped)
                ptx::tc_fence_after();
#pragma unroll
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t r[32];
                    ptx::tmem_ld32(tl + C::kColDQ + c * 32, r);
                    ptx::tmem_ld_wait();
                    if (q_valid) {
                    if (sizeof(TOut) == 4) {
                        float4* d4 = reinterpret_cast<float4*>(dst + c * 32);
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            d4[e] = make_float4(__uint_as_float(r[4 * e]) * a.scale, __uint_as_float(r[4 * e + 1]) * a.scale,
                                                __uint_as_float(r[4 * e + 2]) * a.scale, __uint_as_float(r[4 * e + 3]) * a.scale);
                    } else {
                        uint4* d4 = reinterpret_cast<uint4*>(dst + c * 32);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            uint4 o;
                            o.x = ptx::Pack2<T>::pack(__uint_as_float(r[8 * e + 0]) * a.scale, __uint_as_float(r[8 * e + 1]) * a.scale);
                            o.y = ptx::Pack2<T>::pack(__uint_as_float(r[8 * e + 2]) * a.scale, __uint_as_float(r[8 * e + 3]) * a.scale);
                            o.z = ptx::Pack2<T>::pack(__uint_as_float(r[8 * e + 4]) * a.scale, __uint_as_float(r[8 * e + 5]) * a.scale);
                            o.w = ptx::Pack2<T>::pack(__uint_as_float(r[8 * e + 6]) * a.scale, __uint_as_float(r[8 * e + 7]) * a.scale);
                            d4[e] = o;
                        }
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
