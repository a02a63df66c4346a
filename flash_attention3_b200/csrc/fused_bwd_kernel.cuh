// Fused five-GEMM attention backward for sm_100a.
//
// One CTA owns one (batch, KV head, 128-key tile) and walks every 128-row query
// tile that can see those keys, for each of the G query heads that share the
// KV head.  dK and dV stay in tensor memory for the whole walk, so a GQA group
// is reduced inside the kernel and written once.  Per query tile ("step"):
//
//     S^T  = K  Q^T        [key j on TMEM lanes, query i on columns]   SS MMA
//     dP^T = V  dO^T                                                    SS MMA
//     P^T  = exp2(S^T * scale*log2e - m_i) * r_i      (CUDA cores, -> TMEM b16)
//     dV  += P^T dO        A = P^T from TMEM, B = dO (MN-major)         TS MMA
//     dS^T = P^T o (dP^T - delta_i)                   (CUDA cores, -> smem b16)
//     dK  += dS^T Q        A = dS^T (K-major), B = Q (MN-major)         SS MMA
//     dQ   = dS K          A = dS^T read MN-major, B = K (MN-major)     SS MMA
//     dQacc[tile] += dQ    TMEM -> regs -> smem -> TMA reduce-add (fp32)
//
// The softmax scale is applied once at the end (dK in the epilogue, dQ in the
// convert kernel) instead of per element of dS.
//
// Epilogue: when the last MMA has completed, every softmax warp stages its 32 key rows of dK
// (scaled) or dV over the dead Q / dO / dS^T buffers in the layout of a swizzled TMA box and one
// lane stores them with the copy engine.  On problems too small to fill the GPU the query steps
// of a key tile are cut into chunks, one CTA each (a table in the kernel parameters says which,
// longest chunks first); such a CTA stores its partial dK / dV to its own slab and the convert
// kernel adds the slabs of a tile in chunk order.
//
// Warp roles (512 threads, four warpgroups): warp 0 = TMA producer, warp 1 = MMA
// issuer and TMEM owner; warps 4-7 and 8-11 = two softmax / dS warpgroups (thread
// j of each owns TMEM lane j = key j; the first takes queries 0-63 of the tile,
// the second queries 64-127); warps 12-15 = dQ drain warpgroup.  Registers are
// re-split with setmaxnreg (96 / 112 / 112 / 176 per thread at D=128).  All hand-offs go
// through mbarriers; every wait is bounded and a time-out raises an error flag
// instead of hanging.
//
// Tensor-memory ledger (512 columns x 128 lanes x 32 bit):
//     D = 128:  dK [0,128)  dV [128,256)  S/P [256,384)  dP and dQ share [384,512)
//     D =  64:  dK [0,64)   dV [64,128)   S/P [128,256)  dP [256,384)  dQ [384,448)
// P^T (16-bit, two per column) is written over S^T in place: queries 0-63 on the
// first 32 columns of the S region, queries 64-127 on columns 64-95, so that each
// softmax warpgroup only overwrites columns it has already read itself.
//
// Shared-memory ledger (bytes; every tile is made of 16 KiB boxes of
// [128 rows][64 x 16 bit] in the 128-byte swizzle):
//     K, V            2 x D*256            resident for the CTA
//     Q               2 stages x D*256
//     dO              1 stage (D=128) or 2 stages (D=64) x D*256
//     dS^T            32 KiB               [128 keys][128 queries]
//     dQ staging      32 KiB               4 warps x 2 boxes of [32 rows][32 fp32]
//     row statistics  2 KiB / 3 KiB        {-m + log2 r, delta} x 128 rows x 2 buffers (D=128) / 3 (D=64)
//     mbarriers       256
//     total           231,680 (D=128) / 167,168 (D=64)   of 232,448 available
#pragma once

#include <cuda.h>

#include <type_traits>

#include "geometry.h"
#include "ptx.cuh"

namespace fa3b200 {

enum DeviceError : int {
    kDevOk = 0,
    kDevWaitTimeout = 1,
    kDevSmemMisaligned = 2,
};

// First error raised by any kernel since the flag was last cleared.
__device__ int g_device_error = 0;

#ifdef FA3B200_TRACE
// Instrumented builds only: cycle stamps of every CTA, by role (0 producer, 1 MMA warp,
// 2 first softmax warp, 3 first drain warp) and event slot.
constexpr int kTraceCtas = 1024;
constexpr int kTraceEvents = 64;
__device__ long long g_trace[kTraceCtas][4][kTraceEvents];
__device__ long long g_trace_rowwise[4];  // {delta first start, delta last end, convert first start, convert last end} (globaltimer)
__device__ __forceinline__ long long trace_globaltimer() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define TRACE(role, ev) do { if ((threadIdx.x & 31) == 0 && blockIdx.x < kTraceCtas && (ev) < kTraceEvents) g_trace[blockIdx.x][role][ev] = clock64(); } while (0)
#define TRACE_GT(role, ev) do { if ((threadIdx.x & 31) == 0 && blockIdx.x < kTraceCtas) g_trace[blockIdx.x][role][ev] = trace_globaltimer(); } while (0)
#else
#define TRACE(role, ev) do {} while (0)
#define TRACE_GT(role, ev) do {} while (0)
#endif

struct FusedArgs {
    const float* sidecar;  // [B,Hq,Sq,3] = {m, r, delta} per query row (packed sequences: [Hq, total_q, 3])
    void* dk;              // [B,Hkv,Sk,D] or [B,Sk,Hkv,D], see kv_strides
    void* dv;
    void* dkv_slabs;       // split tiles: a CTA writes its partial dK (scaled) to slab 2x and dV to slab 2x+1,
                           // each [128 rows][D], fp16 for fp16 inputs and fp32 for bf16 inputs; the convert
                           // kernel adds the slabs of a tile
    TensorStrides kv_strides;  // element strides of dk / dv
    int batch;
    int heads_q;
    int heads_kv;
    Band band;             // sequence lengths and the visible band (geometry.h); with packed
                           // sequences the lengths are the maxima and each CTA reads its own
    const int* cu_seqlens_q;  // non-null: sequences are packed ([total, H, D] tensors) and sequence b
    const int* cu_seqlens_k;  // owns rows cu[b] .. cu[b+1]-1; the tensor maps then have batch = 1
    const int* seqused_q;     // non-null: only the first seqused[b] rows of batch entry b take part; the
    const int* seqused_k;     // gradient rows behind them, up to the end of the entry's slot, are zero
    int sidecar_rows;      // rows per head of the sidecar / accumulators (seqlen_q, or total_q when packed)
    float scale;
    float scale_log2;
    // softcap variant: the scaled scores go through softcap * tanh(x / softcap) before the softmax;
    // in log2 units that is softcap_post * tanh(score * softcap_pre), softcap_pre = scale / softcap,
    // softcap_post = softcap * log2(e)
    float softcap_pre;
    float softcap_post;
    int order_mode;        // see cta_order.h
    int order_width;
    int head_group;        // heads per scheduling group: block = (group * n_tiles + tile slot) * head_group + head
    int chunk_steps;       // > 0: the steps of a key tile are cut into chunks of this many steps, one CTA
                           // per chunk, and the partial dK/dV of every chunk go to its own fp32 slab
    int chunks_per_head;   // number of chunks of one (batch, KV head) when chunk_steps > 0
    // chunk_steps > 0: which chunk CTA x runs, longest chunks first.  Entry = key tile | chunk index
    // inside the tile << 8 | slab << 16, where slab = (batch, KV head) * chunks_per_head + the chunk's
    // place in the head's list (key tile 0 first): the CTA's partial dK goes to slab 2*slab, dV to 2*slab+1.
    uint32_t cta_table[kMaxSplitCtas];
};

__host__ __device__ inline int remap_k_tile(int physical, int count, int mode, int width) {
    if (mode == 0) return physical;                 // heaviest (lowest index) first
    if (mode == 1) return count - 1 - physical;     // lightest first
    // mode 2: serpentine inside rounds of `width` tiles
    const int round = physical / width;
    const int base = round * width;
    const int slot = physical - base;
    int span = count - base;
    if (span > width) span = width;
    return base + ((round & 1) == 0 ? slot : span - 1 - slot);
}

template <int D>
struct FusedCfg {
    static constexpr int kTile = 128;
    static constexpr int kThreads = 512;
    static constexpr int kBoxBytes = 128 * 128;
    static constexpr int kBoxes = D / 64;
    static constexpr int kOperandBytes = kBoxes * kBoxBytes;
    static constexpr int kQStages = 2;
    static constexpr int kDoStages = D == 128 ? 1 : 2;
    static constexpr int kDsBytes = 2 * kBoxBytes;
    static constexpr int kStageBoxBytes = 32 * 128;
    static constexpr int kStageBytes = 4 * 2 * kStageBoxBytes;

    static constexpr int kOffK = 0;
    static constexpr int kOffV = kOffK + kOperandBytes;
    static constexpr int kOffQ = kOffV + kOperandBytes;
    static constexpr int kOffDO = kOffQ + kQStages * kOperandBytes;
    static constexpr int kOffDS = kOffDO + kDoStages * kOperandBytes;
    static constexpr int kOffStage = kOffDS + kDsBytes;
    static constexpr int kOffStats = kOffStage + kStageBytes;
    // Row statistics: kStatsBufs buffers of 128 x {log2 r - m} followed by as many of 128 x {delta}.  With three
    // buffers (D=64, where the softmax warpgroups bound the step) a step's statistics are written one
    // step ahead, so nobody waits for the writers; D=128 has no shared memory left for a third.
    static constexpr int kStatsBufs = D == 64 ? 3 : 2;
    static constexpr int kOffBar = kOffStats + kStatsBufs * 1024;
    static constexpr int kSmemBytes = kOffBar + 256;
    static_assert(kSmemBytes <= 232448, "shared-memory ledger exceeds 227 KiB");
    static_assert(kOffStage % 1024 == 0 && kOffDS % 1024 == 0, "swizzled regions need 1 KiB alignment");

    // setmaxnreg split per warpgroup (producer+MMA / softmax x2 / drain); sums to <= 512
    static constexpr int kRegsControl = 96;
    static constexpr int kRegsCompute = D == 128 ? 112 : 136;
    static constexpr int kRegsDrain = D == 128 ? 176 : 136;
    static_assert(kRegsControl + 2 * kRegsCompute + kRegsDrain <= 512, "register file over-committed");

    static constexpr int kTmemCols = 512;
    static constexpr int kColDK = 0;
    static constexpr int kColDV = D;
    static constexpr int kColS = 2 * D;
    static constexpr int kColDP = 2 * D + 128;
    static constexpr int kColDQ = D == 128 ? kColDP : kColDP + 128;
    static_assert(kColDQ + D <= kTmemCols, "tensor-memory ledger exceeds 512 columns");
    static_assert(8 * (D / 32) * kStageBoxBytes <= kOffStage - kOffQ, "epilogue staging does not fit");
};

enum Bar : int {
    kKvFull = 0,
    kQFull = 1,     // 2 stages
    kQEmpty = 3,    // 2 stages
    kDoFull = 5,    // up to 2 stages
    kDoEmpty = 7,   // up to 2 stages
    kSFull = 9,
    kDpFull = 10,
    kPReady = 11,
    kDsReady = 12,
    kDqFull = 13,
    kDqEmpty = 14,
    kDkvFull = 15,
    kStatsFull = 16,  // 2 buffers (not used where the statistics are published a step ahead)
    kNumBars = 18,
};

constexpr long long kWaitTimeoutCycles = 2000000000LL;  // about one second

// Bounded mbarrier wait.  Returns false when the wait timed out here or was
// abandoned because another thread of the CTA timed out.
template <bool kBackoff = false>
__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity,
                                             volatile uint32_t* abort_flag) {
#pragma unroll 1
    for (int i = 0; i < 4; ++i) {
        if (ptx::mbar_try_wait(bar, parity)) return true;
    }
    const long long start = clock64();
#pragma unroll 1
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 16; ++i) {
            if (ptx::mbar_try_wait(bar, parity)) return true;
            if (kBackoff) __nanosleep(32);  // keep a waiting warp off the issue ports
        }
        if (*abort_flag != 0) return false;
        if (clock64() - start > kWaitTimeoutCycles) {
            *abort_flag = 1;
            atomicCAS(&g_device_error, kDevOk, kDevWaitTimeout);
            return false;
        }
    }
}

template <bool kBackoff = true>
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity,
                                          volatile uint32_t* abort_flag) {
    const bool ok = bounded_wait<kBackoff>(bar, parity, abort_flag);
    return __all_sync(0xffffffffu, ok);
}

// kCausal: general form -- the visible band may be bounded (causal mask, sliding window) and the
// sequence lengths need not be multiples of 128; tiles that need it are masked in registers and the
// query tiles of a key tile are walked in ascending order from the first one that sees it.
// false = full attention over whole tiles only: no masking code at all, query sweep rotated per CTA
// (measured: carrying the unused masking code costs the D=64 full-attention kernel 6 %).
// T: storage type of Q/K/V/dO (__half or __nv_bfloat16).  TOut: type of the dK
// and dV outputs (T for the fused path, float for the split path).  kWithDq:
// false turns the kernel into the four-GEMM dK/dV half of the split path.
// kSoftcap: softcapped scores (general form only).  dS then carries the slope 1 - tanh^2 of the cap,
// which the second softmax phase recovers from P itself (t = (log2 P - (log2 r - m)) / softcap_post)
// instead of keeping it in registers between the phases.
template <typename T, int D, bool kCausal, bool kWithDq, typename TOut, bool kSoftcap = false>
__global__ void __launch_bounds__(512, 1)
fused_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                 const __grid_constant__ CUtensorMap tm_dqacc, const __grid_constant__ CUtensorMap tm_dk,
                 const __grid_constant__ CUtensorMap tm_dv, const __grid_constant__ FusedArgs a) {
    using C = FusedCfg<D>;
    constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = ptx::smem_u32(smem);
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int wg = warp >> 2;
    auto bar = [&](int i) -> uint32_t { return sbase + C::kOffBar + 8 * i; };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + C::kOffBar + 8 * kNumBars);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    if (threadIdx.x == 0) {
        TRACE(0, 0);
        TRACE_GT(0, 1);
    }
    // ---- which tile is ours ------------------------------------------------
    const int n_tiles = tiles_of(a.band.seqlen_k);      // key tiles (of the longest sequence)
    const int bh_count = a.batch * a.heads_kv;
    const bool split = a.chunk_steps > 0;
    const int group = a.heads_q / a.heads_kv;
    int kt, bhi, t_begin_split = 0, slab = 0;
    if (!split) {
        // groups of head_group heads; inside a group tile slot major, head minor (see cta_order.h)
        const int per_group = n_tiles * a.head_group;
        const int hg = int(blockIdx.x) / per_group;
        const int rem = int(blockIdx.x) - hg * per_group;
        const int heads_here = min(a.head_group, bh_count - hg * a.head_group);
        const int tile_slot = rem / heads_here;
        bhi = hg * a.head_group + (rem - tile_slot * heads_here);
        kt = remap_k_tile(tile_slot, n_tiles, a.order_mode, a.order_width);
    } else {
        const uint32_t entry = a.cta_table[blockIdx.x];
        kt = int(entry & 0xffu);
        t_begin_split = int((entry >> 8) & 0xffu) * a.chunk_steps;
        slab = int(entry >> 16);
        bhi = slab / a.chunks_per_head;
    }
    const int b = bhi / a.heads_kv;
    const int kvh = bhi % a.heads_kv;
    // Packed sequences: this batch entry's own lengths and first rows; tensors are addressed as one
    // batch of `total` rows, so rows past the end of a sequence belong to its neighbour (or read as
    // zero past the end of the tensor) and are masked like any ragged tile end.
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
    const int slot_k = band.seqlen_k;  // rows of dK / dV this batch entry owns
    if (a.seqused_q != nullptr || a.seqused_k != nullptr) {
        if (a.seqused_q != nullptr) band.seqlen_q = max(0, min(band.seqlen_q, a.seqused_q[b]));
        if (a.seqused_k != nullptr) band.seqlen_k = max(0, min(band.seqlen_k, a.seqused_k[b]));
        band.off = band.seqlen_k - band.seqlen_q;
    }
    const int n_q_tiles = tiles_of(band.seqlen_q);
    const bool tile_exists = kt * C::kTile < band.seqlen_k;  // false only with packed sequences
    const int q_begin = first_q_tile(kt, band);
    const int steps_per_head = tile_exists ? q_tiles_of_k_tile(kt, band) : 0;
    // this CTA's share of the tile's steps (all of them unless the tile is split)
    const int total_steps = group * steps_per_head;
    const int t_begin = t_begin_split;
    const int t_end = split ? min(total_steps, t_begin + a.chunk_steps) : total_steps;
    const int n_steps = t_end - t_begin;
    // "misaligned" also covers a CTA without work: every role is skipped, set-up and teardown still run
    const bool misaligned = (sbase & 1023u) != 0 || n_steps == 0;
    // an unsplit key tile that no query sees (possible with a left-bounded window) still owes zeros
    // to dK / dV
    const bool owes_zeros = !split && n_steps == 0 && (sbase & 1023u) == 0;

    if (threadIdx.x == 0) {
        TRACE(0, 4);
        if ((sbase & 1023u) != 0) atomicCAS(&g_device_error, kDevOk, kDevSmemMisaligned);
        ptx::mbar_init(bar(kKvFull), 1);
        for (int s = 0; s < 2; ++s) {
            ptx::mbar_init(bar(kQFull + s), 1);
            ptx::mbar_init(bar(kQEmpty + s), 1);
            ptx::mbar_init(bar(kDoFull + s), 1);
            ptx::mbar_init(bar(kDoEmpty + s), 1);
        }
        for (int s = 0; s < 2; ++s) ptx::mbar_init(bar(kStatsFull + s), 128);  // (unused with three buffers)
        ptx::mbar_init(bar(kSFull), 1);
        ptx::mbar_init(bar(kDpFull), 1);
        ptx::mbar_init(bar(kPReady), 256);
        ptx::mbar_init(bar(kDsReady), 256);
        ptx::mbar_init(bar(kDqFull), 1);
        ptx::mbar_init(bar(kDqEmpty), 128);
        ptx::mbar_init(bar(kDkvFull), 1);
        *abort_flag = 0;
        ptx::fence_mbar_init();
        TRACE(0, 2);
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), C::kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    // The kernel behind this one (dQ convert) may begin to launch; it waits for our completion itself.
    ptx::launch_dependents();

    // Query tiles are visited in ascending order starting at the diagonal (causal) or at a
    // per-CTA rotation (non-causal), so that CTAs of one head that run together add into
    // different dQ tiles at any moment.
    const int rotation = (kCausal || n_q_tiles == 0) ? 0 : kt % n_q_tiles;
    auto step_coords = [&](int t_local, int& hq, int& qt) {
        const int t = t_begin + t_local;
        const int g = t / steps_per_head;
        hq = kvh * group + g;
        const int r = t - g * steps_per_head;
        if (kCausal) {
            qt = q_begin + r;
        } else {
            qt = r + rotation;
            if (qt >= n_q_tiles) qt -= n_q_tiles;
        }
    };

    if (wg == 0) {
        ptx::setmaxnreg_dec<C::kRegsControl>();
        if (!misaligned && warp == 0) {
            // =================================================== TMA producer
            if (lane == 0) {
                ptx::prefetch_tensormap(&tm_q);
                ptx::prefetch_tensormap(&tm_k);
                ptx::prefetch_tensormap(&tm_v);
                ptx::prefetch_tensormap(&tm_do);
                // tensor maps are [batch][head][row][D]; rows past the end of a sequence read as zero
                ptx::mbar_arrive_expect_tx(bar(kKvFull), 2 * C::kOperandBytes);
#pragma unroll
                for (int bx = 0; bx < C::kBoxes; ++bx) {
                    ptx::tma_load_4d(sbase + C::kOffK + bx * C::kBoxBytes, &tm_k, bar(kKvFull), bx * 64,
                                     k_base + kt * C::kTile, kvh, b_coord);
                    ptx::tma_load_4d(sbase + C::kOffV + bx * C::kBoxBytes, &tm_v, bar(kKvFull), bx * 64,
                                     k_base + kt * C::kTile, kvh, b_coord);
                }
                TRACE(0, 3);
#pragma unroll 1
                for (int t = 0; t < n_steps; ++t) {
                    int hq, qt;
                    step_coords(t, hq, qt);
                    const int q_row = q_base + qt * C::kTile;
                    const int s = t % C::kQStages;
                    if (!bounded_wait<true>(bar(kQEmpty + s), ((t / C::kQStages) & 1) ^ 1, abort_flag)) break;
                    ptx::mbar_arrive_expect_tx(bar(kQFull + s), C::kOperandBytes);
#pragma unroll
                    for (int bx = 0; bx < C::kBoxes; ++bx) {
                        ptx::tma_load_4d(sbase + C::kOffQ + s * C::kOperandBytes + bx * C::kBoxBytes, &tm_q,
                                         bar(kQFull + s), bx * 64, q_row, hq, b_coord);
                    }
                    const int sd = t % C::kDoStages;
                    if (!bounded_wait<true>(bar(kDoEmpty + sd), ((t / C::kDoStages) & 1) ^ 1, abort_flag)) break;
                    ptx::mbar_arrive_expect_tx(bar(kDoFull + sd), C::kOperandBytes);
#pragma unroll
                    for (int bx = 0; bx < C::kBoxes; ++bx) {
                        ptx::tma_load_4d(sbase + C::kOffDO + sd * C::kOperandBytes + bx * C::kBoxBytes, &tm_do,
                                         bar(kDoFull + sd), bx * 64, q_row, hq, b_coord);
                    }
                }
            }
        } else if (!misaligned && warp == 1) {
            // ===================================================== MMA issuer
            // The whole warp runs this role converged; MMAs and commits elect their lane inside the asm.
            {
                TRACE(1, 0);
                constexpr uint32_t kIdSdP = ptx::instr_desc_f16(kBf16, 128, 128, false, false);
                constexpr uint32_t kIdDkv = ptx::instr_desc_f16(kBf16, 128, D, false, true);
                constexpr uint32_t kIdDq = ptx::instr_desc_f16(kBf16, 128, D, true, true);
                // Descriptor low words (address >> 4 | LBO) of every operand tile; a K step advances them
                // by a compile-time constant: K-major +2 per 16 elements inside a box and +box/16 per box,
                // MN-major +128 per 16 rows.  One constant high word serves every descriptor.
                constexpr uint32_t kHi = ptx::kDescHiSw128;
                constexpr uint32_t kBoxStep = C::kBoxBytes >> 4;
                auto k_step = [](int kk) -> uint32_t { return uint32_t(kk >> 2) * kBoxStep + uint32_t(kk & 3) * 2u; };
                auto mn_step = [](int kk) -> uint32_t { return uint32_t(kk) * 128u; };
                const uint32_t loK_k = ptx::desc_lo_k_major(sbase + C::kOffK);
                const uint32_t loV_k = ptx::desc_lo_k_major(sbase + C::kOffV);
                const uint32_t loDS_k = ptx::desc_lo_k_major(sbase + C::kOffDS);
                const uint32_t loK_mn = ptx::desc_lo_mn_major(sbase + C::kOffK, C::kBoxBytes);
                const uint32_t loDS_mn = ptx::desc_lo_mn_major(sbase + C::kOffDS, C::kBoxBytes);
                auto sQ = [&](int t) { return sbase + C::kOffQ + (t % C::kQStages) * C::kOperandBytes; };
                auto sDO = [&](int t) { return sbase + C::kOffDO + (t % C::kDoStages) * C::kOperandBytes; };
                auto issue_s = [&](int t) {
                    const uint32_t loQ = ptx::desc_lo_k_major(sQ(t));
                    ptx::mma_ss_lean<false>(tmem + C::kColS, loK_k, loQ, kHi, kIdSdP);
#pragma unroll
                    for (int kk = 1; kk < D / 16; ++kk)
                        ptx::mma_ss_lean<true>(tmem + C::kColS, loK_k + k_step(kk), loQ + k_step(kk), kHi, kIdSdP);
                    ptx::tc_commit_elect(bar(kSFull));
                };
                auto issue_dp = [&](int t) {
                    const uint32_t loDO = ptx::desc_lo_k_major(sDO(t));
                    ptx::mma_ss_lean<false>(tmem + C::kColDP, loV_k, loDO, kHi, kIdSdP);
#pragma unroll
                    for (int kk = 1; kk < D / 16; ++kk)
                        ptx::mma_ss_lean<true>(tmem + C::kColDP, loV_k + k_step(kk), loDO + k_step(kk), kHi, kIdSdP);
                    ptx::tc_commit_elect(bar(kDpFull));
                };
                bool ok = warp_wait<false>(bar(kKvFull), 0, abort_flag) &&
                          warp_wait<false>(bar(kQFull + 0), 0, abort_flag);
                TRACE(1, 1);
                if (ok) {
                    ptx::tc_fence_after();
                    issue_s(0);
                    TRACE(1, 2);
                    ok = warp_wait<false>(bar(kDoFull + 0), 0, abort_flag);
                }
                if (ok) {
                    ptx::tc_fence_after();
                    issue_dp(0);
                    TRACE(1, 4);
                }
#pragma unroll 1
                for (int t = 0; ok && t < n_steps; ++t) {
                    const bool more = t + 1 < n_steps;
                    // dV += P^T dO.  P^T of queries 0-63 sits on columns [0,32) of the S
                    // region, of queries 64-127 on columns [64,96).
                    if (!(ok = warp_wait<false>(bar(kPReady), t & 1, abort_flag))) break;
                    if (t < 6) TRACE(1, 8 + 8 * t + 0);
                    ptx::tc_fence_after();
                    {
                        const uint32_t loDO = ptx::desc_lo_mn_major(sDO(t), C::kBoxBytes);
                        ptx::mma_ts_lean_rt(tmem + C::kColDV, tmem + C::kColS, loDO, kHi, kIdDkv, t > 0 ? 1u : 0u);
#pragma unroll
                        for (int kk = 1; kk < 8; ++kk)
                            ptx::mma_ts_lean<true>(tmem + C::kColDV, tmem + C::kColS + (kk >> 2) * 64 + (kk & 3) * 8,
                                                   loDO + mn_step(kk), kHi, kIdDkv);
                    }
                    ptx::tc_commit_elect(bar(kDoEmpty + t % C::kDoStages));
                    if (t < 6) TRACE(1, 8 + 8 * t + 1);
                    // S(t+1) may overwrite S/P(t): MMAs execute in issue order.
                    if (more) {
                        if (!(ok = warp_wait<false>(bar(kQFull + (t + 1) % C::kQStages),
                                                ((t + 1) / C::kQStages) & 1, abort_flag))) break;
                        ptx::tc_fence_after();
                        issue_s(t + 1);
                    }
                    if (t < 6) TRACE(1, 8 + 8 * t + 2);
                    // dK += dS^T Q
                    if (!(ok = warp_wait<false>(bar(kDsReady), t & 1, abort_flag))) break;
                    if (t < 6) TRACE(1, 8 + 8 * t + 3);
                    ptx::tc_fence_after();
                    {
                        const uint32_t loQ = ptx::desc_lo_mn_major(sQ(t), C::kBoxBytes);
                        ptx::mma_ss_lean_rt(tmem + C::kColDK, loDS_k, loQ, kHi, kIdDkv, t > 0 ? 1u : 0u);
#pragma unroll
                        for (int kk = 1; kk < 8; ++kk)
                            ptx::mma_ss_lean<true>(tmem + C::kColDK, loDS_k + k_step(kk), loQ + mn_step(kk), kHi, kIdDkv);
                    }
                    ptx::tc_commit_elect(bar(kQEmpty + t % C::kQStages));
                    if (kWithDq) {
                        if (D == 64) {  // own dQ region: wait for the drain of step t-1
                            if (!(ok = warp_wait<false>(bar(kDqEmpty), (t & 1) ^ 1, abort_flag))) break;
                            ptx::tc_fence_after();
                        }
                        // dQ = dS K  (overwrites dP(t) when D = 128: dP(t) was consumed before kDsReady)
                        ptx::mma_ss_lean<false>(tmem + C::kColDQ, loDS_mn, loK_mn, kHi, kIdDq);
#pragma unroll
                        for (int kk = 1; kk < 8; ++kk)
                            ptx::mma_ss_lean<true>(tmem + C::kColDQ, loDS_mn + mn_step(kk), loK_mn + mn_step(kk), kHi, kIdDq);
                        ptx::tc_commit_elect(bar(kDqFull));
                    }
                    if (t < 6) TRACE(1, 8 + 8 * t + 4);
                    if (more) {
                        if (!(ok = warp_wait<false>(bar(kDoFull + (t + 1) % C::kDoStages),
                                                ((t + 1) / C::kDoStages) & 1, abort_flag))) break;
                        if (t < 6) TRACE(1, 8 + 8 * t + 5);
                        if (kWithDq && D == 128) {  // dP(t+1) reuses the dQ(t) columns
                            if (!(ok = warp_wait<false>(bar(kDqEmpty), t & 1, abort_flag))) break;
                        }
                        if (t < 6) TRACE(1, 8 + 8 * t + 6);
                        ptx::tc_fence_after();
                        issue_dp(t + 1);
                        if (t < 6) TRACE(1, 8 + 8 * t + 7);
                    }
                }
                if (ok) ptx::tc_commit_elect(bar(kDkvFull));
                TRACE(1, 62);
            }
        }
    } else if (wg == 1 || wg == 2) {
        // ============================================ softmax / dS warpgroups
        if (C::kRegsCompute < 128) ptx::setmaxnreg_dec<C::kRegsCompute>();
        else ptx::setmaxnreg_inc<C::kRegsCompute>();
        if (!misaligned) {
            const int half = wg - 1;          // which 64 queries of the tile
            const int j = threadIdx.x & 127;  // key row inside the tile == TMEM lane
            const uint32_t tl = tmem + (uint32_t((warp & 3) * 32) << 16);
            const uint32_t s_cols = tl + C::kColS + half * 64;
            const uint32_t dp_cols = tl + C::kColDP + half * 64;
            float* stats = reinterpret_cast<float*>(smem + C::kOffStats);
            uint32_t ppk[32];
            const float* side_base = a.sidecar;
            float s0 = 0.f, s1 = 0.f, s2 = 0.f;
            bool s_valid = false;
            // Statistics of query row qi of head hq, fetched one step ahead.  The loaded values are
            // not touched here (their first use, one step later, is what waits for the loads); rows
            // past the end of the sequence read row 0 instead and are replaced at that first use.
            auto load_stats = [&](int hq, int qt) {
                const int qi = qt * C::kTile + j;
                s_valid = qi < band.seqlen_q;
                const int64_t row = int64_t(b_coord * a.heads_q + hq) * a.sidecar_rows + q_base + (s_valid ? qi : 0);
                s0 = side_base[row * 3 + 0];
                s1 = side_base[row * 3 + 1];
                s2 = side_base[row * 3 + 2];
            };
            // the sidecar comes from the delta kernel, which may still be running (programmatic launch);
            // Q, K, V, dO are inputs of the call, so the TMA and MMA warps did not have to wait
            ptx::grid_dependency_wait();
            constexpr int kNB = C::kStatsBufs;
            constexpr bool kStatsAhead = kNB == 3;
            // row statistics of query row j of a tile, for both warpgroups:
            // P = exp2(x - m) * r = exp2(x + (log2 r - m)); a row past the end of the sequence
            // gets -inf, which makes its P (and with it dS) exactly zero
            auto publish_stats = [&](int buf) {
                stats[buf * 128 + j] = (!kCausal || s_valid) ? __log2f(s1) - s0 : -INFINITY;
                stats[kNB * 128 + buf * 128 + j] = (!kCausal || s_valid) ? s2 : 0.f;
                if (!kStatsAhead) ptx::mbar_arrive(bar(kStatsFull + buf));
            };
            if (half == 0) {
                int hq, qt;
                step_coords(0, hq, qt);
                load_stats(hq, qt);
                if (kStatsAhead) {
                    publish_stats(0);
                    if (n_steps > 1) {
                        step_coords(1, hq, qt);
                        load_stats(hq, qt);
                    }
                }
            }
            // (step 0's statistics are the exception: one meeting of the two warpgroups)
            if (kStatsAhead) asm volatile("bar.sync 1, 256;" ::: "memory");
            bool ok = true;
#pragma unroll 1
            for (int t = 0; t < n_steps; ++t) {
                if (warp == 4 && t == 3) TRACE(2, 0);
                int hq, qt;
                step_coords(t, hq, qt);
                if (warp == 4 && t == 3) TRACE(2, 1);
                const int buf = t % kNB;
                const float* negp = stats + buf * 128 + half * 64;
                const float* delp = stats + kNB * 128 + buf * 128 + half * 64;
                if (half == 0) {
                    if (kStatsAhead) {
                        // the registers hold step t+1: publish it now (its buffer was last read in step
                        // t-2, which every warp has left: this warpgroup could not have written dS(t-1)
                        // before dS(t-2) of both was consumed), then fetch step t+2
                        if (t + 1 < n_steps) publish_stats((t + 1) % kNB);
                        if (warp == 4 && t == 3) TRACE(2, 2);
                    } else {
                        publish_stats(buf);
                        if (warp == 4 && t == 3) TRACE(2, 2);
                        if (t + 1 < n_steps) {
                            int hq1, qt1;
                            step_coords(t + 1, hq1, qt1);
                            load_stats(hq1, qt1);
                        }
                    }
                }
                if (warp == 4 && t == 3) TRACE(2, 3);
                // Published one step ahead, the statistics of step t need no barrier of their own: their
                // writers arrived at "P ready" of step t-1 after writing them, S(t) was issued after that
                // barrier completed, and every reader waits for S(t) below.
                if (!kStatsAhead) {
                    if (!(ok = warp_wait(bar(kStatsFull + buf), (t / kNB) & 1, abort_flag))) break;
                }
                if (warp == 4 && t < 7) TRACE(2, 4 + 8 * t + 0);
                if (!(ok = warp_wait(bar(kSFull), t & 1, abort_flag))) break;
                if (warp == 4 && t < 7) TRACE(2, 4 + 8 * t + 1);
                ptx::tc_fence_after();
                // A tile that crosses an edge of the band or holds keys past the end of the sequence is
                // masked: element (key j, query i) survives iff mask_from <= i <= mask_to.
                const bool diagonal = kCausal && tile_needs_mask(kt, qt, band);
                int mask_from = 0, mask_to = 0;  // set only on masked tiles
                // ---- P^T = exp2(S^T * scale_log2 + neg_i), masked as above.
                // (two copies of the chunk code, so that unmasked tiles carry no per-element test)
                // score in log2 units, relative to the row's reference: s * scale*log2e + (log2 r - m), or the
                // capped score + (log2 r - m)
                auto log2_score = [&](uint32_t raw, float neg) {
                    return kSoftcap ? fmaf(a.softcap_post, ptx::tanh_approx(__uint_as_float(raw) * a.softcap_pre), neg)
                                    : fmaf(__uint_as_float(raw), a.scale_log2, neg);
                };
                auto softmax_chunk = [&](int c, const uint32_t* r, auto masked_tag) {
                    constexpr bool kMasked = decltype(masked_tag)::value;
#pragma unroll
                    for (int e = 0; e < 32; e += 4) {
                        const float4 n4 = *reinterpret_cast<const float4*>(negp + c * 32 + e);
                        float p0 = ptx::ex2_approx(log2_score(r[e + 0], n4.x));
                        float p1 = ptx::ex2_approx(log2_score(r[e + 1], n4.y));
                        float p2 = ptx::ex2_approx(log2_score(r[e + 2], n4.z));
                        float p3 = ptx::ex2_approx(log2_score(r[e + 3], n4.w));
                        if (kMasked) {
                            const int i = half * 64 + c * 32 + e;
                            p0 = (i + 0 >= mask_from && i + 0 <= mask_to) ? p0 : 0.0f;
                            p1 = (i + 1 >= mask_from && i + 1 <= mask_to) ? p1 : 0.0f;
                            p2 = (i + 2 >= mask_from && i + 2 <= mask_to) ? p2 : 0.0f;
                            p3 = (i + 3 >= mask_from && i + 3 <= mask_to) ? p3 : 0.0f;
                        }
                        ppk[c * 16 + e / 2 + 0] = ptx::Pack2<T>::pack(p0, p1);
                        ppk[c * 16 + e / 2 + 1] = ptx::Pack2<T>::pack(p2, p3);
                    }
                    // P chunk c -> columns [16c, 16c+16) of this half's S columns (already read)
                    ptx::tmem_st16(s_cols + c * 16, &ppk[c * 16]);
                };
                if (diagonal) {
                    query_range_of_key(kt * C::kTile + j, qt * C::kTile, band, &mask_from, &mask_to);
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        uint32_t r[32];
                        ptx::tmem_ld32(s_cols + c * 32, r);
                        ptx::tmem_ld_wait();
                        softmax_chunk(c, r, std::true_type{});
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        uint32_t r[32];
                        ptx::tmem_ld32(s_cols + c * 32, r);
                        ptx::tmem_ld_wait();
                        softmax_chunk(c, r, std::false_type{});
                    }
                }
                if (warp == 4 && t < 7) TRACE(2, 4 + 8 * t + 2);
                ptx::tmem_st_wait();
                ptx::tc_fence_before();
                ptx::mbar_arrive(bar(kPReady));
                if (kStatsAhead && half == 0 && t + 2 < n_steps) {
                    // (requested here, where the warp is about to wait for dP anyway)
                    int hq2, qt2;
                    step_coords(t + 2, hq2, qt2);
                    load_stats(hq2, qt2);
                }
                if (warp == 4 && t < 7) TRACE(2, 4 + 8 * t + 3);
                // ---- dS^T = P^T * (dP^T - delta_i), stored [key][query] in the 128-byte swizzle
                if (!(ok = warp_wait(bar(kDpFull), t & 1, abort_flag))) break;
                if (warp == 4 && t < 7) TRACE(2, 4 + 8 * t + 4);
                // (the dS buffer is free: dP(t) was issued behind dK(t-1), dQ(t-1), the readers of dS(t-1),
                // and the barrier just passed completes only when every MMA issued before it has)
                if (warp == 4 && t < 7) TRACE(2, 4 + 8 * t + 5);
                ptx::tc_fence_after();
                const uint32_t ds_row = sbase + C::kOffDS + half * C::kBoxBytes + j * 128;
                const float inv_post = kSoftcap ? 1.0f / a.softcap_post : 0.0f;
                auto ds_chunk = [&](int c, const uint32_t* r) {
#pragma unroll
                    for (int e = 0; e < 32; e += 8) {
                        const float4 d0 = *reinterpret_cast<const float4*>(delp + c * 32 + e);
                        const float4 d1 = *reinterpret_cast<const float4*>(delp + c * 32 + e + 4);
                        const float2 pa = ptx::Pack2<T>::unpack(ppk[c * 16 + e / 2 + 0]);
                        const float2 pb = ptx::Pack2<T>::unpack(ppk[c * 16 + e / 2 + 1]);
                        const float2 pc = ptx::Pack2<T>::unpack(ppk[c * 16 + e / 2 + 2]);
                        const float2 pd = ptx::Pack2<T>::unpack(ppk[c * 16 + e / 2 + 3]);
                        uint4 o;
                        if (kSoftcap) {
                            // dS = P (dP - delta) (1 - t^2), t recovered from P and the row's reference
                            const float4 n0 = *reinterpret_cast<const float4*>(negp + c * 32 + e);
                            const float4 n1 = *reinterpret_cast<const float4*>(negp + c * 32 + e + 4);
                            auto capped = [&](float p, uint32_t dp, float del, float neg) {
                                const float t = (__log2f(p) - neg) * inv_post;
                                const float slope = fmaxf(1.0f - t * t, 0.0f);
                                return p > 0.0f ? p * (__uint_as_float(dp) - del) * slope : 0.0f;
                            };
                            o.x = ptx::Pack2<T>::pack(capped(pa.x, r[e + 0], d0.x, n0.x), capped(pa.y, r[e + 1], d0.y, n0.y));
                            o.y = ptx::Pack2<T>::pack(capped(pb.x, r[e + 2], d0.z, n0.z), capped(pb.y, r[e + 3], d0.w, n0.w));
                            o.z = ptx::Pack2<T>::pack(capped(pc.x, r[e + 4], d1.x, n1.x), capped(pc.y, r[e + 5], d1.y, n1.y));
                            o.w = ptx::Pack2<T>::pack(capped(pd.x, r[e + 6], d1.z, n1.z), capped(pd.y, r[e + 7], d1.w, n1.w));
                        } else {
                        o.x = ptx::Pack2<T>::pack(pa.x * (__uint_as_float(r[e + 0]) - d0.x),
                                                  pa.y * (__uint_as_float(r[e + 1]) - d0.y));
                        o.y = ptx::Pack2<T>::pack(pb.x * (__uint_as_float(r[e + 2]) - d0.z),
                                                  pb.y * (__uint_as_float(r[e + 3]) - d0.w));
                        o.z = ptx::Pack2<T>::pack(pc.x * (__uint_as_float(r[e + 4]) - d1.x),
                                                  pc.y * (__uint_as_float(r[e + 5]) - d1.y));
                        o.w = ptx::Pack2<T>::pack(pd.x * (__uint_as_float(r[e + 6]) - d1.z),
                                                  pd.y * (__uint_as_float(r[e + 7]) - d1.w));
                        }
                        const int chunk = c * 4 + e / 8;  // 16-byte chunk inside this half's box
                        const uint32_t addr = ds_row + ((chunk ^ (j & 7)) << 4);
                        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(o.x),
                                     "r"(o.y), "r"(o.z), "r"(o.w) : "memory");
                    }
                };
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t r[32];
                    ptx::tmem_ld32(dp_cols + c * 32, r);
                    ptx::tmem_ld_wait();
                    ds_chunk(c, r);
                }
                if (warp == 4 && t < 7) TRACE(2, 4 + 8 * t + 6);
                ptx::fence_proxy_async_smem();
                ptx::tc_fence_before();
                ptx::mbar_arrive(bar(kDsReady));
                if (warp == 4 && t < 7) TRACE(2, 4 + 8 * t + 7);
            }
            // ---- epilogue: the first warpgroup writes dK (scaled), the second dV
            if (ok) ok = warp_wait(bar(kDkvFull), 0, abort_flag);
            if (warp == 4) TRACE(2, 60);
            if (ok) {
                // Every MMA has completed, so the Q / dO / dS^T buffers are dead.  Each warp stages its
                // 32 key rows there in the layout of a swizzled TMA box and one lane stores them with
                // the copy engine: whole 128-byte lines, rows past the end of the tensor clipped by the
                // hardware.  (A thread storing its own row straight from registers writes 16 bytes per
                // line and instruction: measured 6 us per CTA instead of under 1.)
                ptx::tc_fence_after();
                const float mul = half == 0 ? a.scale : 1.0f;
                const uint32_t col0 = tl + (half == 0 ? C::kColDK : C::kColDV);
                const int w4 = warp & 3;  // which 32 rows of the tile
                // packed sequences: the rows behind this sequence's end belong to its neighbour, which the
                // copy engine cannot know; fp32 outputs of the split path: plain rows.  Both keep per-thread stores.
                const bool staged = split || (sizeof(TOut) == 2 && a.cu_seqlens_q == nullptr);
                if (staged && split && !kBf16) {
                    // fp16 inputs: the partial sums go to this CTA's slabs (slab 2x: dK, 2x+1: dV) as fp16,
                    // boxes of [32 rows][64 x 16 bit].  (fp16 keeps 11 significant bits, three more than a
                    // bf16 result would; the bytes written, not the arithmetic, bound this epilogue.)
                    const uint32_t scratch = sbase + C::kOffQ + (half * 4 + w4) * (C::kBoxes * C::kStageBoxBytes);
#pragma unroll
                    for (int c = 0; c < D / 32; ++c) {
                        uint32_t r[32];
                        ptx::tmem_ld32(col0 + c * 32, r);
                        ptx::tmem_ld_wait();
                        const uint32_t row_addr = scratch + (c >> 1) * C::kStageBoxBytes + lane * 128;
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const uint32_t o0 = ptx::Pack2<__half>::pack(__uint_as_float(r[8 * e + 0]) * mul, __uint_as_float(r[8 * e + 1]) * mul);
                            const uint32_t o1 = ptx::Pack2<__half>::pack(__uint_as_float(r[8 * e + 2]) * mul, __uint_as_float(r[8 * e + 3]) * mul);
                            const uint32_t o2 = ptx::Pack2<__half>::pack(__uint_as_float(r[8 * e + 4]) * mul, __uint_as_float(r[8 * e + 5]) * mul);
                            const uint32_t o3 = ptx::Pack2<__half>::pack(__uint_as_float(r[8 * e + 6]) * mul, __uint_as_float(r[8 * e + 7]) * mul);
                            const int chunk = (c & 1) * 4 + e;
                            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};"
                                         ::"r"(row_addr + ((chunk ^ (lane & 7)) << 4)), "r"(o0), "r"(o1), "r"(o2), "r"(o3)
                                         : "memory");
                        }
                    }
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
#pragma unroll
                        for (int bx = 0; bx < C::kBoxes; ++bx)
                            ptx::tma_store_4d(&tm_dk, scratch + bx * C::kStageBoxBytes, bx * 64, w4 * 32, slab * 2 + half, 0);
                        ptx::bulk_commit_group();
                        ptx::bulk_wait_group_read<0>();
                    }
                } else if (staged && split) {
                    // bf16 inputs: fp32 partial sums -> this CTA's slabs, boxes of [32 rows][32 fp32]
                    constexpr int kBoxesPerWarp = D / 32;
                    const uint32_t scratch = sbase + C::kOffQ + (half * 4 + w4) * (kBoxesPerWarp * C::kStageBoxBytes);
#pragma unroll
                    for (int c = 0; c < kBoxesPerWarp; ++c) {
                        uint32_t r[32];
                        ptx::tmem_ld32(col0 + c * 32, r);
                        ptx::tmem_ld_wait();
                        const uint32_t row_addr = scratch + c * C::kStageBoxBytes + lane * 128;
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};"
                                         ::"r"(row_addr + ((e ^ (lane & 7)) << 4)),
                                           "f"(__uint_as_float(r[4 * e]) * mul), "f"(__uint_as_float(r[4 * e + 1]) * mul),
                                           "f"(__uint_as_float(r[4 * e + 2]) * mul), "f"(__uint_as_float(r[4 * e + 3]) * mul)
                                         : "memory");
                        }
                    }
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
#pragma unroll
                        for (int c = 0; c < kBoxesPerWarp; ++c)
                            ptx::tma_store_3d(&tm_dk, scratch + c * C::kStageBoxBytes, c * 32, w4 * 32,
                                              slab * 2 + half);
                        ptx::bulk_commit_group();
                        ptx::bulk_wait_group_read<0>();
                    }
                } else if (staged) {
                    // 16-bit outputs -> dk / dv through their tensor maps, boxes of [32 rows][64 x 16 bit]
                    const uint32_t scratch = sbase + C::kOffQ + (half * 4 + w4) * (C::kBoxes * C::kStageBoxBytes);
#pragma unroll
                    for (int c = 0; c < D / 32; ++c) {
                        uint32_t r[32];
                        ptx::tmem_ld32(col0 + c * 32, r);
                        ptx::tmem_ld_wait();
                        // 32 columns = 64 bytes = chunks 4*(c&1) .. 4*(c&1)+3 of this row of box c/2
                        const uint32_t row_addr = scratch + (c >> 1) * C::kStageBoxBytes + lane * 128;
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const uint32_t o0 = ptx::Pack2<T>::pack(__uint_as_float(r[8 * e + 0]) * mul, __uint_as_float(r[8 * e + 1]) * mul);
                            const uint32_t o1 = ptx::Pack2<T>::pack(__uint_as_float(r[8 * e + 2]) * mul, __uint_as_float(r[8 * e + 3]) * mul);
                            const uint32_t o2 = ptx::Pack2<T>::pack(__uint_as_float(r[8 * e + 4]) * mul, __uint_as_float(r[8 * e + 5]) * mul);
                            const uint32_t o3 = ptx::Pack2<T>::pack(__uint_as_float(r[8 * e + 6]) * mul, __uint_as_float(r[8 * e + 7]) * mul);
                            const int chunk = (c & 1) * 4 + e;
                            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};"
                                         ::"r"(row_addr + ((chunk ^ (lane & 7)) << 4)), "r"(o0), "r"(o1), "r"(o2), "r"(o3)
                                         : "memory");
                        }
                    }
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        const void* map = half == 0 ? static_cast<const void*>(&tm_dk) : static_cast<const void*>(&tm_dv);
#pragma unroll
                        for (int bx = 0; bx < C::kBoxes; ++bx)
                            ptx::tma_store_4d(map, scratch + bx * C::kStageBoxBytes, bx * 64,
                                              kt * C::kTile + w4 * 32, kvh, b);
                        ptx::bulk_commit_group();
                        ptx::bulk_wait_group_read<0>();
                    }
                } else {
                    // (tensor-memory loads are warp-wide: every lane runs them, only the stores of key rows
                    // past the end of the sequence are skipped)
                    // (rows between the used length and the end of the slot hold exact zeros)
                    const bool key_valid = kt * C::kTile + j < slot_k;
                    const int64_t off = b_coord * a.kv_strides.batch + kvh * a.kv_strides.head +
                                        int64_t(k_base + kt * C::kTile + j) * a.kv_strides.row;
                    TOut* dst = reinterpret_cast<TOut*>(half == 0 ? a.dk : a.dv) + off;
#pragma unroll
                    for (int c = 0; c < D / 32; ++c) {
                        uint32_t r[32];
                        ptx::tmem_ld32(col0 + c * 32, r);
                        ptx::tmem_ld_wait();
                        if (key_valid) {
                            if (sizeof(TOut) == 4) {
                                float4* d4 = reinterpret_cast<float4*>(dst + c * 32);
#pragma unroll
                                for (int e = 0; e < 8; ++e)
                                    d4[e] = make_float4(__uint_as_float(r[4 * e]) * mul, __uint_as_float(r[4 * e + 1]) * mul,
                                                        __uint_as_float(r[4 * e + 2]) * mul, __uint_as_float(r[4 * e + 3]) * mul);
                            } else {
                                uint4* d4 = reinterpret_cast<uint4*>(dst + c * 32);
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    uint4 o;
                                    o.x = ptx::Pack2<T>::pack(__uint_as_float(r[8 * e + 0]) * mul, __uint_as_float(r[8 * e + 1]) * mul);
                                    o.y = ptx::Pack2<T>::pack(__uint_as_float(r[8 * e + 2]) * mul, __uint_as_float(r[8 * e + 3]) * mul);
                                    o.z = ptx::Pack2<T>::pack(__uint_as_float(r[8 * e + 4]) * mul, __uint_as_float(r[8 * e + 5]) * mul);
                                    o.w = ptx::Pack2<T>::pack(__uint_as_float(r[8 * e + 6]) * mul, __uint_as_float(r[8 * e + 7]) * mul);
                                    d4[e] = o;
                                }
                            }
                        }
                        __syncwarp();  // reconverge before the next warp-wide load
                    }
                }
            }
            if (warp == 4) TRACE(2, 61);
        } else if (owes_zeros) {
            // nobody attends to these keys: the first warpgroup clears dK, the second dV
            const int j = threadIdx.x & 127;
            if (kt * C::kTile + j < slot_k) {
                const int64_t off = b_coord * a.kv_strides.batch + kvh * a.kv_strides.head +
                                    int64_t(k_base + kt * C::kTile + j) * a.kv_strides.row;
                uint4* d4 = reinterpret_cast<uint4*>(reinterpret_cast<TOut*>(wg == 1 ? a.dk : a.dv) + off);
#pragma unroll
                for (int e = 0; e < int(D * sizeof(TOut) / 16); ++e) d4[e] = make_uint4(0u, 0u, 0u, 0u);
            }
        }
    } else {
        // ==================================================== dQ drain warpgroup
        if (!kWithDq) {
            ptx::setmaxnreg_dec<C::kRegsControl>();
        } else {
            ptx::setmaxnreg_inc<C::kRegsDrain>();
            if (!misaligned) {
                const int qd = warp & 3;
                const uint32_t tl = tmem + (uint32_t(qd * 32) << 16);
                const uint32_t stage = sbase + C::kOffStage + qd * 2 * C::kStageBoxBytes;
                bool pending = false;
                // the accumulators are cleared by the delta kernel: do not add into them before it is done
                ptx::grid_dependency_wait();
#pragma unroll 1
                for (int t = 0; t < n_steps; ++t) {
                    int hq, qt;
                    step_coords(t, hq, qt);
                    const int q_row = qt * C::kTile + qd * 32;  // row inside the head
                    const int q_head = b_coord * a.heads_q + hq;
                    if (!warp_wait(bar(kDqFull), t & 1, abort_flag)) break;
                    if (warp == 12 && t < 12) TRACE(3, 4 + 4 * t + 0);
                    ptx::tc_fence_after();
                    // pull the whole dQ tile row into registers and hand the columns back at once
                    uint32_t r[D / 32][32];
#pragma unroll
                    for (int c = 0; c < D / 32; ++c) ptx::tmem_ld32(tl + C::kColDQ + c * 32, r[c]);
                    ptx::tmem_ld_wait();
                    ptx::tc_fence_before();
                    ptx::mbar_arrive(bar(kDqEmpty));
                    if (warp == 12 && t < 12) TRACE(3, 4 + 4 * t + 1);
#pragma unroll
                    for (int hf = 0; hf < D / 64; ++hf) {
                        if (pending) {
                            if (lane == 0) ptx::bulk_wait_group_read<0>();
                            __syncwarp();
                        }
#pragma unroll
                        for (int bx = 0; bx < 2; ++bx) {
                            const uint32_t row_addr = stage + bx * C::kStageBoxBytes + lane * 128;
#pragma unroll
                            for (int c = 0; c < 8; ++c) {
                                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};"
                                             ::"r"(row_addr + ((c ^ (lane & 7)) << 4)), "r"(r[hf * 2 + bx][4 * c]),
                                               "r"(r[hf * 2 + bx][4 * c + 1]), "r"(r[hf * 2 + bx][4 * c + 2]),
                                               "r"(r[hf * 2 + bx][4 * c + 3])
                                             : "memory");
                            }
                        }
                        ptx::fence_proxy_async_smem();
                        __syncwarp();
                        // accumulator map: [batch*head][row][D]; rows past the sequence end are dropped
                        if (lane == 0 && q_row < band.seqlen_q) {
                            ptx::tma_reduce_add_3d(&tm_dqacc, stage, hf * 64, q_base + q_row, q_head);
                            ptx::tma_reduce_add_3d(&tm_dqacc, stage + C::kStageBoxBytes, hf * 64 + 32, q_base + q_row, q_head);
                            ptx::bulk_commit_group();
                        }
                        pending = true;
                    }
                    if (warp == 12 && t < 12) TRACE(3, 4 + 4 * t + 2);
                }
                if (lane == 0) ptx::bulk_wait_group<0>();
                if (warp == 12) TRACE(3, 59);
            }
        }
    }

    // ---- teardown: everybody meets, then the allocating warp frees TMEM
    if (threadIdx.x == 0) ptx::grid_dependency_wait();
    __syncwarp();
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem, C::kTmemCols);
    }
    if (threadIdx.x == 0) {
        TRACE(0, 63);
        TRACE_GT(0, 62);
    }
}

}  // namespace fa3b200
