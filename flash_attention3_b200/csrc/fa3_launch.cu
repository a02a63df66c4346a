// Launch layer of the C ABI: tensor-map construction, kernel dispatch over
// (dtype, head_dim, causal) and the stage chaining of shaobo_fa3_bwd_v2
// (role of reference src/shaobo_fa3_bwd_api.cpp:206-260 and
// src/fused_bwd_kernel.cpp:1673-1764).  No allocation happens here: every
// buffer, the workspace included, belongs to the caller.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <map>
#include <mutex>
#include <tuple>
#include <vector>

#include "cta_order.h"
#include "fa3_host.h"
#include "fused_bwd_kernel.cuh"
#include "dq_kernel.cuh"
#include "fwd_kernel.cuh"
#include "rowwise_kernels.cuh"
#include "shaobo_fa3_b200_ext.h"
#include "shaobo_fa3_components.h"

namespace fa3b200 {
namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) !=
                cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            p = nullptr;
        }
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// 16-bit [batch][head][row][D] tensor in either layout, addressed with coordinates (column, row,
// head, batch); boxes of [128 rows][64 columns] with the 128-byte swizzle.  Rows past the end of a
// sequence are outside the tensor for the copy engine and read as zero.
bool make_map_16(CUtensorMap* map, CUtensorMapDataType type, const void* base, int batch, int heads,
                 int seqlen, int d, bool bshd, int box_rows = 128) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return false;
    const TensorStrides st = strides_of(bshd, heads, seqlen, d);
    const cuuint64_t dims[4] = {cuuint64_t(d), cuuint64_t(seqlen), cuuint64_t(heads), cuuint64_t(batch)};
    const cuuint64_t strides[3] = {cuuint64_t(st.row) * 2, cuuint64_t(st.head) * 2, cuuint64_t(st.batch) * 2};
    const cuuint32_t box[4] = {64, cuuint32_t(box_rows), 1, 1};
    const cuuint32_t elem_strides[4] = {1, 1, 1, 1};
    return fn(map, type, 4, const_cast<void*>(base), dims, strides, box, elem_strides,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// fp32 accumulator [batch*head][row][D] contiguous, coordinates (column, row, batch*head), boxes of
// [32 rows][32 columns] with the 128-byte swizzle.  Reduce-adds drop the rows past the sequence end.
bool make_map_accum(CUtensorMap* map, const float* base, int64_t batch_heads, int seqlen, int d) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[3] = {cuuint64_t(d), cuuint64_t(seqlen), cuuint64_t(batch_heads)};
    const cuuint64_t strides[2] = {cuuint64_t(d) * 4, cuuint64_t(seqlen) * cuuint64_t(d) * 4};
    const cuuint32_t box[3] = {32, 32, 1};
    const cuuint32_t elem_strides[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box,
              elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The kernels come in two forms: a lean one for full attention over whole 128-row tiles and a general
// one (causal mask, sliding window, ragged sequence ends).
bool needs_general_form(const ShaoboFa3Params* p) {
    return is_varlen(p) || has_seqused(p) || p->softcap > 0.0f || !band_is_full(band_of(p)) ||
           p->seqlen_q % kTileRows != 0 ||
           p->seqlen_k % kTileRows != 0;
}

// How the tensors of a call are addressed.  Packed sequences are one batch entry of `total` rows in
// the token-major layout ([total, H, D] is [B,S,H,D] with B = 1, S = total).
struct TensorShape {
    int batch;     // batch entries of the tensors (1 when packed)
    int rows_q;    // rows per (batch entry, head) of the query-side tensors
    int rows_k;
    bool bshd;
};
TensorShape shape_of(const ShaoboFa3Params* p) {
    if (is_varlen(p)) return TensorShape{1, int(p->total_q), int(p->total_k), true};
    return TensorShape{p->batch, p->seqlen_q, p->seqlen_k, p->layout == SHAOBO_FA3_LAYOUT_BSHD};
}

RowLayout row_layout(const ShaoboFa3Params* p, int heads, int rows, bool bshd) {
    RowLayout l;
    l.strides = strides_of(bshd, heads, rows, p->head_dim_qk);
    l.heads = heads;
    l.seqlen = rows;
    l.contiguous = bshd ? 0 : 1;
    return l;
}

cudaStream_t stream_of(const ShaoboFa3Params* p) {
    return static_cast<cudaStream_t>(p->reserved_ptr[SHAOBO_FA3_RESERVED_PTR_STREAM]);
}

int sm_count() {
    static std::mutex mu;
    static std::map<int, int> cache;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(dev);
    if (it != cache.end()) return it->second;
    int n = 148;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cache[dev] = n;
    return n;
}

CtaOrderPlan cached_plan(const TileWork& work, int bh, int group, int sms, long long dq_bytes) {
    static std::mutex mu;
    static std::map<std::tuple<int, int, int, int, int, int, int, long long>, CtaOrderPlan> cache;
    const auto key = std::make_tuple(work.band.seqlen_q, work.band.seqlen_k, work.band.left,
                                     work.band.right, bh, group, sms, dq_bytes);
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
    const CtaOrderPlan plan = plan_cta_order(work, bh, group, sms, dq_bytes);
    cache[key] = plan;
    return plan;
}

// Remembers, per CUDA device, that a one-time set-up step has been done
// (function attributes are per device).
struct DeviceOnce {
    std::mutex mu;
    uint64_t mask[2] = {0, 0};
    static int device() {
        int d = 0;
        cudaGetDevice(&d);
        return d & 127;
    }
    bool done() {
        const int d = device();
        std::lock_guard<std::mutex> lock(mu);
        return (mask[d >> 6] >> (d & 63)) & 1;
    }
    void mark() {
        const int d = device();
        std::lock_guard<std::mutex> lock(mu);
        mask[d >> 6] |= uint64_t(1) << (d & 63);
    }
};

// Optional per-stage timing of shaobo_fa3_bwd_v2 (off by default): when
// enabled, four events bracket the three launches of a call on its stream.
// A benchmarking aid for one timed call at a time: the events are shared, so calls from several
// host threads while timing is on record over each other (the mutex only keeps the bookkeeping
// itself consistent).  Off, it costs every call one relaxed atomic load per launch.
struct StageTimer {
    std::atomic<bool> enabled{false};
    std::mutex mu;  // guards valid and ev
    bool valid = false;
    cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};
};
StageTimer g_stage_timer;

void stage_mark(int i, cudaStream_t st) {
    if (!g_stage_timer.enabled.load(std::memory_order_relaxed)) return;
    std::lock_guard<std::mutex> lock(g_stage_timer.mu);
    if (g_stage_timer.enabled.load(std::memory_order_relaxed) && g_stage_timer.ev[i] != nullptr) {
        cudaEventRecord(g_stage_timer.ev[i], st);
        if (i == 3) g_stage_timer.valid = true;
    }
}

// An entry point that launches calls begin() first.  The runtime keeps one "last error" per host
// thread, and an error another library left there (a not-ready event query, for one) must not be
// reported as a failure of this call by finish().
// The first call on a host thread also makes a runtime call that needs the device context, which
// binds the primary context to the thread: tensor maps are encoded through the driver API before
// anything is launched, and the driver API only works on a thread that has a current context (a
// thread started by another library, an autograd worker for one, may not have made one yet).
void begin() {
    thread_local bool context_bound = false;
    if (!context_bound) {
        int lo = 0, hi = 0;  // (a query that needs the context but touches no stream)
        (void)cudaDeviceGetStreamPriorityRange(&lo, &hi);
        context_bound = true;
    }
    (void)cudaGetLastError();
}

int finish(const ShaoboFa3Params* p, bool sync) {
    if (cudaGetLastError() != cudaSuccess) return SHAOBO_FA3_STATUS_HIP_ERROR;
    if (sync && cudaStreamSynchronize(stream_of(p)) != cudaSuccess) {
        return SHAOBO_FA3_STATUS_HIP_ERROR;
    }
    return SHAOBO_FA3_STATUS_SUCCESS;
}

// ------------------------------------------------------------------ delta
template <typename T, int D>
void launch_delta_t(const void* dout, const void* out, const float* aux0, const float* aux1,
                    float* delta, float* sidecar, float* zero_rows, int64_t rows, bool lse,
                    float scale_log2, const RowLayout& layout, cudaStream_t st) {
    constexpr int kRowsPerBlock = 8 * (32 / (D / 8));
    int64_t blocks = (rows + kRowsPerBlock - 1) / kRowsPerBlock;
    const int64_t cap = int64_t(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    // programmatic launch: behind the convert kernel of a preceding call the blocks are placed while
    // that one drains (the kernel itself waits for everything in front of it before it touches memory)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(blocks));
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const T* dout_t = static_cast<const T*>(dout);
    const T* out_t = static_cast<const T*>(out);
    if (lse) {
        cudaLaunchKernelEx(&cfg, delta_sidecar_kernel<T, D, true>, dout_t, out_t, aux0, aux1, delta, sidecar,
                           zero_rows, rows, scale_log2, layout);
    } else {
        cudaLaunchKernelEx(&cfg, delta_sidecar_kernel<T, D, false>, dout_t, out_t, aux0, aux1, delta, sidecar,
                           zero_rows, rows, scale_log2, layout);
    }
}

// sidecar may be null (only delta is written); zero_rows, when non-null, is the fp32 dQ accumulator
// that the same pass clears.
void launch_delta(const ShaoboFa3Params* p, const void* dout, const void* out, const float* aux0,
                  const float* aux1, float* delta, float* sidecar, float* zero_rows, bool lse) {
    const TensorShape shape = shape_of(p);
    const int64_t rows = int64_t(shape.batch) * p->num_heads_q * shape.rows_q;
    const float scale_log2 = p->softmax_scale * kLog2E;
    cudaStream_t st = stream_of(p);
    const bool bf = p->dtype == SHAOBO_FA3_DTYPE_BF16;
    const RowLayout layout = row_layout(p, p->num_heads_q, shape.rows_q, shape.bshd);
    if (p->head_dim_qk == 128) {
        if (bf) launch_delta_t<__nv_bfloat16, 128>(dout, out, aux0, aux1, delta, sidecar, zero_rows, rows, lse, scale_log2, layout, st);
        else launch_delta_t<__half, 128>(dout, out, aux0, aux1, delta, sidecar, zero_rows, rows, lse, scale_log2, layout, st);
    } else {
        if (bf) launch_delta_t<__nv_bfloat16, 64>(dout, out, aux0, aux1, delta, sidecar, zero_rows, rows, lse, scale_log2, layout, st);
        else launch_delta_t<__half, 64>(dout, out, aux0, aux1, delta, sidecar, zero_rows, rows, lse, scale_log2, layout, st);
    }
}

// ---------------------------------------------------------------- convert
// dq = T(scale * dq_accum); with split tiles also dk, dv = T(sum of the slabs of each key tile) (the
// scale of dK was applied before the partial sums were written).
void launch_convert(const ShaoboFa3Params* p, const float* accum, void* dq,
                    const void* dkv_slabs = nullptr, void* dk = nullptr, void* dv = nullptr) {
    ConvertSegments seg{};
    seg.src[0] = accum;
    seg.dst[0] = dq;
    const TensorShape shape = shape_of(p);
    seg.n_vec8[0] = int64_t(shape.batch) * p->num_heads_q * shape.rows_q * p->head_dim_qk / 8;
    seg.scale[0] = p->softmax_scale;
    seg.layout[0] = row_layout(p, p->num_heads_q, shape.rows_q, shape.bshd);
    seg.head_dim = p->head_dim_qk;
    seg.count = 1;
    int64_t total = seg.n_vec8[0];
    const SplitPlan split = dkv_slabs != nullptr ? split_plan(p) : SplitPlan{};
    if (split.chunk_steps > 0) {
        const int64_t n = int64_t(shape.batch) * p->num_heads_kv * shape.rows_k * p->head_dim_qk;
        seg.dst[1] = dk;
        seg.dst[2] = dv;
        seg.n_vec8[1] = seg.n_vec8[2] = n / 8;
        seg.scale[1] = seg.scale[2] = 1.0f;
        seg.layout[1] = seg.layout[2] = row_layout(p, p->num_heads_kv, shape.rows_k, shape.bshd);
        seg.count = 3;
        seg.slabs = dkv_slabs;
        seg.slabs_f16 = p->dtype == SHAOBO_FA3_DTYPE_FP16 ? 1 : 0;
        seg.rows_k = shape.rows_k;
        seg.chunks_per_head = split.chunks_per_head;
        // the chunk list of a head, as the GEMM kernel numbers its CTAs: key tile 0 first
        const Band band = band_of(p);
        const int group = p->num_heads_q / p->num_heads_kv;
        const int tiles = tiles_of(p->seqlen_k);
        int next = 0;
        for (int kt = 0; kt < tiles && kt < kMaxSplitTiles; ++kt) {
            seg.chunk_begin[kt] = static_cast<unsigned short>(next);
            const int steps = group * q_tiles_of_k_tile(kt, band);
            next += (steps + split.chunk_steps - 1) / split.chunk_steps;
        }
        seg.chunk_begin[tiles] = static_cast<unsigned short>(next);
        total += 2 * (n / 8);
    }
    int64_t blocks = (total + 255) / 256;  // one 8-element vector per thread while the grid allows it
    const int64_t cap = int64_t(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(blocks));
    cfg.blockDim = dim3(256);
    cfg.stream = stream_of(p);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;  // the kernel waits for the GEMM kernel itself
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const bool slabs = seg.count == 3;
    if (p->dtype == SHAOBO_FA3_DTYPE_BF16) {
        if (slabs) cudaLaunchKernelEx(&cfg, dq_convert_kernel<__nv_bfloat16, true>, seg);
        else cudaLaunchKernelEx(&cfg, dq_convert_kernel<__nv_bfloat16, false>, seg);
    } else {
        if (slabs) cudaLaunchKernelEx(&cfg, dq_convert_kernel<__half, true>, seg);
        else cudaLaunchKernelEx(&cfg, dq_convert_kernel<__half, false>, seg);
    }
}

// ------------------------------------------------------- fused / dKV kernel
template <typename T, int D, bool kCausal, bool kWithDq, typename TOut, bool kSoftcap = false>
int launch_fused_t(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                   const CUtensorMap& mdo, const CUtensorMap& mdq, const CUtensorMap& mdk,
                   const CUtensorMap& mdv, const FusedArgs& args, int blocks, cudaStream_t st, bool pdl) {
    auto kernel = fused_bwd_kernel<T, D, kCausal, kWithDq, TOut, kSoftcap>;
    static DeviceOnce configured;  // per instantiation and device
    if (!configured.done()) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 FusedCfg<D>::kSmemBytes) != cudaSuccess) {
            return SHAOBO_FA3_STATUS_HIP_ERROR;
        }
        configured.mark();
    }
    // Programmatic dependent launch: set-up and the first loads overlap the tail of the kernel in front
    // (the delta kernel); the kernel itself waits before it touches what that kernel writes.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(FusedCfg<D>::kThreads);
    cfg.dynamicSmemBytes = FusedCfg<D>::kSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kernel, mq, mk, mv, mdo, mdq, mdk, mdv, args) != cudaSuccess) {
        return SHAOBO_FA3_STATUS_HIP_ERROR;
    }
    return SHAOBO_FA3_STATUS_SUCCESS;
}

template <typename T, bool kWithDq, typename TOut>
int launch_fused_d(const ShaoboFa3Params* p, const CUtensorMap& mq, const CUtensorMap& mk,
                   const CUtensorMap& mv, const CUtensorMap& mdo, const CUtensorMap& mdq,
                   const CUtensorMap& mdk, const CUtensorMap& mdv, const FusedArgs& args, int blocks,
                   bool pdl) {
    cudaStream_t st = stream_of(p);
    const bool banded = needs_general_form(p);
    if (p->softcap > 0.0f) {  // softcapped scores: general form only
        return p->head_dim_qk == 128
                   ? launch_fused_t<T, 128, true, kWithDq, TOut, true>(mq, mk, mv, mdo, mdq, mdk, mdv, args, blocks, st, pdl)
                   : launch_fused_t<T, 64, true, kWithDq, TOut, true>(mq, mk, mv, mdo, mdq, mdk, mdv, args, blocks, st, pdl);
    }
    if (p->head_dim_qk == 128) {
        return banded ? launch_fused_t<T, 128, true, kWithDq, TOut>(mq, mk, mv, mdo, mdq, mdk, mdv, args, blocks, st, pdl)
                         : launch_fused_t<T, 128, false, kWithDq, TOut>(mq, mk, mv, mdo, mdq, mdk, mdv, args, blocks, st, pdl);
    }
    return banded ? launch_fused_t<T, 64, true, kWithDq, TOut>(mq, mk, mv, mdo, mdq, mdk, mdv, args, blocks, st, pdl)
                     : launch_fused_t<T, 64, false, kWithDq, TOut>(mq, mk, mv, mdo, mdq, mdk, mdv, args, blocks, st, pdl);
}

// with_dq: fused five-GEMM kernel writing dK/dV in the input dtype and adding
// dQ into dq_accum (already zero).  !with_dq: four-GEMM dK/dV kernel with fp32
// outputs (split path).
// dkv_slabs non-null (fused path only): key tiles are split as split_plan(p) says and every CTA
// writes its partial dK/dV to its own pair of fp32 slabs instead of dk / dv.
// Everything the launch of the five-GEMM / dK-dV kernel needs, built on the host ahead of time: the
// v2 entry prepares it before it launches the delta kernel, so that the GPU does not sit idle
// between the two launches while the host encodes the tensor maps.
struct FusedLaunch {
    int status = SHAOBO_FA3_STATUS_SUCCESS;
    CUtensorMap mq, mk, mv, mdo, mdq, mdk, mdv;
    FusedArgs args;
    int blocks = 0;
    bool with_dq = false;
    bool dkv_f32 = false;
};

FusedLaunch prepare_fused(const ShaoboFa3Params* p, const void* dout, const void* q, const void* k,
                          const void* v, const float* sidecar, float* dq_accum, void* dk, void* dv,
                          bool with_dq, bool dkv_f32 = false, void* dkv_slabs = nullptr) {
    FusedLaunch L;
    L.with_dq = with_dq;
    L.dkv_f32 = dkv_f32;
    CUtensorMap &mq = L.mq, &mk = L.mk, &mv = L.mv, &mdo = L.mdo, &mdq = L.mdq, &mdk = L.mdk, &mdv = L.mdv;
    FusedArgs& args = L.args;
    auto fail = [&](int status) {
        L.status = status;
        return L;
    };
    const bool bf = p->dtype == SHAOBO_FA3_DTYPE_BF16;
    const CUtensorMapDataType type = bf ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const int d = p->head_dim_qk;
    const TensorShape shape = shape_of(p);
    const bool bshd = shape.bshd;
    if (!make_map_16(&mq, type, q, shape.batch, p->num_heads_q, shape.rows_q, d, bshd) ||
        !make_map_16(&mk, type, k, shape.batch, p->num_heads_kv, shape.rows_k, d, bshd) ||
        !make_map_16(&mv, type, v, shape.batch, p->num_heads_kv, shape.rows_k, d, bshd) ||
        !make_map_16(&mdo, type, dout, shape.batch, p->num_heads_q, shape.rows_q, d, bshd)) {
        return fail(SHAOBO_FA3_STATUS_HIP_ERROR);
    }
    if (with_dq) {
        if (!make_map_accum(&mdq, dq_accum, int64_t(shape.batch) * p->num_heads_q, shape.rows_q, d)) {
            return fail(SHAOBO_FA3_STATUS_HIP_ERROR);
        }
    } else {
        mdq = mq;  // unused by the kernel
    }
    const SplitPlan split = (with_dq && dkv_slabs != nullptr) ? split_plan(p) : SplitPlan{};
    // Where the epilogue stores dK / dV through the copy engine: the fp32 slabs of split tiles
    // ([slab][128 rows][D], two slabs per CTA), or dk / dv themselves in boxes of 32 rows (16-bit
    // outputs of fixed-length batches).  Other cases (packed sequences, fp32 outputs) store from
    // registers and do not use these maps.
    if (split.chunk_steps > 0) {
        const int64_t slabs = int64_t(split.chunks_per_head) * p->batch * p->num_heads_kv * 2;
        const bool ok = bf ? make_map_accum(&mdk, static_cast<const float*>(dkv_slabs), slabs, kTileRows, d)
                           : make_map_16(&mdk, type, dkv_slabs, 1, int(slabs), kTileRows, d, false, 32);
        if (!ok) return fail(SHAOBO_FA3_STATUS_HIP_ERROR);
        mdv = mdk;
    } else if (!dkv_f32 && !is_varlen(p)) {
        if (!make_map_16(&mdk, type, dk, shape.batch, p->num_heads_kv, shape.rows_k, d, bshd, 32) ||
            !make_map_16(&mdv, type, dv, shape.batch, p->num_heads_kv, shape.rows_k, d, bshd, 32)) {
            return fail(SHAOBO_FA3_STATUS_HIP_ERROR);
        }
    } else {
        mdk = mq;
        mdv = mq;
    }
    const int n_tiles = tiles_of(plan_seqlen_k(p));
    const Band band = band_of(p);
    const TileWork work = TileWork::of(band);
    const int bh = p->batch * p->num_heads_kv;
    const int group = p->num_heads_q / p->num_heads_kv;
    // bytes of dQ accumulator behind one (batch, KV head): only the fused path adds into it
    const long long dq_bytes_per_head =
        with_dq ? (long long)group * plan_seqlen_q(p) * p->head_dim_qk * 4 : 0;
    const CtaOrderPlan plan = cached_plan(work, bh, group, sm_count(), dq_bytes_per_head);
    args.sidecar = sidecar;
    args.dk = dk;
    args.dv = dv;
    args.dkv_slabs = dkv_slabs;
    // fp32 dK/dV of the split path are always [B,Hkv,Sk,D]; 16-bit outputs follow the layout of K/V
    args.kv_strides = strides_of(bshd && !dkv_f32, p->num_heads_kv, shape.rows_k, d);
    args.batch = p->batch;
    args.heads_q = p->num_heads_q;
    args.heads_kv = p->num_heads_kv;
    args.band = band;
    args.cu_seqlens_q = p->cu_seqlens_q;
    args.cu_seqlens_k = p->cu_seqlens_k;
    args.seqused_q = p->seqused_q;
    args.seqused_k = p->seqused_k;
    args.sidecar_rows = shape.rows_q;
    args.scale = p->softmax_scale;
    args.scale_log2 = p->softmax_scale * kLog2E;
    args.softcap_pre = p->softcap > 0.0f ? p->softmax_scale / p->softcap : 0.0f;
    args.softcap_post = p->softcap * kLog2E;
    args.order_mode = plan.mode;
    args.order_width = plan.width;
    args.head_group = plan.head_group;
    args.chunk_steps = split.chunk_steps;
    args.chunks_per_head = split.chunks_per_head;
    if (split.chunk_steps > 0) {
        // every chunk of every (batch, KV head), longest first (stable: equal lengths keep the order
        // head, key tile, chunk), so that the CTAs beyond one wave are the shortest ones
        struct Chunk { int steps; uint32_t entry; };
        std::vector<Chunk> chunks;
        for (int h = 0; h < bh; ++h) {
            int place = 0;
            for (int kt = 0; kt < n_tiles; ++kt) {
                const int steps = group * q_tiles_of_k_tile(kt, band);
                for (int c = 0, t0 = 0; t0 < steps; ++c, t0 += split.chunk_steps, ++place) {
                    const int n = std::min(split.chunk_steps, steps - t0);
                    const uint32_t slab = uint32_t(h * split.chunks_per_head + place);
                    chunks.push_back(Chunk{n, uint32_t(kt) | (uint32_t(c) << 8) | (slab << 16)});
                }
            }
        }
        if (chunks.size() > size_t(kMaxSplitCtas) || n_tiles > 255) return fail(SHAOBO_FA3_STATUS_UNSUPPORTED);
        std::stable_sort(chunks.begin(), chunks.end(), [](const Chunk& x, const Chunk& y) { return x.steps > y.steps; });
        for (size_t i = 0; i < chunks.size(); ++i) args.cta_table[i] = chunks[i].entry;
    }
    const int64_t blocks64 = split.chunk_steps > 0 ? int64_t(split.chunks_per_head) * bh : int64_t(n_tiles) * bh;
    if (blocks64 > 0x7fffffffLL) return fail(SHAOBO_FA3_STATUS_UNSUPPORTED);
    L.blocks = int(blocks64);
    return L;
}

int run_fused(const ShaoboFa3Params* p, const FusedLaunch& L, bool pdl) {
    if (L.status != SHAOBO_FA3_STATUS_SUCCESS) return L.status;
    const bool bf = p->dtype == SHAOBO_FA3_DTYPE_BF16;
    const CUtensorMap &mq = L.mq, &mk = L.mk, &mv = L.mv, &mdo = L.mdo, &mdq = L.mdq, &mdk = L.mdk, &mdv = L.mdv;
    const FusedArgs& args = L.args;
    const int blocks = L.blocks;
    if (L.with_dq) {
        return bf ? launch_fused_d<__nv_bfloat16, true, __nv_bfloat16>(p, mq, mk, mv, mdo, mdq, mdk, mdv, args, blocks, pdl)
                  : launch_fused_d<__half, true, __half>(p, mq, mk, mv, mdo, mdq, mdk, mdv, args, blocks, pdl);
    }
    if (L.dkv_f32) {
        return bf ? launch_fused_d<__nv_bfloat16, false, float>(p, mq, mk, mv, mdo, mdq, mdk, mdv, args, blocks, pdl)
                  : launch_fused_d<__half, false, float>(p, mq, mk, mv, mdo, mdq, mdk, mdv, args, blocks, pdl);
    }
    return bf ? launch_fused_d<__nv_bfloat16, false, __nv_bfloat16>(p, mq, mk, mv, mdo, mdq, mdk, mdv, args, blocks, pdl)
              : launch_fused_d<__half, false, __half>(p, mq, mk, mv, mdo, mdq, mdk, mdv, args, blocks, pdl);
}

int launch_fused(const ShaoboFa3Params* p, const void* dout, const void* q, const void* k,
                 const void* v, const float* sidecar, float* dq_accum, void* dk, void* dv,
                 bool with_dq, bool dkv_f32 = false, void* dkv_slabs = nullptr, bool pdl = false) {
    return run_fused(p, prepare_fused(p, dout, q, k, v, sidecar, dq_accum, dk, dv, with_dq, dkv_f32, dkv_slabs), pdl);
}

// -------------------------------------------------------------- dQ kernel
template <typename T, int D, bool kCausal, typename TOut, bool kSoftcap = false>
int launch_dq_t(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                const CUtensorMap& mdo, const DqArgs& args, int blocks, cudaStream_t st) {
    auto kernel = dq_bwd_kernel<T, D, kCausal, TOut, kSoftcap>;
    static DeviceOnce configured;
    if (!configured.done()) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 DqCfg<D>::kSmemBytes) != cudaSuccess) {
            return SHAOBO_FA3_STATUS_HIP_ERROR;
        }
        configured.mark();
    }
    kernel<<<blocks, DqCfg<D>::kThreads, DqCfg<D>::kSmemBytes, st>>>(mq, mk, mv, mdo, args);
    return SHAOBO_FA3_STATUS_SUCCESS;
}

template <typename T, typename TOut>
int launch_dq_d(const ShaoboFa3Params* p, const CUtensorMap& mq, const CUtensorMap& mk,
                const CUtensorMap& mv, const CUtensorMap& mdo, const DqArgs& args, int blocks) {
    cudaStream_t st = stream_of(p);
    const bool banded = needs_general_form(p);
    if (p->softcap > 0.0f) {
        return p->head_dim_qk == 128 ? launch_dq_t<T, 128, true, TOut, true>(mq, mk, mv, mdo, args, blocks, st)
                                     : launch_dq_t<T, 64, true, TOut, true>(mq, mk, mv, mdo, args, blocks, st);
    }
    if (p->head_dim_qk == 128) {
        return banded ? launch_dq_t<T, 128, true, TOut>(mq, mk, mv, mdo, args, blocks, st)
                         : launch_dq_t<T, 128, false, TOut>(mq, mk, mv, mdo, args, blocks, st);
    }
    return banded ? launch_dq_t<T, 64, true, TOut>(mq, mk, mv, mdo, args, blocks, st)
                     : launch_dq_t<T, 64, false, TOut>(mq, mk, mv, mdo, args, blocks, st);
}

// Three-GEMM dQ kernel (split path).  out_f32 selects fp32 or input-dtype dq.  The row statistics
// are the packed sidecar, or (sidecar null) aux0 / aux1 / delta as three arrays.
int launch_dq(const ShaoboFa3Params* p, const void* dout, const void* q, const void* k,
              const void* v, const float* sidecar, void* dq, bool out_f32,
              const float* aux0 = nullptr, const float* aux1 = nullptr, const float* delta = nullptr) {
    const bool bf = p->dtype == SHAOBO_FA3_DTYPE_BF16;
    const CUtensorMapDataType type = bf ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const int d = p->head_dim_qk;
    const TensorShape shape = shape_of(p);
    const bool bshd = shape.bshd;
    CUtensorMap mq, mk, mv, mdo;
    if (!make_map_16(&mq, type, q, shape.batch, p->num_heads_q, shape.rows_q, d, bshd) ||
        !make_map_16(&mk, type, k, shape.batch, p->num_heads_kv, shape.rows_k, d, bshd) ||
        !make_map_16(&mv, type, v, shape.batch, p->num_heads_kv, shape.rows_k, d, bshd) ||
        !make_map_16(&mdo, type, dout, shape.batch, p->num_heads_q, shape.rows_q, d, bshd)) {
        return SHAOBO_FA3_STATUS_HIP_ERROR;
    }
    DqArgs args;
    args.sidecar = sidecar;
    args.aux0 = aux0;
    args.aux1 = aux1;
    args.delta = delta;
    args.dq = dq;
    // fp32 dQ of the split path is always [B,Hq,Sq,D]; 16-bit dQ follows the layout of Q
    args.q_strides = strides_of(bshd && !out_f32, p->num_heads_q, shape.rows_q, d);
    args.batch = p->batch;
    args.heads_q = p->num_heads_q;
    args.heads_kv = p->num_heads_kv;
    args.band = band_of(p);
    args.cu_seqlens_q = p->cu_seqlens_q;
    args.cu_seqlens_k = p->cu_seqlens_k;
    args.seqused_q = p->seqused_q;
    args.seqused_k = p->seqused_k;
    args.sidecar_rows = shape.rows_q;
    args.scale = p->softmax_scale;
    args.scale_log2 = p->softmax_scale * kLog2E;
    args.softcap_pre = p->softcap > 0.0f ? p->softmax_scale / p->softcap : 0.0f;
    args.softcap_post = p->softcap * kLog2E;
    const int64_t blocks64 = int64_t(tiles_of(plan_seqlen_q(p))) * p->batch * p->num_heads_q;
    if (blocks64 > 0x7fffffffLL) return SHAOBO_FA3_STATUS_UNSUPPORTED;
    const int blocks = int(blocks64);
    if (out_f32) {
        return bf ? launch_dq_d<__nv_bfloat16, float>(p, mq, mk, mv, mdo, args, blocks)
                  : launch_dq_d<__half, float>(p, mq, mk, mv, mdo, args, blocks);
    }
    return bf ? launch_dq_d<__nv_bfloat16, __nv_bfloat16>(p, mq, mk, mv, mdo, args, blocks)
              : launch_dq_d<__half, __half>(p, mq, mk, mv, mdo, args, blocks);
}

// ---------------------------------------------------------- forward kernel
template <typename T, int D, bool kMasked, bool kSoftcap = false>
int launch_fwd_t(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                 const FwdArgs& args, int blocks, cudaStream_t st) {
    auto kernel = fwd_kernel<T, D, kMasked, kSoftcap>;
    static DeviceOnce configured;
    if (!configured.done()) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 FwdCfg<D>::kSmemBytes) != cudaSuccess) {
            return SHAOBO_FA3_STATUS_HIP_ERROR;
        }
        configured.mark();
    }
    kernel<<<blocks, FwdCfg<D>::kThreads, FwdCfg<D>::kSmemBytes, st>>>(mq, mk, mv, args);
    return SHAOBO_FA3_STATUS_SUCCESS;
}

template <typename T>
int launch_fwd_d(const ShaoboFa3Params* p, const CUtensorMap& mq, const CUtensorMap& mk,
                 const CUtensorMap& mv, const FwdArgs& args, int blocks) {
    cudaStream_t st = stream_of(p);
    const bool masked = needs_general_form(p);
    if (p->softcap > 0.0f) {
        return p->head_dim_qk == 128 ? launch_fwd_t<T, 128, true, true>(mq, mk, mv, args, blocks, st)
                                     : launch_fwd_t<T, 64, true, true>(mq, mk, mv, args, blocks, st);
    }
    if (p->head_dim_qk == 128) {
        return masked ? launch_fwd_t<T, 128, true>(mq, mk, mv, args, blocks, st)
                      : launch_fwd_t<T, 128, false>(mq, mk, mv, args, blocks, st);
    }
    return masked ? launch_fwd_t<T, 64, true>(mq, mk, mv, args, blocks, st)
                  : launch_fwd_t<T, 64, false>(mq, mk, mv, args, blocks, st);
}

int launch_fwd(const ShaoboFa3Params* p, const void* q, const void* k, const void* v, void* out,
               float* lse) {
    const bool bf = p->dtype == SHAOBO_FA3_DTYPE_BF16;
    const CUtensorMapDataType type = bf ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const int d = p->head_dim_qk;
    const TensorShape shape = shape_of(p);
    CUtensorMap mq, mk, mv;
    if (!make_map_16(&mq, type, q, shape.batch, p->num_heads_q, shape.rows_q, d, shape.bshd) ||
        !make_map_16(&mk, type, k, shape.batch, p->num_heads_kv, shape.rows_k, d, shape.bshd) ||
        !make_map_16(&mv, type, v, shape.batch, p->num_heads_kv, shape.rows_k, d, shape.bshd)) {
        return SHAOBO_FA3_STATUS_HIP_ERROR;
    }
    FwdArgs args;
    args.out = out;
    args.lse = lse;
    args.o_strides = strides_of(shape.bshd, p->num_heads_q, shape.rows_q, d);
    args.batch = p->batch;
    args.heads_q = p->num_heads_q;
    args.heads_kv = p->num_heads_kv;
    args.band = band_of(p);
    args.cu_seqlens_q = p->cu_seqlens_q;
    args.cu_seqlens_k = p->cu_seqlens_k;
    args.seqused_q = p->seqused_q;
    args.seqused_k = p->seqused_k;
    args.lse_rows = shape.rows_q;
    args.scale_log2 = p->softmax_scale * kLog2E;
    args.softcap_pre = p->softcap > 0.0f ? p->softmax_scale / p->softcap : 0.0f;
    args.softcap_post = p->softcap * kLog2E;
    // one CTA per pair of query tiles
    const int64_t blocks64 = int64_t((tiles_of(plan_seqlen_q(p)) + 1) / 2) * p->batch * p->num_heads_q;
    if (blocks64 > 0x7fffffffLL) return SHAOBO_FA3_STATUS_UNSUPPORTED;
    return bf ? launch_fwd_d<__nv_bfloat16>(p, mq, mk, mv, args, int(blocks64))
              : launch_fwd_d<__half>(p, mq, mk, mv, args, int(blocks64));
}

bool stage_params_ok(const ShaoboFa3Params* p) {
    // (the component entry points take fixed-length batches only)
    return p != nullptr && !is_varlen(p) && !has_seqused(p) && p->softcap == 0.0f && dtype_supported(p->dtype) && layout_supported(p->layout) &&
           (p->causal == 0 || p->causal == 1) && fused_shape_ok(p);
}

}  // namespace
}  // namespace fa3b200

using namespace fa3b200;

// Extension (no counterpart in the reference): reads and optionally clears the
// device-side error flag that a kernel raises when a bounded wait runs out
// (1) or shared memory is misaligned (2).  Synchronises the device.
extern "C" int shaobo_fa3_b200_device_error(int clear) {
    int value = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(&value, g_device_error, sizeof(int)) != cudaSuccess) return -1;
    if (clear && value != 0) {
        const int zero = 0;
        if (cudaMemcpyToSymbol(g_device_error, &zero, sizeof(int)) != cudaSuccess) return -1;
    }
    return value;
}

// Extension (no counterpart in the reference): per-stage device timing of
// shaobo_fa3_bwd_v2 for benchmarking.  enable != 0 creates four CUDA events on
// the current device and makes every following v2 call record them around its
// three launches; enable == 0 stops recording and destroys them.
extern "C" int shaobo_fa3_b200_stage_timing(int enable) {
    std::lock_guard<std::mutex> lock(g_stage_timer.mu);
    if (enable != 0 && !g_stage_timer.enabled.load()) {
        for (auto& e : g_stage_timer.ev) {
            if (cudaEventCreate(&e) != cudaSuccess) {
                for (auto& made : g_stage_timer.ev) {
                    if (made != nullptr) cudaEventDestroy(made);
                    made = nullptr;
                }
                return SHAOBO_FA3_STATUS_HIP_ERROR;
            }
        }
        g_stage_timer.valid = false;
        g_stage_timer.enabled.store(true);
    } else if (enable == 0 && g_stage_timer.enabled.load()) {
        g_stage_timer.enabled.store(false);
        for (auto& e : g_stage_timer.ev) {
            cudaEventDestroy(e);
            e = nullptr;
        }
    }
    return SHAOBO_FA3_STATUS_SUCCESS;
}

// Milliseconds of the three stages of the last timed v2 call (waits for it):
// fused path {delta, five-GEMM kernel, dQ convert}; deterministic path
// {delta, dK/dV kernel, dQ kernel}.
extern "C" int shaobo_fa3_b200_last_stage_ms(float* ms3) {
    std::lock_guard<std::mutex> lock(g_stage_timer.mu);
    if (!g_stage_timer.enabled.load() || !g_stage_timer.valid || ms3 == nullptr) {
        return SHAOBO_FA3_STATUS_INVALID_VALUE;
    }
    if (cudaEventSynchronize(g_stage_timer.ev[3]) != cudaSuccess) return SHAOBO_FA3_STATUS_HIP_ERROR;
    for (int i = 0; i < 3; ++i) {
        if (cudaEventElapsedTime(&ms3[i], g_stage_timer.ev[i], g_stage_timer.ev[i + 1]) != cudaSuccess) {
            return SHAOBO_FA3_STATUS_HIP_ERROR;
        }
    }
    return SHAOBO_FA3_STATUS_SUCCESS;
}

#ifdef FA3B200_TRACE
// Instrumented builds only: copy out (and clear) the per-CTA cycle stamps and the row-wise kernels'
// first-start / last-end times.
extern "C" int shaobo_fa3_b200_trace_read(long long* stamps, long long* rowwise) {
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(stamps, g_trace, sizeof(long long) * kTraceCtas * 4 * kTraceEvents) != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(rowwise, g_trace_rowwise, sizeof(long long) * 4) != cudaSuccess) return -1;
    static long long zeros[kTraceCtas * 4 * kTraceEvents];
    cudaMemcpyToSymbol(g_trace, zeros, sizeof(zeros));
    const long long init[4] = {0x7fffffffffffffffLL, 0, 0x7fffffffffffffffLL, 0};
    cudaMemcpyToSymbol(g_trace_rowwise, init, sizeof(init));
    return 0;
}
#endif

extern "C" int shaobo_fa3_bwd_dot_do_o(const void* dout, const void* out, const void* aux0,
                                       const void* aux1, void* delta, void* packed_sidecar,
                                       const ShaoboFa3Params* params) {
    begin();
    const bool ok = params != nullptr && params->batch > 0 && params->seqlen_q > 0 &&
                    params->num_heads_q > 0 && head_dim_supported(params->head_dim_qk) &&
                    params->head_dim_v == params->head_dim_qk && dtype_supported(params->dtype) &&
                    layout_supported(params->layout) &&
                    (params->softmax_aux_mode == SHAOBO_FA3_SOFTMAX_AUX_SMAX_SSUM ||
                     params->softmax_aux_mode == SHAOBO_FA3_SOFTMAX_AUX_LSE);
    if (!ok) return SHAOBO_FA3_STATUS_UNSUPPORTED;
    const bool lse = params->softmax_aux_mode == SHAOBO_FA3_SOFTMAX_AUX_LSE;
    if (dout == nullptr || out == nullptr || aux0 == nullptr || (!lse && aux1 == nullptr) ||
        delta == nullptr || packed_sidecar == nullptr) {
        return SHAOBO_FA3_STATUS_INVALID_VALUE;
    }
    launch_delta(params, dout, out, static_cast<const float*>(aux0),
                 static_cast<const float*>(aux1), static_cast<float*>(delta),
                 static_cast<float*>(packed_sidecar), nullptr, lse);
    return finish(params, params->sync_after_launch != 0);
}

extern "C" int shaobo_fa3_bwd_fused5(const void* dout, const void* q, const void* k,
                                     const void* v, const void* packed_sidecar, void* dq, void* dk,
                                     void* dv, const ShaoboFa3Params* params) {
    begin();
    if (params == nullptr || dout == nullptr || q == nullptr || k == nullptr || v == nullptr ||
        packed_sidecar == nullptr || dq == nullptr || dk == nullptr || dv == nullptr) {
        return SHAOBO_FA3_STATUS_INVALID_VALUE;
    }
    if (!stage_params_ok(params)) return SHAOBO_FA3_STATUS_UNSUPPORTED;
    const size_t dq_bytes = dq_accum_bytes(params);
    const size_t dkv_bytes = dkv_accum_bytes(params);
    const size_t need = dq_bytes + dkv_bytes;
    if (dq_bytes == 0 || params->workspace == nullptr || params->workspace_bytes < need) {
        return SHAOBO_FA3_STATUS_INVALID_VALUE;
    }
    float* accum = static_cast<float*>(params->workspace);
    void* dkv_slabs = dkv_bytes != 0 ? static_cast<uint8_t*>(params->workspace) + dq_bytes : nullptr;
    if (cudaMemsetAsync(accum, 0, dq_bytes, stream_of(params)) != cudaSuccess) {  // (the slabs are written, not added into)
        return SHAOBO_FA3_STATUS_HIP_ERROR;
    }
    int status = launch_fused(params, dout, q, k, v, static_cast<const float*>(packed_sidecar),
                              accum, dk, dv, true, false, dkv_slabs);
    if (status != SHAOBO_FA3_STATUS_SUCCESS) return status;
    launch_convert(params, accum, dq, dkv_slabs, dk, dv);
    return finish(params, params->sync_after_launch != 0);
}

extern "C" int shaobo_fa3_bwd_dkv(const void* dout, const void* q, const void* k, const void* v,
                                  const void* out, const void* aux0, const void* aux1, void* dq,
                                  void* dk, void* dv, const ShaoboFa3Params* params) {
    begin();
    (void)out; (void)aux0; (void)aux1; (void)dq;
    if (params == nullptr) return SHAOBO_FA3_STATUS_INVALID_VALUE;
    if (params->dkv_path == SHAOBO_FA3_DKV_PATH_REFERENCE) return SHAOBO_FA3_STATUS_NOT_IMPLEMENTED;
    if (params->dkv_path != SHAOBO_FA3_DKV_PATH_CANONICAL || !stage_params_ok(params)) {
        return SHAOBO_FA3_STATUS_UNSUPPORTED;
    }
    const void* sidecar = params->reserved_ptr[SHAOBO_FA3_RESERVED_PTR_SIDECAR];
    if (dout == nullptr || q == nullptr || k == nullptr || v == nullptr || dk == nullptr ||
        dv == nullptr || sidecar == nullptr) {
        return SHAOBO_FA3_STATUS_INVALID_VALUE;
    }
    const int status = launch_fused(params, dout, q, k, v, static_cast<const float*>(sidecar),
                                    nullptr, dk, dv, false, true);
    if (status != SHAOBO_FA3_STATUS_SUCCESS) return status;
    return finish(params, params->sync_after_launch != 0);
}

extern "C" int shaobo_fa3_bwd(const void* dout, const void* q, const void* k, const void* v,
                              const void* out, const void* aux0, const void* aux1, void* dq,
                              void* dk, void* dv, const ShaoboFa3Params* params) {
    return shaobo_fa3_bwd_dkv(dout, q, k, v, out, aux0, aux1, dq, dk, dv, params);
}

extern "C" int shaobo_fa3_bwd_dq(const void* dout, const void* q, const void* k, const void* v,
                                 const void* out, const void* aux0, const void* aux1, void* dq,
                                 void* dk, void* dv, const ShaoboFa3Params* params) {
    begin();
    (void)out; (void)dk; (void)dv;
    if (params == nullptr) return SHAOBO_FA3_STATUS_INVALID_VALUE;
    if (params->dq_path == SHAOBO_FA3_DQ_PATH_REFERENCE) return SHAOBO_FA3_STATUS_NOT_IMPLEMENTED;
    if (params->dq_path != SHAOBO_FA3_DQ_PATH_CANONICAL || !stage_params_ok(params)) {
        return SHAOBO_FA3_STATUS_UNSUPPORTED;
    }
    // Two calling conventions.  The reference's (src/dq_kernel.cpp:1515-1549): row maximum and row
    // sum in softmax_aux0 / softmax_aux1 (or the log-sum-exp and NULL when softmax_aux_mode is LSE)
    // and delta in reserved_ptr[0]; when these are all given they are used, as in the reference.
    // Otherwise the packed sidecar of the delta stage in reserved_ptr[3], like the dK/dV half.
    const float* sidecar = static_cast<const float*>(params->reserved_ptr[SHAOBO_FA3_RESERVED_PTR_SIDECAR]);
    const float* delta = static_cast<const float*>(params->reserved_ptr[SHAOBO_FA3_RESERVED_PTR_DELTA]);
    const bool lse = params->softmax_aux_mode == SHAOBO_FA3_SOFTMAX_AUX_LSE;
    const bool arrays_complete = aux0 != nullptr && (lse || aux1 != nullptr) && delta != nullptr;
    if (dout == nullptr || q == nullptr || k == nullptr || v == nullptr || dq == nullptr ||
        (sidecar == nullptr && !arrays_complete)) {
        return SHAOBO_FA3_STATUS_INVALID_VALUE;
    }
    const int status =
        arrays_complete
            ? launch_dq(params, dout, q, k, v, nullptr, dq, true, static_cast<const float*>(aux0),
                        lse ? nullptr : static_cast<const float*>(aux1), delta)
            : launch_dq(params, dout, q, k, v, sidecar, dq, true);
    if (status != SHAOBO_FA3_STATUS_SUCCESS) return status;
    return finish(params, params->sync_after_launch != 0);
}

extern "C" int shaobo_fa3_bwd_v2(const void* dout, const void* q, const void* k, const void* v,
                                 const void* out, const void* softmax_lse, void* dq, void* dk,
                                 void* dv, void* softmax_d, const ShaoboFa3Params* params) {
    begin();
    const int validation = validate_v2(params);
    if (validation != SHAOBO_FA3_STATUS_SUCCESS) return validation;
    if (dout == nullptr || q == nullptr || k == nullptr || v == nullptr || out == nullptr ||
        softmax_lse == nullptr || dq == nullptr || dk == nullptr || dv == nullptr) {
        return SHAOBO_FA3_STATUS_INVALID_VALUE;
    }
    const V2Workspace ws = v2_workspace(params);
    if (!ws.valid || params->workspace == nullptr || params->workspace_bytes < ws.total_bytes) {
        return SHAOBO_FA3_STATUS_INVALID_VALUE;
    }
    uint8_t* base = static_cast<uint8_t*>(params->workspace);
    float* accum = reinterpret_cast<float*>(base);
    float* delta = softmax_d != nullptr ? static_cast<float*>(softmax_d)
                                        : reinterpret_cast<float*>(base + ws.delta_offset);
    float* sidecar = reinterpret_cast<float*>(base + ws.sidecar_offset);

    ShaoboFa3Params launch = *params;
    launch.softmax_aux_mode = SHAOBO_FA3_SOFTMAX_AUX_LSE;
    if (launch.softmax_scale_is_set == 0) {
        launch.softmax_scale = 1.0f / std::sqrt(float(launch.head_dim_qk));
    }

    int status = SHAOBO_FA3_STATUS_SUCCESS;
    if (launch.deterministic == 0) {
        // delta + sidecar, and the dQ accumulator is cleared in the same pass
        cudaStream_t st = stream_of(&launch);
        void* dkv_slabs = ws.dkv_accum_bytes != 0 ? base + ws.dq_accum_bytes : nullptr;
        // host work of the second launch first, then the three launches back to back
        const FusedLaunch fused = prepare_fused(&launch, dout, q, k, v, sidecar, accum, dk, dv, true, false, dkv_slabs);
        if (fused.status != SHAOBO_FA3_STATUS_SUCCESS) return fused.status;
        stage_mark(0, st);
        launch_delta(&launch, dout, out, static_cast<const float*>(softmax_lse), nullptr, delta,
                     sidecar, accum, true);
        stage_mark(1, st);
        status = run_fused(&launch, fused, true);
        stage_mark(2, st);
        if (status == SHAOBO_FA3_STATUS_SUCCESS) launch_convert(&launch, accum, dq, dkv_slabs, dk, dv);
        stage_mark(3, st);
    } else {
        // Atomic-free split path (bitwise reproducible): dK/dV by the four-GEMM
        // kernel, dQ by the three-GEMM kernel; both write the input dtype directly.
        cudaStream_t st = stream_of(&launch);
        stage_mark(0, st);
        launch_delta(&launch, dout, out, static_cast<const float*>(softmax_lse), nullptr, delta,
                     sidecar, nullptr, true);
        stage_mark(1, st);
        status = launch_fused(&launch, dout, q, k, v, sidecar, nullptr, dk, dv, false, false);
        stage_mark(2, st);
        if (status == SHAOBO_FA3_STATUS_SUCCESS) {
            status = launch_dq(&launch, dout, q, k, v, sidecar, dq, false);
        }
        stage_mark(3, st);
    }
    if (status != SHAOBO_FA3_STATUS_SUCCESS) return status;
    return finish(&launch, params->sync_after_launch != 0);
}

// Extension (no counterpart in the reference, which has no forward at all): the attention forward
// that produces the out and softmax_lse inputs of shaobo_fa3_bwd_v2.  Same parameter block and the
// same validation as the backward (deterministic is ignored: the forward has no atomics); no
// workspace.
extern "C" int shaobo_fa3_b200_fwd(const void* q, const void* k, const void* v, void* out,
                                   void* softmax_lse, const ShaoboFa3Params* params) {
    begin();
    const int validation = validate_v2(params);
    if (validation != SHAOBO_FA3_STATUS_SUCCESS) return validation;
    if (q == nullptr || k == nullptr || v == nullptr || out == nullptr || softmax_lse == nullptr) {
        return SHAOBO_FA3_STATUS_INVALID_VALUE;
    }
    ShaoboFa3Params launch = *params;
    if (launch.softmax_scale_is_set == 0) {
        launch.softmax_scale = 1.0f / std::sqrt(float(launch.head_dim_qk));
    }
    const int status = launch_fwd(&launch, q, k, v, out, static_cast<float*>(softmax_lse));
    if (status != SHAOBO_FA3_STATUS_SUCCESS) return status;
    return finish(&launch, params->sync_after_launch != 0);
}

// ---------------------------------------------------------------------------
// Backward for callers that cannot allocate device memory.
//
// Some hosts of this library never get to call cudaMalloc: a plugin that runs
// inside another framework's pre-sized memory arena, a real-time loop where
// allocation is forbidden after start-up, or a process whose memory budget is
// fixed by its launcher.  shaobo_fa3_bwd_v2 needs scratch beyond its inputs and
// outputs (the fp32 dQ accumulator, delta and the packed sidecar), which such a
// caller has nowhere to get from.  This entry point keeps that scratch in a
// fixed array that is part of the library image: it exists on every GPU that
// loads the library, from load until the process exits, whether or not the
// entry point is ever called.  It holds whatever the caller's workspace would:
// the dQ accumulator, the partial dK/dV sums of split key tiles, delta and the
// sidecar; a problem fits when shaobo_fa3_bwd_v2_workspace_bytes says so.
__device__ __align__(256) static unsigned char g_static_scratch[SHAOBO_FA3_B200_STATIC_SCRATCH_BYTES];

namespace {

// Device address of g_static_scratch, resolved once per device.  In host code
// the array's name is only a handle for the runtime, not an address a kernel
// could use, so the address is asked for explicitly.
struct StaticScratch {
    std::mutex mu;
    void* ptr[128] = {};
    bool known[128] = {};
    void* get() {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 128) return nullptr;
        std::lock_guard<std::mutex> lock(mu);
        if (!known[dev]) {
            void* p = nullptr;
            if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) {
                (void)cudaGetLastError();
                return nullptr;
            }
            ptr[dev] = p;
            known[dev] = true;
        }
        return ptr[dev];
    }
};
StaticScratch g_scratch_lookup;

}  // namespace

extern "C" int shaobo_fa3_b200_bwd_v2_noalloc(const void* dout, const void* q, const void* k,
                                              const void* v, const void* out,
                                              const void* softmax_lse, void* dq, void* dk,
                                              void* dv, void* softmax_d,
                                              const ShaoboFa3Params* params) {
    const int validation = validate_v2(params);
    if (validation != SHAOBO_FA3_STATUS_SUCCESS) return validation;
    // same order of checks as shaobo_fa3_bwd_v2: tensor pointers before anything about scratch
    if (dout == nullptr || q == nullptr || k == nullptr || v == nullptr || out == nullptr ||
        softmax_lse == nullptr || dq == nullptr || dk == nullptr || dv == nullptr) {
        return SHAOBO_FA3_STATUS_INVALID_VALUE;
    }
    const V2Workspace ws = v2_workspace(params);
    if (!ws.valid) return SHAOBO_FA3_STATUS_INVALID_VALUE;
    if (ws.total_bytes > size_t(SHAOBO_FA3_B200_STATIC_SCRATCH_BYTES)) {
        // the problem needs more scratch than the built-in array holds
        return SHAOBO_FA3_STATUS_UNSUPPORTED;
    }
    void* scratch = g_scratch_lookup.get();
    if (scratch == nullptr) return SHAOBO_FA3_STATUS_HIP_ERROR;
    ShaoboFa3Params with_scratch = *params;
    with_scratch.workspace = scratch;
    with_scratch.workspace_bytes = size_t(SHAOBO_FA3_B200_STATIC_SCRATCH_BYTES);
    return shaobo_fa3_bwd_v2(dout, q, k, v, out, softmax_lse, dq, dk, dv, softmax_d, &with_scratch);
}

// ---------------------------------------------------------------------------
// Backward for callers whose tensors live in host memory.
//
// The inputs are copied to the GPU, shaobo_fa3_bwd_v2 runs, dq/dk/dv are copied back.  Over PCIe the
// copies, not the kernels, bound such a call, so the problem is cut into contiguous (batch, KV head)
// shards (the backward has no reduction across them) that go round-robin over a few streams: the
// host-to-device copy of one shard, the kernels of another and the device-to-host copy of a third
// overlap.  Device memory comes from the caller (one staging buffer); the streams and events the
// pipeline needs are created once per device and kept.
namespace {

constexpr int kHostLanes = 3;

struct HostLanes {
    std::mutex mu;             // guards creation
    std::mutex enqueue[128];   // one call at a time enqueues on a device's lanes (see the entry point)
    bool ready[128] = {};
    cudaStream_t stream[128][kHostLanes] = {};
    cudaStream_t aux[128][kHostLanes] = {};      // second stream of a lane: carries half of its copies-in
    cudaEvent_t fork[128] = {};
    cudaEvent_t join[128][kHostLanes] = {};
    cudaEvent_t aux_done[128][kHostLanes] = {};
    bool get(int dev) {
        std::lock_guard<std::mutex> lock(mu);
        if (ready[dev]) return true;
        bool ok = cudaEventCreateWithFlags(&fork[dev], cudaEventDisableTiming) == cudaSuccess;
        for (int i = 0; ok && i < kHostLanes; ++i) {
            ok = cudaStreamCreateWithFlags(&stream[dev][i], cudaStreamNonBlocking) == cudaSuccess &&
                 cudaStreamCreateWithFlags(&aux[dev][i], cudaStreamNonBlocking) == cudaSuccess &&
                 cudaEventCreateWithFlags(&join[dev][i], cudaEventDisableTiming) == cudaSuccess &&
                 cudaEventCreateWithFlags(&aux_done[dev][i], cudaEventDisableTiming) == cudaSuccess;
        }
        if (!ok) {  // give back what was made: the next call starts from nothing
            if (fork[dev] != nullptr) cudaEventDestroy(fork[dev]);
            fork[dev] = nullptr;
            for (int i = 0; i < kHostLanes; ++i) {
                if (stream[dev][i] != nullptr) cudaStreamDestroy(stream[dev][i]);
                if (aux[dev][i] != nullptr) cudaStreamDestroy(aux[dev][i]);
                if (join[dev][i] != nullptr) cudaEventDestroy(join[dev][i]);
                if (aux_done[dev][i] != nullptr) cudaEventDestroy(aux_done[dev][i]);
                stream[dev][i] = nullptr;
                aux[dev][i] = nullptr;
                join[dev][i] = nullptr;
                aux_done[dev][i] = nullptr;
            }
            (void)cudaGetLastError();
            return false;
        }
        ready[dev] = true;
        return true;
    }
};
HostLanes g_host_lanes;

// One piece of the (batch x KV head) range: whole batch entries, or a KV-head range inside one.
struct HostPiece {
    int batch_begin, batch_count, kv_head_begin, kv_head_count;
};

// First unit of shard r of n: contiguous shards, as even as possible.  (A small last shard, to shorten
// the tail nothing overlaps, measured slower: 395 against 368 us on 16.8 MB.)
long long host_shard_begin(long long units, int r, int n) { return units * r / n; }

// Pieces of shard r of n.
int host_pieces(const ShaoboFa3Params* p, int r, int n, HostPiece* out) {
    const long long units = (long long)p->batch * p->num_heads_kv;
    long long lo = host_shard_begin(units, r, n);
    const long long hi = r + 1 == n ? units : host_shard_begin(units, r + 1, n);
    int count = 0;
    while (lo < hi && count < 3) {
        const int b = int(lo / p->num_heads_kv), h = int(lo % p->num_heads_kv);
        if (h == 0 && hi - lo >= p->num_heads_kv) {
            const int nb = int((hi - lo) / p->num_heads_kv);
            out[count++] = HostPiece{b, nb, 0, p->num_heads_kv};
            lo += (long long)nb * p->num_heads_kv;
        } else {
            const int nh = int(std::min<long long>(p->num_heads_kv - h, hi - lo));
            out[count++] = HostPiece{b, 1, h, nh};
            lo += nh;
        }
    }
    return count;
}

ShaoboFa3Params piece_params(const ShaoboFa3Params* p, const HostPiece& pc) {
    ShaoboFa3Params s = *p;
    const int group = p->num_heads_q / p->num_heads_kv;
    s.batch = pc.batch_count;
    s.num_heads_kv = pc.kv_head_count;
    s.num_heads_q = pc.kv_head_count * group;
    s.sync_after_launch = 0;
    return s;
}

bool host_call_supported(const ShaoboFa3Params* p) {
    return validate_v2(p) == SHAOBO_FA3_STATUS_SUCCESS && !is_varlen(p) && !has_seqused(p) &&
           p->layout == SHAOBO_FA3_LAYOUT_BHSD;
}

int host_shard_count(const ShaoboFa3Params* p) {
    // about one shard per 8 MB of PCIe traffic, at most 8, at most one per (batch, KV head): every copy
    // costs about 5 us on the copy engine besides its bytes, so small problems want few, large copies
    // (measured on 16.8 MB: one shard 388 us, two 365 us, four 465 us)
    const size_t elem = 2;
    const size_t total = (size_t(5) * p->num_heads_q + size_t(4) * p->num_heads_kv) * p->batch *
                         p->seqlen_q * p->head_dim_qk * elem;
    long long n = (long long)(total / (size_t(8) << 20));
    const long long units = (long long)p->batch * p->num_heads_kv;
    n = std::max<long long>(1, std::min<long long>(8, std::min(n, units)));
    return int(n);
}

size_t host_lane_workspace(const ShaoboFa3Params* p) {
    const int n = host_shard_count(p);
    size_t need = 0;
    for (int r = 0; r < n; ++r) {
        HostPiece pcs[3];
        const int cnt = host_pieces(p, r, n, pcs);
        for (int i = 0; i < cnt; ++i) {
            const ShaoboFa3Params s = piece_params(p, pcs[i]);
            const V2Workspace w = v2_workspace(&s);
            if (!w.valid) return 0;
            need = std::max(need, w.total_bytes);
        }
    }
    size_t out = 0;
    return round_up_256(need, &out) ? out : 0;
}

}  // namespace

namespace {
struct HostStaging {
    size_t q_bytes = 0, kv_bytes = 0, lse_bytes = 0, lane_ws = 0, total = 0;
};
HostStaging host_staging(const ShaoboFa3Params* p) {
    HostStaging h;
    if (!host_call_supported(p)) return h;
    h.q_bytes = size_t(p->batch) * p->num_heads_q * p->seqlen_q * p->head_dim_qk * 2;
    h.kv_bytes = size_t(p->batch) * p->num_heads_kv * p->seqlen_k * p->head_dim_qk * 2;
    size_t lse = size_t(p->batch) * p->num_heads_q * p->seqlen_q * sizeof(float);
    if (!round_up_256(lse, &h.lse_bytes)) return HostStaging{};
    h.lane_ws = host_lane_workspace(p);
    if (h.lane_ws == 0) return HostStaging{};
    h.total = 4 * h.q_bytes + 4 * h.kv_bytes + h.lse_bytes + kHostLanes * h.lane_ws;
    return h;
}
}  // namespace

// Extension (no counterpart in the reference): bytes of device memory shaobo_fa3_b200_bwd_v2_host
// needs in `staging` for these parameters (device copies of the nine tensors plus one workspace per
// stream); 0 when the parameters are not accepted.  Host only.
extern "C" size_t shaobo_fa3_b200_bwd_v2_host_staging_bytes(const ShaoboFa3Params* params) {
    return host_staging(params).total;
}

// Extension (no counterpart in the reference): shaobo_fa3_bwd_v2 for tensors in host memory (pinned
// for full speed), [B,H,S,D], fixed lengths.  Enqueues copies and kernels behind the caller's stream
// (params->reserved_ptr[7], NULL = default stream) and makes that stream wait for them; the host
// buffers may be read once that stream has been synchronised (or at once with sync_after_launch).
extern "C" int shaobo_fa3_b200_bwd_v2_host(const void* dout, const void* q, const void* k,
                                           const void* v, const void* out, const void* softmax_lse,
                                           void* dq, void* dk, void* dv, void* staging,
                                           size_t staging_bytes, const ShaoboFa3Params* params) {
    begin();
    const int validation = validate_v2(params);
    if (validation != SHAOBO_FA3_STATUS_SUCCESS) return validation;
    if (!host_call_supported(params)) return SHAOBO_FA3_STATUS_UNSUPPORTED;
    const HostStaging hs = host_staging(params);
    if (dout == nullptr || q == nullptr || k == nullptr || v == nullptr || out == nullptr ||
        softmax_lse == nullptr || dq == nullptr || dk == nullptr || dv == nullptr ||
        staging == nullptr || hs.total == 0 || staging_bytes < hs.total) {
        return SHAOBO_FA3_STATUS_INVALID_VALUE;
    }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 128 || !g_host_lanes.get(dev)) {
        return SHAOBO_FA3_STATUS_HIP_ERROR;
    }
    uint8_t* base = static_cast<uint8_t*>(staging);
    uint8_t* d_q = base;
    uint8_t* d_do = d_q + hs.q_bytes;
    uint8_t* d_out = d_do + hs.q_bytes;
    uint8_t* d_dq = d_out + hs.q_bytes;
    uint8_t* d_k = d_dq + hs.q_bytes;
    uint8_t* d_v = d_k + hs.kv_bytes;
    uint8_t* d_dk = d_v + hs.kv_bytes;
    uint8_t* d_dv = d_dk + hs.kv_bytes;
    uint8_t* d_lse = d_dv + hs.kv_bytes;
    uint8_t* d_ws = d_lse + hs.lse_bytes;

    // The fork and join events and the three lane streams are shared by every call on this device.
    // A stream wait refers to the event's latest record at the moment the wait is enqueued, so one
    // call's record -> wait pairs must not interleave with another call's: the whole enqueue (not the
    // GPU work) runs under a per-device lock.  Calls from several host threads then queue up on the
    // same lanes in lock order; each needs its own staging buffer.
    std::lock_guard<std::mutex> enqueue_lock(g_host_lanes.enqueue[dev]);
    cudaStream_t caller = stream_of(params);
    if (cudaEventRecord(g_host_lanes.fork[dev], caller) != cudaSuccess) return SHAOBO_FA3_STATUS_HIP_ERROR;
    const int group = params->num_heads_q / params->num_heads_kv;
    const size_t q_head = size_t(params->seqlen_q) * params->head_dim_qk * 2;   // bytes of one query head
    const size_t kv_head = size_t(params->seqlen_k) * params->head_dim_qk * 2;
    const size_t lse_head = size_t(params->seqlen_q) * sizeof(float);
    const int n = host_shard_count(params);
    bool used[kHostLanes] = {};
    auto enqueue_all = [&]() -> int {
        int piece_index = 0;
        for (int r = 0; r < n; ++r) {
            HostPiece pcs[3];
            const int cnt = host_pieces(params, r, n, pcs);
            for (int i = 0; i < cnt; ++i, ++piece_index) {
                const int lane = piece_index % kHostLanes;
                cudaStream_t st = g_host_lanes.stream[dev][lane];
                cudaStream_t ax = g_host_lanes.aux[dev][lane];
                if (!used[lane]) {
                    if (cudaStreamWaitEvent(st, g_host_lanes.fork[dev], 0) != cudaSuccess ||
                        cudaStreamWaitEvent(ax, g_host_lanes.fork[dev], 0) != cudaSuccess) {
                        return SHAOBO_FA3_STATUS_HIP_ERROR;
                    }
                    used[lane] = true;
                }
                const HostPiece& pc = pcs[i];
                const size_t qh = size_t(pc.batch_begin) * params->num_heads_q + size_t(pc.kv_head_begin) * group;
                const size_t kh = size_t(pc.batch_begin) * params->num_heads_kv + pc.kv_head_begin;
                const size_t q_n = size_t(pc.batch_count) * pc.kv_head_count * group;  // query heads in the piece
                const size_t k_n = size_t(pc.batch_count) * pc.kv_head_count;
                // the copies-in of a piece alternate between the lane's two streams: one stream hands the
                // copy engine its next copy only after the previous one has completed, two keep it fed
                int h2d_count = 0;
                auto h2d = [&](uint8_t* d, const void* h, size_t off, size_t bytes) {
                    cudaStream_t s_copy = (h2d_count++ & 1) ? ax : st;
                    return cudaMemcpyAsync(d + off, static_cast<const uint8_t*>(h) + off, bytes, cudaMemcpyHostToDevice, s_copy) == cudaSuccess;
                };
                auto d2h = [&](void* h, const uint8_t* d, size_t off, size_t bytes) {
                    return cudaMemcpyAsync(static_cast<uint8_t*>(h) + off, d + off, bytes, cudaMemcpyDeviceToHost, st) == cudaSuccess;
                };
                if (!h2d(d_q, q, qh * q_head, q_n * q_head) || !h2d(d_k, k, kh * kv_head, k_n * kv_head) ||
                    !h2d(d_v, v, kh * kv_head, k_n * kv_head) || !h2d(d_do, dout, qh * q_head, q_n * q_head) ||
                    !h2d(d_out, out, qh * q_head, q_n * q_head) || !h2d(d_lse, softmax_lse, qh * lse_head, q_n * lse_head) ||
                    cudaEventRecord(g_host_lanes.aux_done[dev][lane], ax) != cudaSuccess ||
                    cudaStreamWaitEvent(st, g_host_lanes.aux_done[dev][lane], 0) != cudaSuccess) {
                    return SHAOBO_FA3_STATUS_HIP_ERROR;
                }
                ShaoboFa3Params s = piece_params(params, pc);
                s.workspace = d_ws + size_t(lane) * hs.lane_ws;
                s.workspace_bytes = hs.lane_ws;
                s.reserved_ptr[SHAOBO_FA3_RESERVED_PTR_STREAM] = st;
                const int status = shaobo_fa3_bwd_v2(d_do + qh * q_head, d_q + qh * q_head, d_k + kh * kv_head,
                                                     d_v + kh * kv_head, d_out + qh * q_head, d_lse + qh * lse_head,
                                                     d_dq + qh * q_head, d_dk + kh * kv_head, d_dv + kh * kv_head,
                                                     nullptr, &s);
                if (status != SHAOBO_FA3_STATUS_SUCCESS) return status;
                if (!d2h(dq, d_dq, qh * q_head, q_n * q_head) || !d2h(dk, d_dk, kh * kv_head, k_n * kv_head) ||
                    !d2h(dv, d_dv, kh * kv_head, k_n * kv_head)) {
                    return SHAOBO_FA3_STATUS_HIP_ERROR;
                }
            }
        }
        return SHAOBO_FA3_STATUS_SUCCESS;
    };
    int status = enqueue_all();
    // Whatever happened above, the caller's stream waits for everything that did get enqueued on the
    // lanes: after an error return no copy into the caller's host buffers is left running unordered.
    for (int lane = 0; lane < kHostLanes; ++lane) {
        if (!used[lane]) continue;
        // (the second stream of the lane is joined into the first once more: after an error it may not have been)
        if (cudaEventRecord(g_host_lanes.aux_done[dev][lane], g_host_lanes.aux[dev][lane]) != cudaSuccess ||
            cudaStreamWaitEvent(g_host_lanes.stream[dev][lane], g_host_lanes.aux_done[dev][lane], 0) != cudaSuccess ||
            cudaEventRecord(g_host_lanes.join[dev][lane], g_host_lanes.stream[dev][lane]) != cudaSuccess ||
            cudaStreamWaitEvent(caller, g_host_lanes.join[dev][lane], 0) != cudaSuccess) {
            if (status == SHAOBO_FA3_STATUS_SUCCESS) status = SHAOBO_FA3_STATUS_HIP_ERROR;
        }
    }
    if (status != SHAOBO_FA3_STATUS_SUCCESS) {
        (void)cudaGetLastError();
        return status;
    }
    return finish(params, params->sync_after_launch != 0);
}
