// Host-only half of the C ABI: parameter initialisation, capability report,
// validation, workspace sizing and status strings.  This translation unit has
// no CUDA dependency, so the contract tests can exercise it on a machine
// without a GPU.  Behaviour follows reference src/shaobo_fa3_bwd_api.cpp
// (validation order and status codes, lines 70-120; workspace carving, lines
// 122-156), widened to BF16 and head_dim 64.
#include <cmath>
#include <cstring>
#include <map>
#include <mutex>
#include <queue>
#include <tuple>
#include <vector>
#include <limits>

#include "fa3_host.h"
#include "shaobo_fa3_components.h"

namespace fa3b200 {

bool mul_ok(size_t a, size_t b, size_t* out) {
    if (a != 0 && b > std::numeric_limits<size_t>::max() / a) return false;
    *out = a * b;
    return true;
}

bool add_ok(size_t a, size_t b, size_t* out) {
    if (b > std::numeric_limits<size_t>::max() - a) return false;
    *out = a + b;
    return true;
}

bool round_up_256(size_t bytes, size_t* out) {
    size_t padded = 0;
    if (!add_ok(bytes, kWorkspaceAlignment - 1, &padded)) return false;
    *out = padded & ~(kWorkspaceAlignment - 1);
    return true;
}

namespace {

bool is_flag(int32_t v) { return v == 0 || v == 1; }

bool finite_nonneg(float v) { return std::isfinite(v) && v >= 0.0f; }

// The reference only takes windows that cover every key a causal / full mask would cover
// (src/shaobo_fa3_bwd_api.cpp:53-68); here any window is accepted, negative = unbounded, and
// make_band() applies the same normalisation (causal forces right = 0).
bool lengths_in_range(const ShaoboFa3Params* p) {
    return p->seqlen_q < kUnbounded && p->seqlen_k < kUnbounded;
}

// Packed sequences need both offset arrays, the two maxima and the two totals.
bool varlen_fields_ok(const ShaoboFa3Params* p) {
    if (p->cu_seqlens_q == nullptr || p->cu_seqlens_k == nullptr) return false;
    if (p->max_seqlen_q <= 0 || p->max_seqlen_k <= 0 || p->total_q <= 0 || p->total_k <= 0) return false;
    if (p->max_seqlen_q >= kUnbounded || p->max_seqlen_k >= kUnbounded) return false;
    if (p->total_q >= (int64_t(1) << 31) || p->total_k >= (int64_t(1) << 31)) return false;
    return p->max_seqlen_q <= p->total_q && p->max_seqlen_k <= p->total_k;
}

bool lengths_are_fixed(const ShaoboFa3Params* p) {
    if (p->cu_seqlens_q || p->cu_seqlens_k) return false;
    if (p->max_seqlen_q != 0 && p->max_seqlen_q != p->seqlen_q) return false;
    if (p->max_seqlen_k != 0 && p->max_seqlen_k != p->seqlen_k) return false;
    const int64_t tq = int64_t(p->batch) * p->seqlen_q;
    const int64_t tk = int64_t(p->batch) * p->seqlen_k;
    if (p->total_q != 0 && p->total_q != tq) return false;
    if (p->total_k != 0 && p->total_k != tk) return false;
    return true;
}

// Query rows over all heads: B*Hq*Sq, or Hq*total_q for packed sequences.
size_t row_count(const ShaoboFa3Params* p, bool* ok) {
    size_t rows = is_varlen(p) ? size_t(p->total_q) : size_t(p->batch);
    *ok = mul_ok(rows, size_t(p->num_heads_q), &rows) &&
          (is_varlen(p) || mul_ok(rows, size_t(p->seqlen_q), &rows));
    return rows;
}

}  // namespace

int validate_v2(const ShaoboFa3Params* p) {
    // ---- malformed input: INVALID_VALUE -------------------------------------
    if (p == nullptr || p->struct_size < sizeof(ShaoboFa3Params)) {
        return SHAOBO_FA3_STATUS_INVALID_VALUE;
    }
    const bool dims_ok = p->batch > 0 && p->seqlen_q > 0 && p->seqlen_k > 0 &&
                         p->num_heads_q > 0 && p->num_heads_kv > 0 &&
                         p->num_heads_q % p->num_heads_kv == 0;
    const bool flags_ok = is_flag(p->causal) && is_flag(p->deterministic) &&
                          is_flag(p->sync_after_launch) && is_flag(p->softmax_scale_is_set);
    const bool scale_ok = p->softmax_scale_is_set == 0 || finite_nonneg(p->softmax_scale);
    const bool reals_ok = finite_nonneg(p->softcap) && finite_nonneg(p->dropout_p) &&
                          p->dropout_p < 1.0f;
    if (!(dims_ok && flags_ok && scale_ok && reals_ok)) {
        return SHAOBO_FA3_STATUS_INVALID_VALUE;
    }
    // ---- well-formed but outside the capability set: UNSUPPORTED ------------
    // (wider than the reference, which also turns away the [B,S,H,D] layout, seqlen_q != seqlen_k,
    // sequence lengths that are not multiples of 128 and sliding windows:
    // src/shaobo_fa3_bwd_api.cpp:109-118)
    const bool lengths_ok = is_varlen(p) ? varlen_fields_ok(p) : lengths_are_fixed(p);
    if (!lengths_ok || !dtype_supported(p->dtype) || !layout_supported(p->layout) ||
        !head_dim_supported(p->head_dim_qk) || p->head_dim_v != p->head_dim_qk ||
        p->dropout_p != 0.0f || p->sm_margin != 0 || !lengths_in_range(p)) {
        return SHAOBO_FA3_STATUS_UNSUPPORTED;
    }
    return SHAOBO_FA3_STATUS_SUCCESS;
}

bool fused_shape_ok(const ShaoboFa3Params* p) {
    return p != nullptr && p->batch > 0 && p->num_heads_q > 0 && p->num_heads_kv > 0 &&
           p->num_heads_q % p->num_heads_kv == 0 && p->seqlen_q > 0 && p->seqlen_k > 0 &&
           head_dim_supported(p->head_dim_qk) && p->head_dim_v == p->head_dim_qk;
}

size_t dq_accum_bytes(const ShaoboFa3Params* p) {
    if (!fused_shape_ok(p)) return 0;
    bool ok = false;
    size_t n = row_count(p, &ok);
    size_t out = 0;
    if (!ok || !mul_ok(n, size_t(p->head_dim_qk), &n) || !mul_ok(n, sizeof(float), &n) ||
        !round_up_256(n, &out)) {
        return 0;
    }
    return out;
}

namespace {
// The plan is a pure function of these; a call asks for it several times (workspace size, launch,
// convert) and the search below simulates a schedule per candidate, so answers are remembered.
using SplitKey = std::tuple<int, int, int, int, int, long long, long long>;
std::mutex g_split_mu;
std::map<SplitKey, SplitPlan> g_split_cache;
}  // namespace

static SplitPlan search_split_plan(const ShaoboFa3Params* p, int tiles, const Band& band, long long heads, long long group);

SplitPlan split_plan(const ShaoboFa3Params* p) {
    // (per-sequence lengths of packed sequences, and used lengths, are not known on the host: no
    // splitting there)
    if (!fused_shape_ok(p) || p->deterministic != 0 || is_varlen(p) || has_seqused(p)) return SplitPlan{};
    const int tiles = tiles_of(p->seqlen_k);
    const Band band = band_of(p);
    const long long heads = (long long)p->batch * p->num_heads_kv;
    if (tiles * heads >= kSplitSmCount) return SplitPlan{};
    const long long group = p->num_heads_q / p->num_heads_kv;
    const SplitKey key{band.seqlen_q, band.seqlen_k, band.left, band.right, band.off, heads, group};
    {
        std::lock_guard<std::mutex> lock(g_split_mu);
        auto it = g_split_cache.find(key);
        if (it != g_split_cache.end()) return it->second;
    }
    const SplitPlan plan = search_split_plan(p, tiles, band, heads, group);
    std::lock_guard<std::mutex> lock(g_split_mu);
    if (g_split_cache.size() > 4096) g_split_cache.clear();
    g_split_cache[key] = plan;
    return plan;
}

static SplitPlan search_split_plan(const ShaoboFa3Params* p, int tiles, const Band& band, long long heads, long long group) {
    (void)p;
    SplitPlan plan;
    long long longest = 0;  // steps of the heaviest key tile
    for (int kt = 0; kt < tiles; ++kt) {
        const long long steps = group * q_tiles_of_k_tile(kt, band);
        if (steps > longest) longest = steps;
    }
    // Modelled makespan of chunk size `chunk`, in half steps: CTAs longest first onto 148 SMs as they
    // free up; a CTA of n steps costs 7 + 2n (measured on B200: set-up, first loads, the first step's
    // pipeline fill and the epilogue together cost about 3.5 steady-state steps).  CTA sizes are few (at most `chunk` different ones), so
    // the list is walked by size class.
    long long best_cost = -1;
    for (long long chunk = 1; chunk <= longest; ++chunk) {
        std::vector<long long> count(size_t(chunk) + 1, 0);  // CTAs of every size, all heads
        long long per_head = 0;
        for (int kt = 0; kt < tiles; ++kt) {
            const long long steps = group * q_tiles_of_k_tile(kt, band);
            if (steps == 0) continue;
            const long long full = steps / chunk, rest = steps % chunk;
            count[size_t(chunk)] += full * heads;
            if (rest != 0) count[size_t(rest)] += heads;
            per_head += full + (rest != 0 ? 1 : 0);
        }
        if (per_head * heads > kMaxSplitCtas) continue;
        std::priority_queue<long long, std::vector<long long>, std::greater<long long>> free_at;
        for (int i = 0; i < kSplitSmCount; ++i) free_at.push(0);
        long long makespan = 0;
        for (long long n = chunk; n >= 1; --n) {
            for (long long i = 0; i < count[size_t(n)]; ++i) {
                const long long end = free_at.top() + 7 + 2 * n;
                free_at.pop();
                free_at.push(end);
                if (end > makespan) makespan = end;
            }
        }
        if (best_cost < 0 || makespan < best_cost) {
            best_cost = makespan;
            plan.chunk_steps = int(chunk);
            plan.chunks_per_head = int(per_head);
        } else if (makespan == best_cost) {
            plan.chunk_steps = int(chunk);      // same makespan with fewer, longer CTAs: fewer partial sums
            plan.chunks_per_head = int(per_head);
        }
    }
    if (plan.chunk_steps >= longest) return SplitPlan{};  // a chunk as long as the heaviest tile is no split at all
    return plan;
}

size_t dkv_accum_bytes(const ShaoboFa3Params* p) {
    const SplitPlan plan = split_plan(p);
    if (plan.chunk_steps == 0) return 0;
    // one dK slab and one dV slab of [128 rows][D] per CTA: fp16 for fp16 inputs, fp32 for bf16 inputs
    const size_t elem = p->dtype == SHAOBO_FA3_DTYPE_FP16 ? 2 : sizeof(float);
    size_t n = size_t(p->batch), out = 0;
    if (!mul_ok(n, size_t(p->num_heads_kv), &n) || !mul_ok(n, size_t(plan.chunks_per_head), &n) ||
        !mul_ok(n, size_t(kSequenceAlignment), &n) || !mul_ok(n, size_t(p->head_dim_qk), &n) ||
        !mul_ok(n, 2 * elem, &n) || !round_up_256(n, &out)) {
        return 0;
    }
    return out;
}

V2Workspace v2_workspace(const ShaoboFa3Params* p) {
    V2Workspace w;
    if (validate_v2(p) != SHAOBO_FA3_STATUS_SUCCESS) return w;
    w.dq_accum_bytes = dq_accum_bytes(p);
    if (w.dq_accum_bytes == 0) return w;
    w.dkv_accum_bytes = dkv_accum_bytes(p);
    if (!add_ok(w.dq_accum_bytes, w.dkv_accum_bytes, &w.delta_offset)) return V2Workspace{};
    bool ok = false;
    const size_t rows = row_count(p, &ok);
    size_t delta_bytes = 0, sidecar_bytes = 0, end_of_delta = 0;
    if (!ok || !mul_ok(rows, sizeof(float), &delta_bytes) ||
        !mul_ok(delta_bytes, size_t(kSidecarFields), &sidecar_bytes) ||
        !add_ok(w.delta_offset, delta_bytes, &end_of_delta) ||
        !round_up_256(end_of_delta, &w.sidecar_offset) ||
        !add_ok(w.sidecar_offset, sidecar_bytes, &w.total_bytes)) {
        return V2Workspace{};
    }
    w.valid = true;
    return w;
}

size_t naive_reference_bytes(const ShaoboFa3Params* p) {
    if (p == nullptr || p->batch <= 0 || p->seqlen_q <= 0 || p->seqlen_k != p->seqlen_q ||
        p->num_heads_q <= 0 || p->num_heads_kv != p->num_heads_q ||
        !head_dim_supported(p->head_dim_qk) || p->head_dim_v != p->head_dim_qk ||
        !dtype_supported(p->dtype) || p->layout != SHAOBO_FA3_LAYOUT_BHSD ||
        p->dropout_p != 0.0f) {
        return 0;
    }
    bool ok = false;
    const size_t rows = row_count(p, &ok);
    size_t pairs = 0, total = 0, tail = 0;
    if (!ok || !mul_ok(rows, size_t(p->seqlen_k), &pairs) || !mul_ok(pairs, 2, &total) ||
        !mul_ok(rows, 3, &tail) || !add_ok(total, tail, &total) ||
        !mul_ok(total, sizeof(float), &total)) {
        return 0;
    }
    return total;
}

}  // namespace fa3b200

using namespace fa3b200;

extern "C" void shaobo_fa3_params_init(ShaoboFa3Params* params) {
    if (params == nullptr) return;
    std::memset(params, 0, sizeof(ShaoboFa3Params));
    params->struct_size = uint32_t(sizeof(ShaoboFa3Params));
    params->window_left = -1;
    params->window_right = -1;
    params->dtype = SHAOBO_FA3_DTYPE_FP16;
    params->layout = SHAOBO_FA3_LAYOUT_BHSD;
    params->softmax_aux_mode = SHAOBO_FA3_SOFTMAX_AUX_LSE;
}

extern "C" int shaobo_fa3_bwd_get_capabilities(ShaoboFa3BwdCapabilities* caps) {
    if (caps == nullptr || caps->struct_size < sizeof(ShaoboFa3BwdCapabilities)) {
        return SHAOBO_FA3_STATUS_INVALID_VALUE;
    }
    caps->api_version = SHAOBO_FA3_API_VERSION;
    // The reference's set (src/shaobo_fa3_bwd_api.cpp:180-187) plus BF16, the [B,S,H,D] layout
    // and sliding windows.
    caps->feature_mask = SHAOBO_FA3_BWD_FEATURE_FIXED_LENGTH | SHAOBO_FA3_BWD_FEATURE_FP16 |
                         SHAOBO_FA3_BWD_FEATURE_BF16 | SHAOBO_FA3_BWD_FEATURE_CAUSAL |
                         SHAOBO_FA3_BWD_FEATURE_GQA | SHAOBO_FA3_BWD_FEATURE_DETERMINISTIC |
                         SHAOBO_FA3_BWD_FEATURE_SOFTMAX_LSE | SHAOBO_FA3_BWD_FEATURE_BHSD |
                         SHAOBO_FA3_BWD_FEATURE_BSHD | SHAOBO_FA3_BWD_FEATURE_LOCAL_WINDOW |
                         SHAOBO_FA3_BWD_FEATURE_VARLEN | SHAOBO_FA3_BWD_FEATURE_SOFTCAP |
                         SHAOBO_FA3_BWD_FEATURE_FULL_ATTENTION;
    caps->min_head_dim = kMinHeadDim;
    caps->max_head_dim = kMaxHeadDim;
    caps->head_dim_alignment = kMinHeadDim;
    caps->sequence_alignment = 1;  // any length; tiles are 128 rows, the last one may be ragged
    return SHAOBO_FA3_STATUS_SUCCESS;
}

extern "C" int shaobo_fa3_bwd_v2_validate(const ShaoboFa3Params* params) {
    return validate_v2(params);
}

extern "C" size_t shaobo_fa3_bwd_v2_workspace_bytes(const ShaoboFa3Params* params) {
    const V2Workspace w = v2_workspace(params);
    return w.valid ? w.total_bytes : 0;
}

extern "C" size_t shaobo_fa3_bwd_fused5_workspace_bytes(const ShaoboFa3Params* params) {
    if (params == nullptr || !dtype_supported(params->dtype) || !layout_supported(params->layout)) {
        return 0;
    }
    // dQ accumulator, then the dK/dV accumulators of split tiles
    size_t total = 0;
    const size_t dq = dq_accum_bytes(params);
    if (dq == 0 || !add_ok(dq, dkv_accum_bytes(params), &total)) return 0;
    return total;
}

extern "C" size_t shaobo_fa3_bwd_dkv_workspace_bytes(const ShaoboFa3Params* params) {
    if (params == nullptr || params->dkv_path != SHAOBO_FA3_DKV_PATH_REFERENCE) return 0;
    return naive_reference_bytes(params);
}

extern "C" size_t shaobo_fa3_bwd_dq_workspace_bytes(const ShaoboFa3Params* params) {
    if (params == nullptr || params->dq_path != SHAOBO_FA3_DQ_PATH_REFERENCE) return 0;
    return naive_reference_bytes(params);
}

extern "C" size_t shaobo_fa3_bwd_workspace_bytes(const ShaoboFa3Params* params) {
    return shaobo_fa3_bwd_dkv_workspace_bytes(params);
}

extern "C" const char* shaobo_fa3_status_string(int status) {
    static const char* const names[] = {"success", "invalid_value", "unsupported",
                                        "not_implemented", "hip_error"};
    if (status < 0 || status > SHAOBO_FA3_STATUS_HIP_ERROR) return "unknown";
    return names[status];
}
