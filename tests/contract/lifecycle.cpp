// Compiled lifecycle harness: a plain C++ caller of the C ABI, the way the reference's own
// integration program is one (reference src/full_bwd_correctness.cpp:175-535).  It reads a golden
// directory (the raw-file set of reference scripts/generate_full_bwd_golden.py:113-132 plus
// lse.f32), allocates with the CUDA runtime, runs
//   (1) shaobo_fa3_bwd_v2                                  (fused path),
//   (2) shaobo_fa3_bwd_v2 with deterministic = 1           (atomic-free path),
//   (3) shaobo_fa3_bwd_dot_do_o -> shaobo_fa3_bwd_dkv -> shaobo_fa3_bwd_dq, called exactly as
//       reference src/full_bwd_correctness.cpp:375-392 calls them (row maximum / row sum in
//       softmax_aux0/1, sidecar in reserved_ptr[3], delta in reserved_ptr[0]),
//   (4) shaobo_fa3_bwd_dq once more with reserved_ptr[3] = NULL, the way the reference's standalone
//       dQ program calls it (reference src/dq_kernel.cpp:1651-1871),
// compares every output with the golden using the five metrics of reference
// src/full_bwd_correctness.cpp:104-137, and prints one key=value line per path and a final
// "lifecycle pass=<0|1>".  Exit code 0 iff every path passed.
//
//   g++ -std=c++17 -I include tests/contract/lifecycle.cpp flash_attention3_b200/libfa3bwd_b200.so \
//       -I/usr/local/cuda/include -L/usr/local/cuda/lib64 -lcudart -o lifecycle
//   ./lifecycle <golden dir> <batch> <heads_q> <heads_kv> <seqlen> <head_dim> <causal>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <string>
#include <vector>

#include "shaobo_fa3_api.h"
#include "shaobo_fa3_components.h"

namespace {

struct Metrics {
    double max_abs = 0, mean_abs = 0, rmse = 0, rel_l2 = 0, cosine_error = 0;
    long nonfinite = 0;
};

Metrics compare(const std::vector<float>& got, const std::vector<float>& want) {
    Metrics m;
    double abs_sum = 0, diff_sq = 0, got_sq = 0, want_sq = 0, dot = 0;
    for (size_t i = 0; i < got.size(); ++i) {
        const double g = got[i], w = want[i];
        if (!std::isfinite(g) || !std::isfinite(w)) {
            ++m.nonfinite;
            continue;
        }
        const double d = std::fabs(g - w);
        if (d > m.max_abs) m.max_abs = d;
        abs_sum += d;
        diff_sq += d * d;
        got_sq += g * g;
        want_sq += w * w;
        dot += g * w;
    }
    const double n = got.empty() ? 1.0 : double(got.size());
    m.mean_abs = abs_sum / n;
    m.rmse = std::sqrt(diff_sq / n);
    m.rel_l2 = std::sqrt(diff_sq / (want_sq > 1e-30 ? want_sq : 1e-30));
    const double norms = std::sqrt(got_sq * want_sq);
    m.cosine_error = norms > 1e-30 ? 1.0 - dot / norms : 0.0;
    return m;
}

template <typename T>
bool read_raw(const std::string& path, size_t count, std::vector<T>* out) {
    std::ifstream f(path, std::ios::binary | std::ios::ate);
    if (!f || size_t(f.tellg()) != count * sizeof(T)) {
        std::fprintf(stderr, "cannot read %zu elements from %s\n", count, path.c_str());
        return false;
    }
    out->resize(count);
    f.seekg(0);
    return bool(f.read(reinterpret_cast<char*>(out->data()), std::streamsize(count * sizeof(T))));
}

struct Device {
    std::vector<void*> owned;
    ~Device() {
        for (void* p : owned) cudaFree(p);
    }
    void* alloc(size_t bytes) {
        void* p = nullptr;
        if (cudaMalloc(&p, bytes ? bytes : 1) != cudaSuccess) {
            std::fprintf(stderr, "cudaMalloc(%zu) failed\n", bytes);
            std::exit(2);
        }
        owned.push_back(p);
        return p;
    }
    template <typename T>
    T* upload(const std::vector<T>& host) {
        T* p = static_cast<T*>(alloc(host.size() * sizeof(T)));
        if (cudaMemcpy(p, host.data(), host.size() * sizeof(T), cudaMemcpyHostToDevice) != cudaSuccess) std::exit(2);
        return p;
    }
};

std::vector<float> download_f32(const void* dev, size_t count) {
    std::vector<float> out(count);
    if (cudaMemcpy(out.data(), dev, count * sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess) std::exit(2);
    return out;
}

std::vector<float> download_f16(const void* dev, size_t count) {
    std::vector<__half> tmp(count);
    if (cudaMemcpy(tmp.data(), dev, count * sizeof(__half), cudaMemcpyDeviceToHost) != cudaSuccess) std::exit(2);
    std::vector<float> out(count);
    for (size_t i = 0; i < count; ++i) out[i] = __half2float(tmp[i]);
    return out;
}

// Gates of the backward: relative L2 <= 5e-3 and max-abs <= 2e-2 for the gradients, 1e-3 relative
// for delta; no non-finite element anywhere.
bool report(const char* path, const char* status, const char* name, const Metrics& m, bool is_delta,
            bool* all) {
    const bool ok = m.nonfinite == 0 && (is_delta ? m.rel_l2 <= 1e-3 : (m.rel_l2 <= 5e-3 && m.max_abs <= 2e-2));
    std::printf(" %s_max_abs=%.3e %s_mean_abs=%.3e %s_rmse=%.3e %s_rel_l2=%.3e %s_cosine_error=%.3e %s_nonfinite=%ld",
                name, m.max_abs, name, m.mean_abs, name, m.rmse, name, m.rel_l2, name, m.cosine_error, name,
                m.nonfinite);
    (void)path;
    (void)status;
    if (!ok) *all = false;
    return ok;
}

}  // namespace

int main(int argc, char** argv) {
    if (argc != 8) {
        std::fprintf(stderr, "usage: %s <golden dir> <batch> <heads_q> <heads_kv> <seqlen> <head_dim> <causal>\n", argv[0]);
        return 2;
    }
    const std::string dir = argv[1];
    const int B = std::atoi(argv[2]), Hq = std::atoi(argv[3]), Hkv = std::atoi(argv[4]);
    const int S = std::atoi(argv[5]), D = std::atoi(argv[6]), causal = std::atoi(argv[7]);
    const size_t nq = size_t(B) * Hq * S * D, nkv = size_t(B) * Hkv * S * D, rows = size_t(B) * Hq * S;

    std::vector<__half> q, k, v, o, dout;
    std::vector<float> smax, ssum, lse, delta_ref, sidecar_ref, dq_ref, dk_ref, dv_ref;
    if (!read_raw(dir + "/q.f16", nq, &q) || !read_raw(dir + "/k.f16", nkv, &k) ||
        !read_raw(dir + "/v.f16", nkv, &v) || !read_raw(dir + "/o.f16", nq, &o) ||
        !read_raw(dir + "/dout.f16", nq, &dout) || !read_raw(dir + "/scores_max.f32", rows, &smax) ||
        !read_raw(dir + "/scores_sum.f32", rows, &ssum) || !read_raw(dir + "/lse.f32", rows, &lse) ||
        !read_raw(dir + "/delta.f32", rows, &delta_ref) ||
        !read_raw(dir + "/packed_sidecar.f32", rows * 3, &sidecar_ref) ||
        !read_raw(dir + "/dq.f32", nq, &dq_ref) || !read_raw(dir + "/dk.f32", nkv, &dk_ref) ||
        !read_raw(dir + "/dv.f32", nkv, &dv_ref)) {
        return 2;
    }

    Device dev;
    const __half* q_d = dev.upload(q);
    const __half* k_d = dev.upload(k);
    const __half* v_d = dev.upload(v);
    const __half* o_d = dev.upload(o);
    const __half* dout_d = dev.upload(dout);
    const float* smax_d = dev.upload(smax);
    const float* ssum_d = dev.upload(ssum);
    const float* lse_d = dev.upload(lse);

    ShaoboFa3Params base;
    shaobo_fa3_params_init(&base);
    base.batch = B;
    base.seqlen_q = base.seqlen_k = S;
    base.num_heads_q = Hq;
    base.num_heads_kv = Hkv;
    base.head_dim_qk = base.head_dim_v = D;
    base.causal = causal;
    base.dtype = SHAOBO_FA3_DTYPE_FP16;
    base.softmax_scale = 1.0f / std::sqrt(float(D));
    base.softmax_scale_is_set = 1;
    base.sync_after_launch = 1;

    bool all = true;

    // ---- (1), (2): the v2 entry, fused and deterministic
    for (int deterministic = 0; deterministic < 2; ++deterministic) {
        ShaoboFa3Params p = base;
        p.deterministic = deterministic;
        const char* name = deterministic ? "v2_deterministic" : "v2_fused5";
        int status = shaobo_fa3_bwd_v2_validate(&p);
        void *dq_d = dev.alloc(nq * 2), *dk_d = dev.alloc(nkv * 2), *dv_d = dev.alloc(nkv * 2);
        float* delta_d = static_cast<float*>(dev.alloc(rows * 4));
        cudaMemset(dq_d, 0xFF, nq * 2);  // NaN patterns: an element the library forgets stays non-finite
        cudaMemset(dk_d, 0xFF, nkv * 2);
        cudaMemset(dv_d, 0xFF, nkv * 2);
        cudaMemset(delta_d, 0xFF, rows * 4);
        if (status == SHAOBO_FA3_STATUS_SUCCESS) {
            p.workspace_bytes = shaobo_fa3_bwd_v2_workspace_bytes(&p);
            p.workspace = dev.alloc(p.workspace_bytes);
            cudaMemset(p.workspace, 0xFF, p.workspace_bytes);
            status = p.workspace_bytes == 0 ? SHAOBO_FA3_STATUS_INVALID_VALUE
                                            : shaobo_fa3_bwd_v2(dout_d, q_d, k_d, v_d, o_d, lse_d, dq_d, dk_d, dv_d, delta_d, &p);
        }
        const bool sync_ok = cudaDeviceSynchronize() == cudaSuccess;
        std::printf("lifecycle path=%s status=%s", name, shaobo_fa3_status_string(status));
        bool ok = status == SHAOBO_FA3_STATUS_SUCCESS && sync_ok;
        if (ok) {
            ok &= report(name, "", "delta", compare(download_f32(delta_d, rows), delta_ref), true, &all);
            ok &= report(name, "", "dq", compare(download_f16(dq_d, nq), dq_ref), false, &all);
            ok &= report(name, "", "dk", compare(download_f16(dk_d, nkv), dk_ref), false, &all);
            ok &= report(name, "", "dv", compare(download_f16(dv_d, nkv), dv_ref), false, &all);
        }
        if (!ok) all = false;
        std::printf(" pass=%d\n", ok ? 1 : 0);
    }

    // ---- (3): the seven-GEMM chain, called as the reference's harness calls it
    {
        ShaoboFa3Params p = base;
        p.softmax_aux_mode = SHAOBO_FA3_SOFTMAX_AUX_SMAX_SSUM;
        p.dkv_path = SHAOBO_FA3_DKV_PATH_CANONICAL;
        p.dq_path = SHAOBO_FA3_DQ_PATH_CANONICAL;
        float* delta_d = static_cast<float*>(dev.alloc(rows * 4));
        float* sidecar_d = static_cast<float*>(dev.alloc(rows * 12));
        float* dq_d = static_cast<float*>(dev.alloc(nq * 4));
        float* dk_d = static_cast<float*>(dev.alloc(nkv * 4));
        float* dv_d = static_cast<float*>(dev.alloc(nkv * 4));
        cudaMemset(dq_d, 0xFF, nq * 4);
        cudaMemset(dk_d, 0xFF, nkv * 4);
        cudaMemset(dv_d, 0xFF, nkv * 4);
        const int dot_status = shaobo_fa3_bwd_dot_do_o(dout_d, o_d, smax_d, ssum_d, delta_d, sidecar_d, &p);
        p.reserved_ptr[SHAOBO_FA3_RESERVED_PTR_SIDECAR] = sidecar_d;
        const int dkv_status = dot_status == SHAOBO_FA3_STATUS_SUCCESS
                                   ? shaobo_fa3_bwd_dkv(dout_d, q_d, k_d, v_d, o_d, smax_d, ssum_d, nullptr, dk_d, dv_d, &p)
                                   : dot_status;
        p.reserved_ptr[SHAOBO_FA3_RESERVED_PTR_DELTA] = delta_d;
        const int dq_status = dkv_status == SHAOBO_FA3_STATUS_SUCCESS
                                  ? shaobo_fa3_bwd_dq(dout_d, q_d, k_d, v_d, o_d, smax_d, ssum_d, dq_d, nullptr, nullptr, &p)
                                  : dkv_status;
        const bool sync_ok = cudaDeviceSynchronize() == cudaSuccess;
        std::printf("lifecycle path=seven_gemm dot_status=%s dkv_status=%s dq_status=%s",
                    shaobo_fa3_status_string(dot_status), shaobo_fa3_status_string(dkv_status),
                    shaobo_fa3_status_string(dq_status));
        bool ok = dq_status == SHAOBO_FA3_STATUS_SUCCESS && sync_ok;
        if (ok) {
            ok &= report("", "", "delta", compare(download_f32(delta_d, rows), delta_ref), true, &all);
            ok &= report("", "", "sidecar", compare(download_f32(sidecar_d, rows * 3), sidecar_ref), true, &all);
            ok &= report("", "", "dq", compare(download_f32(dq_d, nq), dq_ref), false, &all);
            ok &= report("", "", "dk", compare(download_f32(dk_d, nkv), dk_ref), false, &all);
            ok &= report("", "", "dv", compare(download_f32(dv_d, nkv), dv_ref), false, &all);
        }
        if (!ok) all = false;
        std::printf(" pass=%d\n", ok ? 1 : 0);

        // ---- (4): the dQ half alone, statistics as three arrays only (no sidecar), and once in
        // LSE mode (log-sum-exp in softmax_aux0, softmax_aux1 = NULL)
        for (int lse_mode = 0; lse_mode < 2; ++lse_mode) {
            ShaoboFa3Params pq = p;
            pq.reserved_ptr[SHAOBO_FA3_RESERVED_PTR_SIDECAR] = nullptr;
            pq.softmax_aux_mode = lse_mode ? SHAOBO_FA3_SOFTMAX_AUX_LSE : SHAOBO_FA3_SOFTMAX_AUX_SMAX_SSUM;
            cudaMemset(dq_d, 0xFF, nq * 4);
            const int st = lse_mode ? shaobo_fa3_bwd_dq(dout_d, q_d, k_d, v_d, o_d, lse_d, nullptr, dq_d, nullptr, nullptr, &pq)
                                    : shaobo_fa3_bwd_dq(dout_d, q_d, k_d, v_d, o_d, smax_d, ssum_d, dq_d, nullptr, nullptr, &pq);
            const bool synced = cudaDeviceSynchronize() == cudaSuccess;
            std::printf("lifecycle path=%s status=%s", lse_mode ? "dq_alone_lse" : "dq_alone_smax_ssum",
                        shaobo_fa3_status_string(st));
            bool okq = st == SHAOBO_FA3_STATUS_SUCCESS && synced;
            if (okq) okq &= report("", "", "dq", compare(download_f32(dq_d, nq), dq_ref), false, &all);
            if (!okq) all = false;
            std::printf(" pass=%d\n", okq ? 1 : 0);
        }
        // neither form complete: no sidecar, no delta
        ShaoboFa3Params bad = p;
        bad.reserved_ptr[SHAOBO_FA3_RESERVED_PTR_SIDECAR] = nullptr;
        bad.reserved_ptr[SHAOBO_FA3_RESERVED_PTR_DELTA] = nullptr;
        const int st = shaobo_fa3_bwd_dq(dout_d, q_d, k_d, v_d, o_d, smax_d, ssum_d, dq_d, nullptr, nullptr, &bad);
        const bool okb = st == SHAOBO_FA3_STATUS_INVALID_VALUE;
        std::printf("lifecycle path=dq_without_statistics status=%s pass=%d\n", shaobo_fa3_status_string(st), okb ? 1 : 0);
        if (!okb) all = false;
    }

    std::printf("lifecycle pass=%d\n", all ? 1 : 0);
    return all ? 0 : 1;
}
