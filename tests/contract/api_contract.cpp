// Host-only contract check of the C ABI, compiled as C++ against the public
// header and linked with the shared library.  The expectations are the ones of
// reference tests/fused_bwd_api_contract.cpp:34-119, with the two deliberate
// capability extensions of this library: BF16 and head_dim 64 validate, and a
// head_dim outside {64,128} is UNSUPPORTED.
#include <cstddef>
#include <cstdio>
#include <cstring>

#include "shaobo_fa3_api.h"
#include "shaobo_fa3_components.h"

static int failures = 0;

static void expect(const char* what, long long got, long long want) {
    if (got != want) {
        std::fprintf(stderr, "FAIL %s: got %lld want %lld\n", what, got, want);
        ++failures;
    }
}

static ShaoboFa3Params good() {
    ShaoboFa3Params p;
    shaobo_fa3_params_init(&p);
    p.batch = 1;
    p.seqlen_q = p.seqlen_k = 1024;
    p.num_heads_q = 4;
    p.num_heads_kv = 2;
    p.head_dim_qk = p.head_dim_v = 128;
    p.causal = 1;
    p.softmax_scale = 0.125f;
    p.softmax_scale_is_set = 1;
    return p;
}

int main() {
    // layout of the parameter block
    expect("sizeof(params)", (long long)sizeof(ShaoboFa3Params), 296);
    expect("offsetof(batch)", (long long)offsetof(ShaoboFa3Params, batch), 4);
    expect("offsetof(causal)", (long long)offsetof(ShaoboFa3Params, causal), 32);
    expect("offsetof(softmax_scale)", (long long)offsetof(ShaoboFa3Params, softmax_scale), 44);
    expect("offsetof(dtype)", (long long)offsetof(ShaoboFa3Params, dtype), 52);
    expect("offsetof(sync_after_launch)", (long long)offsetof(ShaoboFa3Params, sync_after_launch), 76);
    expect("offsetof(cu_seqlens_q)", (long long)offsetof(ShaoboFa3Params, cu_seqlens_q), 80);
    expect("offsetof(workspace)", (long long)offsetof(ShaoboFa3Params, workspace), 104);
    expect("offsetof(workspace_bytes)", (long long)offsetof(ShaoboFa3Params, workspace_bytes), 112);
    expect("offsetof(reserved_i32)", (long long)offsetof(ShaoboFa3Params, reserved_i32), 120);
    expect("offsetof(reserved_ptr)", (long long)offsetof(ShaoboFa3Params, reserved_ptr), 184);
    expect("offsetof(seqused_q)", (long long)offsetof(ShaoboFa3Params, seqused_q), 248);
    expect("offsetof(total_q)", (long long)offsetof(ShaoboFa3Params, total_q), 264);
    expect("offsetof(softcap)", (long long)offsetof(ShaoboFa3Params, softcap), 280);
    expect("offsetof(deterministic)", (long long)offsetof(ShaoboFa3Params, deterministic), 284);
    expect("offsetof(sm_margin)", (long long)offsetof(ShaoboFa3Params, sm_margin), 288);
    expect("offsetof(softmax_scale_is_set)", (long long)offsetof(ShaoboFa3Params, softmax_scale_is_set), 292);

    // params_init defaults
    ShaoboFa3Params init;
    std::memset(&init, 0xAB, sizeof(init));
    shaobo_fa3_params_init(&init);
    expect("init.struct_size", init.struct_size, sizeof(ShaoboFa3Params));
    expect("init.window_left", init.window_left, -1);
    expect("init.window_right", init.window_right, -1);
    expect("init.dtype", init.dtype, SHAOBO_FA3_DTYPE_FP16);
    expect("init.layout", init.layout, SHAOBO_FA3_LAYOUT_BHSD);
    expect("init.aux", init.softmax_aux_mode, SHAOBO_FA3_SOFTMAX_AUX_LSE);
    expect("init.batch", init.batch, 0);
    shaobo_fa3_params_init(nullptr);  // must not crash

    // capabilities
    ShaoboFa3BwdCapabilities caps;
    std::memset(&caps, 0, sizeof(caps));
    expect("caps without size", shaobo_fa3_bwd_get_capabilities(&caps), SHAOBO_FA3_STATUS_INVALID_VALUE);
    expect("caps null", shaobo_fa3_bwd_get_capabilities(nullptr), SHAOBO_FA3_STATUS_INVALID_VALUE);
    caps.struct_size = sizeof(caps);
    expect("caps", shaobo_fa3_bwd_get_capabilities(&caps), SHAOBO_FA3_STATUS_SUCCESS);
    const ShaoboFa3BwdFeatureMask required =
        SHAOBO_FA3_BWD_FEATURE_FIXED_LENGTH | SHAOBO_FA3_BWD_FEATURE_FP16 |
        SHAOBO_FA3_BWD_FEATURE_BF16 | SHAOBO_FA3_BWD_FEATURE_CAUSAL | SHAOBO_FA3_BWD_FEATURE_GQA |
        SHAOBO_FA3_BWD_FEATURE_DETERMINISTIC | SHAOBO_FA3_BWD_FEATURE_SOFTMAX_LSE |
        SHAOBO_FA3_BWD_FEATURE_BHSD | SHAOBO_FA3_BWD_FEATURE_FULL_ATTENTION;
    expect("caps.api_version", caps.api_version, SHAOBO_FA3_API_VERSION);
    expect("caps.required bits", (caps.feature_mask & required) == required, 1);
    expect("caps.softcap", (caps.feature_mask & SHAOBO_FA3_BWD_FEATURE_SOFTCAP) != 0, 1);
    expect("caps.varlen", (caps.feature_mask & SHAOBO_FA3_BWD_FEATURE_VARLEN) != 0, 1);
    expect("caps.bshd", (caps.feature_mask & SHAOBO_FA3_BWD_FEATURE_BSHD) != 0, 1);
    expect("caps.local window", (caps.feature_mask & SHAOBO_FA3_BWD_FEATURE_LOCAL_WINDOW) != 0, 1);
    // every feature bit the header defines is offered: nothing is set beyond them
    const ShaoboFa3BwdFeatureMask defined_bits =
        required | SHAOBO_FA3_BWD_FEATURE_SOFTCAP | SHAOBO_FA3_BWD_FEATURE_VARLEN |
        SHAOBO_FA3_BWD_FEATURE_BSHD | SHAOBO_FA3_BWD_FEATURE_LOCAL_WINDOW;
    expect("caps.no undefined bits", (caps.feature_mask & ~defined_bits) == 0, 1);
    expect("caps.min_head_dim", caps.min_head_dim, 64);
    expect("caps.max_head_dim", caps.max_head_dim, 128);
    expect("caps.head_dim_alignment", caps.head_dim_alignment, 64);
    expect("caps.sequence_alignment", caps.sequence_alignment, 1);

    // accepted configurations
    ShaoboFa3Params p = good();
    expect("gqa causal", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_SUCCESS);
    expect("workspace nonzero", shaobo_fa3_bwd_v2_workspace_bytes(&p) != 0, 1);
    p.deterministic = 1;
    expect("deterministic", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_SUCCESS);
    p = good(); p.causal = 0;
    expect("full attention", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_SUCCESS);
    p = good(); p.softmax_scale_is_set = 0; p.softmax_scale = 0.0f;
    expect("default scale", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_SUCCESS);
    p = good(); p.dtype = SHAOBO_FA3_DTYPE_BF16;
    expect("bf16 (extension)", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_SUCCESS);
    p = good(); p.head_dim_qk = p.head_dim_v = 64;
    expect("head_dim 64 (extension)", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_SUCCESS);
    p = good(); p.window_left = 1023; p.window_right = 5000;  // covers everything: still causal
    expect("window that covers all keys", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_SUCCESS);
    p = good(); p.max_seqlen_q = 1024; p.total_k = 1024;
    expect("redundant fixed-length fields", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_SUCCESS);

    // accepted here although the reference turns them away (src/shaobo_fa3_bwd_api.cpp:53-68,109-118)
    p = good(); p.window_left = 128;
    expect("local window", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_SUCCESS);
    p = good(); p.causal = 0; p.window_right = 0;
    expect("right window without causal", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_SUCCESS);
    p = good(); p.softcap = 1.0f;
    expect("softcap", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_SUCCESS);
    // unsupported configurations
    p = good(); p.dropout_p = 0.1f;
    expect("dropout", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_UNSUPPORTED);
    p = good(); p.dtype = SHAOBO_FA3_DTYPE_FP8;
    expect("fp8", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_UNSUPPORTED);
    // wider than the reference: [B,S,H,D], seqlen_q != seqlen_k and ragged lengths are accepted
    p = good(); p.layout = SHAOBO_FA3_LAYOUT_BSHD;
    expect("bshd", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_SUCCESS);
    p = good(); p.layout = 2;
    expect("unknown layout", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_UNSUPPORTED);
    p = good(); int32_t cu[2] = {0, 1024}; p.cu_seqlens_q = cu;
    expect("varlen", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_UNSUPPORTED);
    p = good(); p.sm_margin = 1;
    expect("sm_margin", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_UNSUPPORTED);
    p = good(); p.head_dim_qk = p.head_dim_v = 96;
    expect("head_dim 96", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_UNSUPPORTED);
    p = good(); p.head_dim_v = 64;
    expect("head_dim_v != head_dim_qk", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_UNSUPPORTED);
    p = good(); p.seqlen_k = 2048;
    expect("seqlen_q != seqlen_k", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_SUCCESS);
    p = good(); p.seqlen_q = p.seqlen_k = 1000;
    expect("seqlen % 128", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_SUCCESS);
    expect("ragged length has a workspace", (long long)shaobo_fa3_bwd_v2_workspace_bytes(&p) > 0, 1);
    p = good(); p.head_dim_qk = p.head_dim_v = 96;
    expect("unsupported -> zero workspace", (long long)shaobo_fa3_bwd_v2_workspace_bytes(&p), 0);

    // malformed input
    p = good(); p.softmax_scale = -1.0f;
    expect("negative scale", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_INVALID_VALUE);
    p = good(); p.struct_size = 0;
    expect("struct_size 0", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_INVALID_VALUE);
    p = good(); p.num_heads_kv = 3;
    expect("Hq % Hkv", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_INVALID_VALUE);
    p = good(); p.batch = 0;
    expect("batch 0", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_INVALID_VALUE);
    p = good(); p.causal = 2;
    expect("causal 2", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_INVALID_VALUE);
    p = good(); p.dropout_p = 1.0f;
    expect("dropout 1", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_INVALID_VALUE);
    // INVALID_VALUE wins over UNSUPPORTED
    p = good(); p.layout = SHAOBO_FA3_LAYOUT_BSHD; p.softmax_scale = -1.0f;
    expect("invalid before unsupported", shaobo_fa3_bwd_v2_validate(&p), SHAOBO_FA3_STATUS_INVALID_VALUE);
    expect("null params", shaobo_fa3_bwd_v2_validate(nullptr), SHAOBO_FA3_STATUS_INVALID_VALUE);

    // v2 refuses before any launch (no device needed for these returns)
    p = good();
    int dummy = 0;
    void* x = &dummy;
    expect("v2 null tensor", shaobo_fa3_bwd_v2(x, x, x, x, x, nullptr, x, x, x, nullptr, &p), SHAOBO_FA3_STATUS_INVALID_VALUE);
    expect("v2 no workspace", shaobo_fa3_bwd_v2(x, x, x, x, x, x, x, x, x, nullptr, &p), SHAOBO_FA3_STATUS_INVALID_VALUE);
    p.workspace = x; p.workspace_bytes = shaobo_fa3_bwd_v2_workspace_bytes(&p) - 1;
    expect("v2 short workspace", shaobo_fa3_bwd_v2(x, x, x, x, x, x, x, x, x, nullptr, &p), SHAOBO_FA3_STATUS_INVALID_VALUE);
    p = good(); p.dtype = SHAOBO_FA3_DTYPE_FP8;
    expect("v2 unsupported", shaobo_fa3_bwd_v2(x, x, x, x, x, x, x, x, x, nullptr, &p), SHAOBO_FA3_STATUS_UNSUPPORTED);
    p = good();
    expect("fused5 null", shaobo_fa3_bwd_fused5(x, x, x, x, nullptr, x, x, x, &p), SHAOBO_FA3_STATUS_INVALID_VALUE);
    expect("fused5 no workspace", shaobo_fa3_bwd_fused5(x, x, x, x, x, x, x, x, &p), SHAOBO_FA3_STATUS_INVALID_VALUE);
    expect("dot_do_o null", shaobo_fa3_bwd_dot_do_o(x, x, nullptr, nullptr, x, x, &p), SHAOBO_FA3_STATUS_INVALID_VALUE);
    p.head_dim_qk = 96;
    expect("dot_do_o unsupported", shaobo_fa3_bwd_dot_do_o(x, x, x, x, x, x, &p), SHAOBO_FA3_STATUS_UNSUPPORTED);

    // status strings
    const char* names[] = {"success", "invalid_value", "unsupported", "not_implemented", "hip_error"};
    for (int i = 0; i < 5; ++i) expect(names[i], std::strcmp(shaobo_fa3_status_string(i), names[i]), 0);
    expect("unknown", std::strcmp(shaobo_fa3_status_string(99), "unknown"), 0);
    expect("unknown negative", std::strcmp(shaobo_fa3_status_string(-1), "unknown"), 0);

    std::printf("api_contract pass=%d\n", failures == 0 ? 1 : 0);
    return failures == 0 ? 0 : 1;
}
