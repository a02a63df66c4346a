/*
 * Scalar C restatement of the attention-backward golden.  TEST INFRASTRUCTURE
 * ONLY: it is built into oracle/libgolden_scalar.so and called from tests/ as
 * an independent check of oracle/golden.py on small shapes.  The shipped
 * library never links or calls it.
 *
 * The loop structure follows the in-file CPU golden of the reference's fused
 * stage test (reference tests/fused_bwd_correctness.cpp:52-132): per query row,
 * scores -> running maximum -> exp2((s - max) * scale * log2e) -> row sum ->
 * probabilities -> O -> delta -> dS; then a second sweep accumulates dQ, dK
 * and dV.  Generalisations: batch / heads / GQA / any head_dim, and O may be
 * rounded to the storage dtype before delta as the reference's NumPy golden
 * does (reference scripts/generate_full_bwd_golden.py:175-178).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static float round_bf16(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return x; /* NaN */
    u = (u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u;
    memcpy(&x, &u, 4);
    return x;
}

static float round_fp16(float x) {
    _Float16 h = (_Float16)x;
    return (float)h;
}

static float round_storage(float x, int dtype) {
    if (dtype == 0) return round_fp16(x);
    if (dtype == 1) return round_bf16(x);
    return x;
}

/*
 * q, dout: [B,Hq,S,D]; k, v: [B,Hkv,S,D]; all fp32 arrays holding values that
 * are exact in the storage dtype.  dtype: 0 fp16, 1 bf16, -1 keep O in fp32.
 * Outputs (caller-allocated): out [B,Hq,S,D], lse [B,Hq,S] (natural log),
 * sidecar [B,Hq,S,3] = {max*scale*log2e, 1/sum, delta}, dq [B,Hq,S,D],
 * dk, dv [B,Hkv,S,D] (summed over the query heads of each KV head).
 * Returns 0, or 1 when scratch memory could not be allocated.
 */
int fa3_golden_scalar(const float* q, const float* k, const float* v, const float* dout,
                      int B, int Hq, int Hkv, int S, int D, int causal, float scale,
                      int dtype, float* out, float* lse, float* sidecar, float* dq,
                      float* dk, float* dv) {
    const float kLog2E = 1.44269504088896340736f;
    const float scale_log2 = scale * kLog2E;
    const int group = Hq / Hkv;
    float* p = (float*)malloc(sizeof(float) * (size_t)S * S);
    float* ds = (float*)malloc(sizeof(float) * (size_t)S * S);
    float* orow = (float*)malloc(sizeof(float) * (size_t)D);
    if (!p || !ds || !orow) {
        free(p); free(ds); free(orow);
        return 1;
    }
    memset(dq, 0, sizeof(float) * (size_t)B * Hq * S * D);
    memset(dk, 0, sizeof(float) * (size_t)B * Hkv * S * D);
    memset(dv, 0, sizeof(float) * (size_t)B * Hkv * S * D);

    for (int b = 0; b < B; ++b) {
        for (int h = 0; h < Hq; ++h) {
            const int kvh = h / group;
            const float* qh = q + ((size_t)(b * Hq + h) * S) * D;
            const float* doh = dout + ((size_t)(b * Hq + h) * S) * D;
            const float* kh = k + ((size_t)(b * Hkv + kvh) * S) * D;
            const float* vh = v + ((size_t)(b * Hkv + kvh) * S) * D;
            float* outh = out + ((size_t)(b * Hq + h) * S) * D;
            float* dqh = dq + ((size_t)(b * Hq + h) * S) * D;
            float* dkh = dk + ((size_t)(b * Hkv + kvh) * S) * D;
            float* dvh = dv + ((size_t)(b * Hkv + kvh) * S) * D;
            float* lseh = lse + (size_t)(b * Hq + h) * S;
            float* sideh = sidecar + (size_t)(b * Hq + h) * S * 3;

            memset(p, 0, sizeof(float) * (size_t)S * S);
            memset(ds, 0, sizeof(float) * (size_t)S * S);
            for (int qi = 0; qi < S; ++qi) {
                const int keys = causal ? qi + 1 : S;
                float row_max = -INFINITY;
                for (int ki = 0; ki < keys; ++ki) {
                    float s = 0.0f;
                    for (int d = 0; d < D; ++d) s += qh[qi * D + d] * kh[ki * D + d];
                    p[(size_t)qi * S + ki] = s;
                    if (s > row_max) row_max = s;
                }
                double row_sum = 0.0;
                for (int ki = 0; ki < keys; ++ki) {
                    float* e = &p[(size_t)qi * S + ki];
                    *e = exp2f((*e - row_max) * scale_log2);
                    row_sum += *e;
                }
                const float row_sum_f = (float)row_sum;
                const float inv_sum = 1.0f / row_sum_f;
                for (int d = 0; d < D; ++d) orow[d] = 0.0f;
                for (int ki = 0; ki < keys; ++ki) {
                    const float prob = p[(size_t)qi * S + ki] / row_sum_f;
                    p[(size_t)qi * S + ki] = prob;
                    for (int d = 0; d < D; ++d) orow[d] += prob * vh[ki * D + d];
                }
                float delta = 0.0f;
                for (int d = 0; d < D; ++d) {
                    const float o = round_storage(orow[d], dtype);
                    outh[qi * D + d] = o;
                    delta += doh[qi * D + d] * o;
                }
                lseh[qi] = row_max * scale + logf(row_sum_f);
                sideh[qi * 3 + 0] = row_max * scale_log2;
                sideh[qi * 3 + 1] = row_sum_f != 0.0f ? inv_sum : 0.0f;
                sideh[qi * 3 + 2] = delta;
                for (int ki = 0; ki < keys; ++ki) {
                    float dp = 0.0f;
                    for (int d = 0; d < D; ++d) dp += doh[qi * D + d] * vh[ki * D + d];
                    ds[(size_t)qi * S + ki] = p[(size_t)qi * S + ki] * (dp - delta) * scale;
                }
            }
            for (int qi = 0; qi < S; ++qi) {
                const int keys = causal ? qi + 1 : S;
                for (int ki = 0; ki < keys; ++ki) {
                    const float prob = p[(size_t)qi * S + ki];
                    const float dscore = ds[(size_t)qi * S + ki];
                    for (int d = 0; d < D; ++d) {
                        dqh[qi * D + d] += dscore * kh[ki * D + d];
                        dkh[ki * D + d] += dscore * qh[qi * D + d];
                        dvh[ki * D + d] += prob * doh[qi * D + d];
                    }
                }
            }
        }
    }
    free(p); free(ds); free(orow);
    return 0;
}
