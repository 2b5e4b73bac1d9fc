/*
 * CPU oracle for webllm's quantized-linear hot path.
 *
 * TEST INFRASTRUCTURE ONLY. This file restates, in plain C, the TypeScript
 * functions of intplusplus/webllm that define the numerics of the GPTQ int4
 * linear layer and of the Qwen2 forward pass that consumes it. It exists to
 * check the CUDA library and to be timed as the CPU baseline; the shipped
 * library never links, loads or calls it.
 *
 * The reference is TypeScript and no JavaScript engine exists where this is
 * built, so the reference itself cannot be run beside it. Parity is pinned
 * like this:
 *   - dequantiser: the closed-form known-answer test of the reference
 *     (src/tests/qwen/weights.ts:62-137), incl. the "no qzeros" branch;
 *   - fp16 <-> f32 conversions: exhaustive agreement with IEEE binary16
 *     (numpy) over all 65536 bit patterns / a dense f32 sweep;
 *   - xorshift32 RNG: first outputs computed by hand from the recurrence;
 *   - gemmNTRef / forward: the reference's tests hold no stored outputs for
 *     these (they compare GPU results against the same functions at run
 *     time), so they are pinned against an independent float64 numpy
 *     evaluation of the defining formulas on the reference's seeded inputs.
 *
 * JavaScript evaluates every arithmetic expression in double and rounds to
 * float only on a store into a Float32Array; the code below keeps exactly
 * those rounding points. Build with -ffp-contract=off so that no expression
 * is fused differently from the source.
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define WO_EXPORT __attribute__((visibility("default")))

/* ------------------------------------------------------------------ fp16 */

/* src/weights/safetensors.ts:144-152  f16BitsToF32 */
WO_EXPORT float wo_f16_bits_to_f32(uint16_t bits)
{
    double sign = (bits & 0x8000) ? -1.0 : 1.0;
    int exp = (bits >> 10) & 0x1f;
    int mant = bits & 0x03ff;
    if (exp == 0) return (float)(sign * mant * ldexp(1.0, -24));
    if (exp == 31) return mant == 0 ? (float)(sign * INFINITY) : NAN;
    return (float)(sign * (1.0 + mant / 1024.0) * ldexp(1.0, exp - 15));
}

/* src/gpu/buffer.ts:57-100  f32ToF16Bits (round to nearest even) */
WO_EXPORT uint16_t wo_f32_to_f16_bits(float f)
{
    if (isnan(f)) return 0x7e00;
    uint32_t bits;
    memcpy(&bits, &f, 4);
    uint32_t sign = (bits & 0x80000000u) >> 16;
    uint32_t exp = (bits & 0x7f800000u) >> 23;
    uint32_t mant = bits & 0x007fffffu;

    if (exp == 0xff) return (uint16_t)(sign | (mant != 0 ? 0x7e00 : 0x7c00));

    int e = (int)exp - 127;
    if (e > 15) return (uint16_t)(sign | 0x7c00);
    if (e < -24) return (uint16_t)sign;

    if (e < -14) {
        uint32_t m = mant | 0x00800000u;
        int shift = -(e + 1);
        uint32_t half = m >> shift;
        uint32_t rem = m & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half & 1u))) half++;
        return (uint16_t)(sign | half);
    }

    uint32_t half = mant >> 13;
    uint32_t rem = mant & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) {
        half++;
        if (half == 0x400u) {
            half = 0;
            e++;
            if (e > 15) return (uint16_t)(sign | 0x7c00);
        }
    }
    return (uint16_t)(sign | ((uint32_t)(e + 15) << 10) | half);
}

/* Math.f16round as the reference's tests use it (src/tests/qwen/qwen-arch.ts:21-25). */
WO_EXPORT float wo_round_f16(float f) { return wo_f16_bits_to_f32(wo_f32_to_f16_bits(f)); }

WO_EXPORT void wo_f16_to_f32_array(const uint16_t *in, float *out, int64_t n)
{
    for (int64_t i = 0; i < n; i++) out[i] = wo_f16_bits_to_f32(in[i]);
}

/* src/gpu/buffer.ts:103-120  writeF16's conversion loop */
WO_EXPORT void wo_f32_to_f16_array(const float *in, uint16_t *out, int64_t n)
{
    for (int64_t i = 0; i < n; i++) out[i] = wo_f32_to_f16_bits(in[i]);
}

/* ------------------------------------------------------------------- RNG */

/* src/reference/cpu-ref.ts:57-67  makeRng: xorshift32 (13,17,5), state/2^32 */
WO_EXPORT uint32_t wo_rng_seed(uint32_t seed) { return seed ? seed : 1u; }

WO_EXPORT double wo_rng_next(uint32_t *state)
{
    uint32_t s = *state;
    s ^= s << 13;
    s ^= s >> 17;
    s ^= s << 5;
    *state = s;
    return (double)s / 4294967296.0;
}

/* src/reference/cpu-ref.ts:50-54  randomF32: rng()*2-1 stored to f32 */
WO_EXPORT void wo_random_f32(float *out, int64_t n, uint32_t *state)
{
    for (int64_t i = 0; i < n; i++) out[i] = (float)(wo_rng_next(state) * 2.0 - 1.0);
}

/* ------------------------------------------------------------- tolerance */

/* src/reference/cpu-ref.ts:27-47  checkTolerance; returns 1 when ok */
WO_EXPORT int wo_check_tolerance(const float *got, const float *ref, int64_t n, double atol, double rtol,
                                 double *max_abs, double *max_rel)
{
    int ok = 1;
    double ma = 0, mr = 0;
    for (int64_t i = 0; i < n; i++) {
        double diff = fabs((double)got[i] - (double)ref[i]);
        if (diff > atol + rtol * fabs((double)ref[i])) ok = 0;
        if (isnan(diff)) ok = 0; /* JS: NaN > x is false, so NaN would pass there; be strict here */
        if (diff > ma) ma = diff;
        double rel = diff / fmax(1e-30, fabs((double)ref[i]));
        if (rel > mr) mr = rel;
    }
    if (max_abs) *max_abs = ma;
    if (max_rel) *max_rel = mr;
    return ok;
}

/* --------------------------------------------------------------- dequant */

static uint32_t load_u32_le(const uint8_t *p)
{
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}

/*
 * src/weights/quant.ts:42-118  dequantizeGptqInt4.
 * qweight: bytes of I32 [ceil(in/8), out]; qzeros: bytes of I32 [ceil(in/g), ceil(out/8)] or NULL;
 * scales: f32 [ceil(in/g), out]; out: f32 [out, in] row-major.
 * Returns 0, or a negative code with the reference's message text in err.
 */
WO_EXPORT int wo_dequantize_gptq_int4(const uint8_t *qweight, int64_t qweight_bytes, const uint8_t *qzeros,
                                      int64_t qzeros_bytes, const float *scales, int64_t scales_len,
                                      int64_t in_features, int64_t out_features, int64_t group_size, int bits,
                                      float *out, char *err, int err_len)
{
#define WO_FAIL(code, ...)                                   \
    do {                                                     \
        if (err && err_len > 0) snprintf(err, (size_t)err_len, __VA_ARGS__); \
        return code;                                         \
    } while (0)
    if (bits != 4) WO_FAIL(-1, "GPTQ: 当前仅支持 4bit，收到 bits=%d", bits);
    if (group_size <= 0) WO_FAIL(-2, "GPTQ: groupSize 必须为正");
    if (in_features <= 0 || out_features <= 0) WO_FAIL(-3, "GPTQ: in/out 必须为正");

    const int64_t inF = in_features, outF = out_features;
    const int64_t pack = 32 / bits;
    const uint32_t mask = (1u << bits) - 1u;
    const int64_t pack_rows = (inF + pack - 1) / pack;
    const int64_t pack_cols = (outF + pack - 1) / pack;
    const int64_t groups = (inF + group_size - 1) / group_size;

    if (qweight_bytes < pack_rows * outF * 4)
        WO_FAIL(-4, "GPTQ: qweight 字节不足，需要 %lld，实际 %lld", (long long)(pack_rows * outF * 4),
                (long long)qweight_bytes);
    if (scales_len < groups * outF)
        WO_FAIL(-5, "GPTQ: scales 数量不足，需要 %lld，实际 %lld", (long long)(groups * outF), (long long)scales_len);
    if (qzeros && qzeros_bytes < groups * pack_cols * 4)
        WO_FAIL(-6, "GPTQ: qzeros 字节不足，需要 %lld，实际 %lld", (long long)(groups * pack_cols * 4),
                (long long)qzeros_bytes);
    const int symmetric_zero = 1 << (bits - 1);
    if (group_size % pack != 0)
        WO_FAIL(-7, "GPTQ: groupSize=%lld 必须是 packFactor=%lld 的整数倍", (long long)group_size, (long long)pack);
#undef WO_FAIL

    for (int64_t pr = 0; pr < pack_rows; pr++) {
        const int64_t row_base = pr * pack;
        const int64_t g = row_base / group_size;
        const int64_t qw_row = pr * outF;
        for (int64_t o = 0; o < outF; o++) {
            const uint32_t word = load_u32_le(qweight + (qw_row + o) * 4);
            const float scale = scales[g * outF + o];
            int zero;
            if (qzeros) {
                const uint32_t zw = load_u32_le(qzeros + (g * pack_cols + o / pack) * 4);
                zero = (int)((zw >> (bits * (o % pack))) & mask) + 1;
            } else {
                zero = symmetric_zero;
            }
            for (int64_t k = 0; k < pack; k++) {
                const int64_t i = row_base + k;
                if (i >= inF) break;
                const int q = (int)((word >> (bits * k)) & mask);
                out[o * inF + i] = (float)((double)(q - zero) * (double)scale);
            }
        }
    }
    return 0;
}

/* ------------------------------------------------------------------ GEMM */

/*
 * src/reference/qwen-ref.ts:126-145  gemmNTRef: C[M,N] = A[M,K] W[N,K]^T (+bias).
 * double accumulator from 0, k ascending, bias added in double, one rounding to f32.
 * Outputs are independent dot products, so spreading (m,n) over threads changes nothing.
 */
WO_EXPORT void wo_gemm_nt_ref(const float *A, const float *W, int64_t M, int64_t N, int64_t K, const float *bias,
                              float *C, int threads)
{
    (void)threads;
#pragma omp parallel for collapse(2) schedule(static) num_threads(threads > 0 ? threads : 1)
    for (int64_t m = 0; m < M; m++) {
        for (int64_t n = 0; n < N; n++) {
            double acc = 0.0;
            const float *a = A + m * K;
            const float *w = W + n * K;
            for (int64_t k = 0; k < K; k++) acc += (double)a[k] * (double)w[k];
            C[m * N + n] = (float)(bias ? acc + (double)bias[n] : acc);
        }
    }
}

/* --------------------------------------------------------- Qwen2 forward */

/* src/reference/qwen-ref.ts:12-29  rmsNormRef */
WO_EXPORT void wo_rmsnorm_ref(const float *x, const float *w, int64_t rows, int64_t D, double eps, float *out)
{
    for (int64_t r = 0; r < rows; r++) {
        const float *xr = x + r * D;
        double sum = 0.0;
        for (int64_t d = 0; d < D; d++) sum += (double)xr[d] * (double)xr[d];
        const double rstd = 1.0 / sqrt(sum / (double)D + eps);
        for (int64_t d = 0; d < D; d++) out[r * D + d] = (float)((double)xr[d] * rstd * (double)w[d]);
    }
}

/* src/reference/qwen-ref.ts:35-64  ropeHalfRef: pos = row % T + posOffset */
WO_EXPORT void wo_rope_half_ref(const float *x, int64_t rows, int64_t n_head, int64_t D, int64_t T, double base,
                                int64_t pos_offset, float *out)
{
    const int64_t half = D / 2;
    for (int64_t r = 0; r < rows; r++) {
        const double pos = (double)((r % T) + pos_offset);
        for (int64_t h = 0; h < n_head; h++) {
            const int64_t o = (r * n_head + h) * D;
            for (int64_t i = 0; i < half; i++) {
                const double exponent = (double)(2 * i) / (double)D;
                const double angle = pos * pow(base, -exponent);
                const double c = cos(angle), s = sin(angle);
                const double x0 = x[o + i], x1 = x[o + i + half];
                out[o + i] = (float)(x0 * c - x1 * s);
                out[o + i + half] = (float)(x0 * s + x1 * c);
            }
        }
    }
}

/*
 * One (query row, head) of src/reference/qwen-ref.ts:67-116 attentionGqaRef, reading keys and
 * values through base pointers + row strides so the same code serves the uncached layout
 * ([B*T, nKv, D]) and a KV cache ([maxT, nKv*D]). `scores` is the Float32Array of the reference:
 * the scaled dot is stored to f32, the running max keeps the unrounded double.
 */
static void attn_one(const float *q, const float *kbase, const float *vbase, int64_t kv_stride, int64_t n_keys,
                     int64_t D, float *scores, float *out)
{
    const double scale = 1.0 / sqrt((double)D);
    double max_score = -INFINITY;
    for (int64_t s = 0; s < n_keys; s++) {
        const float *k = kbase + s * kv_stride;
        double dot = 0.0;
        for (int64_t d = 0; d < D; d++) dot += (double)q[d] * (double)k[d];
        dot *= scale;
        scores[s] = (float)dot;
        if (dot > max_score) max_score = dot;
    }
    double sum = 0.0;
    for (int64_t s = 0; s < n_keys; s++) {
        const double e = exp((double)scores[s] - max_score);
        scores[s] = (float)e;
        sum += e;
    }
    for (int64_t s = 0; s < n_keys; s++) scores[s] = (float)((double)scores[s] / sum);
    for (int64_t d = 0; d < D; d++) {
        double acc = 0.0;
        for (int64_t s = 0; s < n_keys; s++) acc += (double)scores[s] * (double)vbase[s * kv_stride + d];
        out[d] = (float)acc;
    }
}

/* src/reference/qwen-ref.ts:67-116  attentionGqaRef (causal, no cache) */
WO_EXPORT void wo_attention_gqa_ref(const float *q, const float *k, const float *v, int64_t B, int64_t T,
                                    int64_t n_head, int64_t n_kv, int64_t D, float *out)
{
    const int64_t group = n_head / n_kv;
    float *scores = (float *)malloc(sizeof(float) * (size_t)T);
    for (int64_t b = 0; b < B; b++)
        for (int64_t h = 0; h < n_head; h++) {
            const int64_t kvh = h / group;
            for (int64_t t = 0; t < T; t++) {
                const int64_t qb = ((b * T + t) * n_head + h) * D;
                const int64_t kb = ((b * T) * n_kv + kvh) * D;
                attn_one(q + qb, k + kb, v + kb, n_kv * D, t + 1, D, scores, out + qb);
            }
        }
    free(scores);
}

/* src/reference/qwen-ref.ts:119-123  siluMulRef */
WO_EXPORT void wo_silu_mul_ref(const float *gate, const float *up, int64_t n, float *out)
{
    for (int64_t i = 0; i < n; i++) {
        const double g = gate[i];
        out[i] = (float)((g / (1.0 + exp(-g))) * (double)up[i]);
    }
}

/* src/infer/sampler.ts:30-36  greedy branch of sampleToken: first strict maximum */
WO_EXPORT int64_t wo_sample_greedy(const float *logits, int64_t offset, int64_t vocab)
{
    int64_t best = offset;
    for (int64_t i = 1; i < vocab; i++)
        if (logits[offset + i] > logits[best]) best = offset + i;
    return best - offset;
}

/*
 * Weight bundle for the forward pass: f32 arrays in the reference's QwenWeights layout
 * (src/model/qwen.ts QwenLayerWeights: Linear weights [out, in] row-major, q/k/v with bias).
 */
typedef struct {
    const float *input_norm, *qW, *qB, *kW, *kB, *vW, *vB, *oW, *post_norm, *gateW, *upW, *downW;
} wo_layer_t;

typedef struct {
    int64_t vocab, n_layer, n_head, n_kv_head, n_embd, intermediate;
    double rms_eps, rope_theta;
} wo_config_t;

/*
 * src/reference/qwen-ref.ts:157-211  qwenForwardRef, uncached, B sequences of T tokens.
 * logits: [B*T, vocab]; layer_out (optional): n_layer buffers of [B*T, C].
 */
WO_EXPORT void wo_qwen_forward_ref(const wo_config_t *cfg, const float *embed, const float *final_norm,
                                   const wo_layer_t *layers, const uint32_t *tokens, int64_t B, int64_t T,
                                   float *logits, float **layer_out, int threads)
{
    const int64_t C = cfg->n_embd, H = cfg->n_head, KVH = cfg->n_kv_head, D = C / H, KV = D * KVH;
    const int64_t I = cfg->intermediate, V = cfg->vocab, M = B * T;
    float *x = (float *)malloc(sizeof(float) * (size_t)(M * C));
    float *n1 = (float *)malloc(sizeof(float) * (size_t)(M * C));
    float *q = (float *)malloc(sizeof(float) * (size_t)(M * C));
    float *qr = (float *)malloc(sizeof(float) * (size_t)(M * C));
    float *k = (float *)malloc(sizeof(float) * (size_t)(M * KV));
    float *kr = (float *)malloc(sizeof(float) * (size_t)(M * KV));
    float *v = (float *)malloc(sizeof(float) * (size_t)(M * KV));
    float *att = (float *)malloc(sizeof(float) * (size_t)(M * C));
    float *proj = (float *)malloc(sizeof(float) * (size_t)(M * C));
    float *xa = (float *)malloc(sizeof(float) * (size_t)(M * C));
    float *gate = (float *)malloc(sizeof(float) * (size_t)(M * I));
    float *up = (float *)malloc(sizeof(float) * (size_t)(M * I));
    float *act = (float *)malloc(sizeof(float) * (size_t)(M * I));

    for (int64_t m = 0; m < M; m++) memcpy(x + m * C, embed + (int64_t)tokens[m] * C, sizeof(float) * (size_t)C);

    for (int64_t i = 0; i < cfg->n_layer; i++) {
        const wo_layer_t *L = &layers[i];
        wo_rmsnorm_ref(x, L->input_norm, M, C, cfg->rms_eps, n1);
        wo_gemm_nt_ref(n1, L->qW, M, C, C, L->qB, q, threads);
        wo_gemm_nt_ref(n1, L->kW, M, KV, C, L->kB, k, threads);
        wo_gemm_nt_ref(n1, L->vW, M, KV, C, L->vB, v, threads);
        wo_rope_half_ref(q, M, H, D, T, cfg->rope_theta, 0, qr);
        wo_rope_half_ref(k, M, KVH, D, T, cfg->rope_theta, 0, kr);
        wo_attention_gqa_ref(qr, kr, v, B, T, H, KVH, D, att);
        wo_gemm_nt_ref(att, L->oW, M, C, C, NULL, proj, threads);
        for (int64_t j = 0; j < M * C; j++) xa[j] = x[j] + proj[j];
        wo_rmsnorm_ref(xa, L->post_norm, M, C, cfg->rms_eps, n1);
        wo_gemm_nt_ref(n1, L->gateW, M, I, C, NULL, gate, threads);
        wo_gemm_nt_ref(n1, L->upW, M, I, C, NULL, up, threads);
        wo_silu_mul_ref(gate, up, M * I, act);
        wo_gemm_nt_ref(act, L->downW, M, C, I, NULL, proj, threads);
        for (int64_t j = 0; j < M * C; j++) x[j] = xa[j] + proj[j];
        if (layer_out && layer_out[i]) memcpy(layer_out[i], x, sizeof(float) * (size_t)(M * C));
    }
    wo_rmsnorm_ref(x, final_norm, M, C, cfg->rms_eps, n1);
    wo_gemm_nt_ref(n1, embed, M, V, C, NULL, logits, threads);

    free(x); free(n1); free(q); free(qr); free(k); free(kr); free(v); free(att); free(proj); free(xa);
    free(gate); free(up); free(act);
}

/*
 * The same forward with a KV cache, one sequence: processes rows [past, past+T) and appends their
 * rotated keys / values to k_cache / v_cache ([n_layer][max_t, KV] f32). Row r attends keys
 * 0..past+r, which is what the uncached reference computes for the same absolute positions (the
 * reference asserts this equivalence itself, src/tests/qwen/qwen-arch.ts:139-210).
 * kv_f16 != 0 rounds every cached key/value to fp16 (RNE) on store, modelling an fp16 cache.
 * logits receives only the last processed row, [vocab].
 */
WO_EXPORT void wo_qwen_forward_cached(const wo_config_t *cfg, const float *embed, const float *final_norm,
                                      const wo_layer_t *layers, const uint32_t *tokens, int64_t T, int64_t past,
                                      int64_t max_t, float *k_cache, float *v_cache, int kv_f16, float *logits,
                                      int threads)
{
    const int64_t C = cfg->n_embd, H = cfg->n_head, KVH = cfg->n_kv_head, D = C / H, KV = D * KVH;
    const int64_t I = cfg->intermediate, V = cfg->vocab, M = T, group = H / KVH;
    float *x = (float *)malloc(sizeof(float) * (size_t)(M * C));
    float *n1 = (float *)malloc(sizeof(float) * (size_t)(M * C));
    float *q = (float *)malloc(sizeof(float) * (size_t)(M * C));
    float *qr = (float *)malloc(sizeof(float) * (size_t)(M * C));
    float *k = (float *)malloc(sizeof(float) * (size_t)(M * KV));
    float *kr = (float *)malloc(sizeof(float) * (size_t)(M * KV));
    float *v = (float *)malloc(sizeof(float) * (size_t)(M * KV));
    float *att = (float *)malloc(sizeof(float) * (size_t)(M * C));
    float *proj = (float *)malloc(sizeof(float) * (size_t)(M * C));
    float *xa = (float *)malloc(sizeof(float) * (size_t)(M * C));
    float *gate = (float *)malloc(sizeof(float) * (size_t)(M * I));
    float *up = (float *)malloc(sizeof(float) * (size_t)(M * I));
    float *act = (float *)malloc(sizeof(float) * (size_t)(M * I));

    for (int64_t m = 0; m < M; m++) memcpy(x + m * C, embed + (int64_t)tokens[m] * C, sizeof(float) * (size_t)C);

    for (int64_t i = 0; i < cfg->n_layer; i++) {
        const wo_layer_t *L = &layers[i];
        float *kc = k_cache + i * max_t * KV;
        float *vc = v_cache + i * max_t * KV;
        wo_rmsnorm_ref(x, L->input_norm, M, C, cfg->rms_eps, n1);
        wo_gemm_nt_ref(n1, L->qW, M, C, C, L->qB, q, threads);
        wo_gemm_nt_ref(n1, L->kW, M, KV, C, L->kB, k, threads);
        wo_gemm_nt_ref(n1, L->vW, M, KV, C, L->vB, v, threads);
        /* T = M and posOffset = past give pos = row + past (src/model/qwen.ts:363-365) */
        wo_rope_half_ref(q, M, H, D, M, cfg->rope_theta, past, qr);
        wo_rope_half_ref(k, M, KVH, D, M, cfg->rope_theta, past, kr);
        for (int64_t j = 0; j < M * KV; j++) {
            kc[past * KV + j] = kv_f16 ? wo_round_f16(kr[j]) : kr[j];
            vc[past * KV + j] = kv_f16 ? wo_round_f16(v[j]) : v[j];
        }
#pragma omp parallel num_threads(threads > 0 ? threads : 1)
        {
            float *scores = (float *)malloc(sizeof(float) * (size_t)(past + M));
#pragma omp for collapse(2) schedule(static)
            for (int64_t r = 0; r < M; r++)
                for (int64_t h = 0; h < H; h++) {
                    const int64_t kvh = h / group;
                    attn_one(qr + (r * H + h) * D, kc + kvh * D, vc + kvh * D, KV, past + r + 1, D, scores,
                             att + (r * H + h) * D);
                }
            free(scores);
        }
        wo_gemm_nt_ref(att, L->oW, M, C, C, NULL, proj, threads);
        for (int64_t j = 0; j < M * C; j++) xa[j] = x[j] + proj[j];
        wo_rmsnorm_ref(xa, L->post_norm, M, C, cfg->rms_eps, n1);
        wo_gemm_nt_ref(n1, L->gateW, M, I, C, NULL, gate, threads);
        wo_gemm_nt_ref(n1, L->upW, M, I, C, NULL, up, threads);
        wo_silu_mul_ref(gate, up, M * I, act);
        wo_gemm_nt_ref(act, L->downW, M, C, I, NULL, proj, threads);
        for (int64_t j = 0; j < M * C; j++) x[j] = xa[j] + proj[j];
    }
    wo_rmsnorm_ref(x + (M - 1) * C, final_norm, 1, C, cfg->rms_eps, n1);
    wo_gemm_nt_ref(n1, embed, 1, V, C, NULL, logits, threads);

    free(x); free(n1); free(q); free(qr); free(k); free(kr); free(v); free(att); free(proj); free(xa);
    free(gate); free(up); free(act);
}

WO_EXPORT int wo_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
