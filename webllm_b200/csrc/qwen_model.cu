// Qwen2 forward pass, prefill and decode over the kernels of this library. Follows QwenGpt.runForward
// (src/model/qwen.ts:333-500) step for step; the residual adds are folded into the RMSNorm that follows
// them and q/k/v (gate/up) may run as one fused projection.
#include <math.h>

#include <algorithm>
#include <memory>

#include "qwen_internal.cuh"

using namespace wb;

using wbq::Bufs;
using wbq::LayerW;

namespace {

size_t kv_elem(const wb_qwen *m) { return m->cfg.kv_dtype == WB_F16 ? 2 : 4; }

int find(wb_context *ctx, const std::string &name)
{
    auto it = ctx->by_name.find(name);
    return it == ctx->by_name.end() ? -1 : it->second;
}

int require(wb_context *ctx, const std::string &name, WeightKind kind_a, WeightKind kind_b, int64_t K, int64_t N, int *out)
{
    const int h = find(ctx, name);
    if (h < 0) return fail(WB_ERR_NOT_FOUND, "缺少权重: %s", name.c_str());
    const Weight &w = ctx->weights[h];
    if (w.kind != kind_a && w.kind != kind_b) return fail(WB_ERR_BAD_ARG, "weight %s has the wrong type", name.c_str());
    if (w.kind == WeightKind::F32 ? (w.N != N) : (w.K != K || w.N != N))
        return fail(WB_ERR_BAD_ARG, "weight %s has shape [%lld,%lld], expected [%lld,%lld]", name.c_str(), (long long)w.N,
                    (long long)w.K, (long long)N, (long long)K);
    *out = h;
    return WB_OK;
}

int carve(wb_context *ctx, int arena, uint64_t bytes, void **out)
{
    uint64_t off = 0;
    WB_CHECK(wb_arena_alloc(ctx, arena, bytes, &off));
    *out = ctx->arena[arena].base + off;
    return WB_OK;
}

template <typename T>
int carve_t(wb_context *ctx, int arena, uint64_t count, T **out)
{
    void *p = nullptr;
    WB_CHECK(carve(ctx, arena, count * sizeof(T), &p));
    *out = (T *)p;
    return WB_OK;
}

int alloc_bufs(wb_qwen *m, int arena, int64_t M, int64_t logit_rows, Bufs *b)
{
    wb_context *ctx = m->ctx;
    const int C = m->C, KV = m->KV, I = m->I;
    const bool fused_qkv = m->layers[0].qkv >= 0, fused_gu = m->layers[0].gate_up >= 0;
    WB_CHECK(carve_t(ctx, arena, M, &b->tokens));
    WB_CHECK(carve_t(ctx, arena, M * C, &b->x));
    WB_CHECK(carve_t(ctx, arena, M * C, &b->xa));
    WB_CHECK(carve_t(ctx, arena, M * C, &b->n));
    WB_CHECK(carve_t(ctx, arena, M * (C + 2 * KV), &b->q));
    if (fused_qkv) {
        b->k = b->q + C, b->v = b->q + C + KV;
        b->ldq = b->ldk = b->ldv = C + 2 * KV;
    } else {
        b->k = b->q + M * C, b->v = b->k + M * KV;
        b->ldq = C, b->ldk = b->ldv = KV;
    }
    WB_CHECK(carve_t(ctx, arena, M * C, &b->att));
    WB_CHECK(carve_t(ctx, arena, M * C, &b->proj));
    WB_CHECK(carve_t(ctx, arena, M * 2 * I, &b->gu));
    b->ld_gu = fused_gu ? 2 * I : I;
    WB_CHECK(carve_t(ctx, arena, M * I, &b->act));
    b->h16 = nullptr;
    if (M > 8) WB_CHECK(carve_t(ctx, arena, M * (int64_t)std::max(C, I), &b->h16));
    WB_CHECK(carve_t(ctx, arena, logit_rows * m->V, &b->logits));
    return WB_OK;
}

// `next` (optional): the weight of the linear that follows in the forward pass. A decode step used to ask the L2 for
// it while this projection runs (wb_linear_hint_next does that for any caller); since every kernel releases its
// successor after its own wait, the successor's own first weight requests already run under this kernel, and the extra
// prefetch traffic measured 1.2 % slower on the decode step (0.552 against 0.546 ms), so the model no longer asks.
int linear(wb_qwen *m, int wh, const float *A, float *Cout, int bias, int64_t M, int next = -1,
           const LinearFusion *fusion = nullptr)
{
    wb_context *ctx = m->ctx;
    (void)next;
    ctx->prefetch_weight = -1;
    const Weight &w = ctx->weights[wh];
    const float *bp = bias >= 0 ? (const float *)(ctx->arena[WB_ARENA_WEIGHTS].base + ctx->weights[bias].off_main) : nullptr;
    return launch_linear(ctx, w, A, Cout, bp, M, WB_F32, WB_F32, m->exact, fusion);
}

// The same with the activation already in fp16 (written so by the step before it: see `half_in` in forward_impl).
int linear_h16(wb_qwen *m, int wh, const __half *A, float *Cout, int bias, int64_t M)
{
    wb_context *ctx = m->ctx;
    ctx->prefetch_weight = -1;
    const Weight &w = ctx->weights[wh];
    const float *bp = bias >= 0 ? (const float *)(ctx->arena[WB_ARENA_WEIGHTS].base + ctx->weights[bias].off_main) : nullptr;
    return launch_linear(ctx, w, A, Cout, bp, M, WB_F16, WB_F32, 0, nullptr);
}

// One forward pass over rows [0, M). past_ptr != nullptr: positions come from device memory (graph replay).
int forward_impl(wb_qwen *m, const Bufs &b, int64_t M, int64_t B, int64_t T, int64_t past, const int *past_ptr,
                 bool use_cache, bool last_only)
{
    wb_context *ctx = m->ctx;
    const int C = m->C, H = m->H, KVH = m->KVH, D = m->D, KV = m->KV, I = m->I;
    const char *wbase = ctx->arena[WB_ARENA_WEIGHTS].base;
    auto f32w = [&](int h) { return (const float *)(wbase + ctx->weights[h].off_main); };
    const bool kv16 = m->cfg.kv_dtype == WB_F16;
    const size_t layer_stride = (size_t)m->cfg.max_t * KV * kv_elem(m);

    WB_CHECK(op_embed(ctx, (const __half *)(wbase + ctx->weights[m->embed].off_main), b.tokens, b.x, (int)M, C, m->V));
    const float *delta = nullptr;  // pending residual contribution, folded into the next rmsnorm
    float *x = b.x;                // residual stream before `delta` is added
    // A decode step over fused int4 projections runs five kernels per layer: the norms, silu * up and the rotary
    // embedding + cache append ride inside the projections and the attention kernel (see GemvPrologue).
    const LayerW &L0 = m->layers[0];
    const bool fused_step = M == 1 && use_cache && L0.qkv >= 0 && L0.gate_up >= 0 && D % 8 == 0 && D <= 128 &&
                            op_attention_decode_smem(D, m->cfg.max_t, kv16) <= 160 * 1024 &&
                            linear_fusion_supported(ctx, ctx->weights[L0.qkv], 1) &&
                            linear_fusion_supported(ctx, ctx->weights[L0.gate_up], 1) &&
                            linear_fusion_supported(ctx, ctx->weights[L0.down], 1);
    for (int i = 0; i < m->cfg.n_layer; i++) {
        const LayerW &L = m->layers[i];
        char *kc = use_cache ? m->k_cache + i * layer_stride : nullptr;
        char *vc = use_cache ? m->v_cache + i * layer_stride : nullptr;
        if (fused_step) {
            const int max_keys = past_ptr ? m->cfg.max_t : (int)(past + M);
            float *x_in = (delta ? (x == b.x ? b.xa : b.x) : x);
            LinearFusion f{};
            f.kind = 1, f.delta = delta, f.x_out = delta ? x_in : nullptr, f.norm_w = f32w(L.in_norm), f.eps = m->cfg.rms_eps;
            WB_CHECK(linear(m, L.qkv, x, b.q, L.qkvb, 1, L.o, &f));
            x = x_in;
            // (the kernel in front is the q|k|v GEMV, which releases this one after its own wait: the cache and the position
            // are complete by the time this kernel can start, so it reads them before it waits)
            static const int early_kv = [] { const char *e = getenv("WEBLLM_B200_ATT_EARLY"); return (e && e[0] == '0') ? 0 : 1; }();
            WB_CHECK(op_attention_decode(ctx, b.q, kc, vc, kv16, b.att, m->att_scratch, m->att_counters, H, KVH, D, past_ptr,
                                         (int)past, max_keys, KV, b.k, b.v, m->cs_table, early_kv));
            WB_CHECK(linear(m, L.o, b.att, b.proj, -1, 1, L.gate_up));
            float *xa = (x == b.x ? b.xa : b.x);
            f.delta = b.proj, f.x_out = xa, f.norm_w = f32w(L.post_norm);
            WB_CHECK(linear(m, L.gate_up, x, b.gu, -1, 1, L.down, &f));
            x = xa;
            LinearFusion g{};
            g.kind = 2, g.up = b.gu + I, g.ld = 2 * I;
            WB_CHECK(linear(m, L.down, b.gu, b.proj, -1, 1, i + 1 < m->cfg.n_layer ? m->layers[i + 1].qkv : -1, &g));
            delta = b.proj;
            continue;
        }
        // --- attention sub-layer
        // Default mode at prefill sizes: every projection runs on the tensor cores and would round its f32 input to
        // fp16 first; the step that produces that input writes the fp16 value itself (same numbers, one pass over
        // the activations fewer per projection). Only where the fused projections exist (one consumer per producer).
        const bool half_in = !m->exact && b.h16 != nullptr && L.qkv >= 0 && L.gate_up >= 0;
        float *x_in = (delta ? (x == b.x ? b.xa : b.x) : x);
        WB_CHECK(op_rmsnorm(ctx, x, delta, x_in, f32w(L.in_norm), b.n, (int)M, C, m->cfg.rms_eps, half_in ? b.h16 : nullptr));
        x = x_in;
        if (L.qkv >= 0) {
            if (half_in) WB_CHECK(linear_h16(m, L.qkv, b.h16, b.q, L.qkvb, M));
            else WB_CHECK(linear(m, L.qkv, b.n, b.q, L.qkvb, M, L.o));
        } else {
            WB_CHECK(linear(m, L.q, b.n, b.q, L.qb, M));
            WB_CHECK(linear(m, L.k, b.n, b.k, L.kb, M));
            WB_CHECK(linear(m, L.v, b.n, b.v, L.vb, M));
        }
        WB_CHECK(op_rope_kv(ctx, b.q, b.k, b.v, kc, vc, kv16, m->cs_table, (int)M, H, KVH, D, (int)T, past_ptr, (int)past,
                            b.ldq, b.ldk, b.ldv));
        bool att_half = false;
        if (use_cache) {
            const int max_keys = past_ptr ? m->cfg.max_t : (int)(past + M);
            if (M == 1 && D % 8 == 0 && D <= 128 && op_attention_decode_smem(D, max_keys, kv16) <= 160 * 1024) {
                WB_CHECK(op_attention_decode(ctx, b.q, kc, vc, kv16, b.att, m->att_scratch, m->att_counters, H, KVH, D, past_ptr,
                                             (int)past, max_keys, KV));
            } else if (!m->exact && op_attention_prefill_supported((int)M, H, KVH, D, b.ldq, KV)) {
                // prefill in the default mode: causal attention on the tensor cores (fp16 operands, like the linears)
                att_half = half_in;
                WB_CHECK(op_attention_prefill(ctx, b.q, kc, vc, kv16, b.att, (int)M, H, KVH, D, past_ptr, (int)past, b.ldq, KV,
                                              att_half ? b.h16 : nullptr));
            } else {
                WB_CHECK(op_attention(ctx, b.q, kc, vc, kv16, b.att, (int)M, H, KVH, D, (int)T, past_ptr, (int)past, 1, max_keys,
                                      b.ldq, KV));
            }
        } else {
            WB_CHECK(op_attention(ctx, b.q, b.k, b.v, 0, b.att, (int)M, H, KVH, D, (int)T, nullptr, 0, 0, (int)T, b.ldq, b.ldk));
        }
        if (att_half) WB_CHECK(linear_h16(m, L.o, b.h16, b.proj, -1, M));
        else WB_CHECK(linear(m, L.o, b.att, b.proj, -1, M, L.gate_up));
        // --- MLP sub-layer: xa = x + proj; n = rmsnorm(xa)
        float *xa = (x == b.x ? b.xa : b.x);
        WB_CHECK(op_rmsnorm(ctx, x, b.proj, xa, f32w(L.post_norm), b.n, (int)M, C, m->cfg.rms_eps, half_in ? b.h16 : nullptr));
        x = xa;
        if (L.gate_up >= 0) {
            if (half_in) WB_CHECK(linear_h16(m, L.gate_up, b.h16, b.gu, -1, M));
            else WB_CHECK(linear(m, L.gate_up, b.n, b.gu, -1, M, L.down));
            WB_CHECK(op_silu_mul(ctx, b.gu, b.gu + I, b.act, (int)M, I, 2 * I, half_in ? b.h16 : nullptr));
        } else {
            WB_CHECK(linear(m, L.gate, b.n, b.gu, -1, M));
            WB_CHECK(linear(m, L.up, b.n, b.gu + M * I, -1, M));
            WB_CHECK(op_silu_mul(ctx, b.gu, b.gu + M * I, b.act, (int)M, I, I));
        }
        if (half_in) WB_CHECK(linear_h16(m, L.down, b.h16, b.proj, -1, M));
        else WB_CHECK(linear(m, L.down, b.act, b.proj, -1, M, i + 1 < m->cfg.n_layer ? m->layers[i + 1].qkv : -1));
        delta = b.proj;
    }
    // final norm (+ the last residual add), then the tied lm_head
    float *xf = (x == b.x ? b.xa : b.x);
    if (last_only) {
        const int64_t r = M - 1;
        WB_CHECK(op_rmsnorm(ctx, x + r * C, delta + r * C, xf, f32w(m->final_norm), b.n, 1, C, m->cfg.rms_eps));
        WB_CHECK(linear(m, m->embed, b.n, b.logits, -1, 1));
    } else {
        WB_CHECK(op_rmsnorm(ctx, x, delta, xf, f32w(m->final_norm), b.n, (int)M, C, m->cfg.rms_eps));
        WB_CHECK(linear(m, m->embed, b.n, b.logits, -1, M));
    }
    return WB_OK;
}

}  // namespace

#define WB_MODEL(m)                                                          \
    do {                                                                     \
        if (!(m)) return wb::fail(WB_ERR_BAD_ARG, "model is NULL");          \
        WB_CUDA(cudaSetDevice((m)->ctx->device));                            \
    } while (0)

static void drop_graph(wb_qwen *m)
{
    if (m->graph) cudaGraphExecDestroy(m->graph);
    m->graph = nullptr;
}

extern "C" {

int wb_qwen_create(wb_context *ctx, const wb_qwen_config *cfg, wb_qwen **out)
{
    if (!ctx || !cfg || !out) return fail(WB_ERR_BAD_ARG, "wb_qwen_create: NULL argument");
    WB_CUDA(cudaSetDevice(ctx->device));
    WB_NOT_RECORDING(ctx, "wb_qwen_create");
    if (cfg->n_head <= 0 || cfg->n_embd % cfg->n_head != 0)
        return fail(WB_ERR_BAD_ARG, "nEmbd(%d) 必须能被 nHead(%d) 整除", cfg->n_embd, cfg->n_head);
    if (cfg->n_kv_head <= 0 || cfg->n_head % cfg->n_kv_head != 0)
        return fail(WB_ERR_BAD_ARG, "nHead(%d) must be a multiple of nKvHead(%d)", cfg->n_head, cfg->n_kv_head);
    if (cfg->max_t <= 0 || cfg->n_layer <= 0 || cfg->vocab_size <= 0 || cfg->intermediate <= 0)
        return fail(WB_ERR_BAD_ARG, "wb_qwen_create: sizes must be positive");
    if (cfg->kv_dtype != WB_F32 && cfg->kv_dtype != WB_F16) return fail(WB_ERR_BAD_ARG, "kv_dtype must be WB_F32 or WB_F16");
    std::unique_ptr<wb_qwen> m(new wb_qwen());
    m->ctx = ctx;
    m->cfg = *cfg;
    m->C = cfg->n_embd, m->H = cfg->n_head, m->KVH = cfg->n_kv_head, m->D = cfg->n_embd / cfg->n_head;
    m->KV = m->D * m->KVH, m->I = cfg->intermediate, m->V = cfg->vocab_size;
    if (m->D % 2) return fail(WB_ERR_BAD_ARG, "head dimension must be even");
    const int C = m->C, KV = m->KV, I = m->I, V = m->V;
    const WeightKind G = WeightKind::Gptq, F = WeightKind::DenseF16, R = WeightKind::F32;
    WB_CHECK(require(ctx, "embed", F, F, C, V, &m->embed));
    WB_CHECK(require(ctx, "finalNorm", R, R, 1, C, &m->final_norm));
    m->layers.resize(cfg->n_layer);
    for (int i = 0; i < cfg->n_layer; i++) {
        LayerW &L = m->layers[i];
        const std::string p = "L" + std::to_string(i) + ".";
        WB_CHECK(require(ctx, p + "inNorm", R, R, 1, C, &L.in_norm));
        WB_CHECK(require(ctx, p + "postNorm", R, R, 1, C, &L.post_norm));
        if (find(ctx, p + "qkvW") >= 0) {
            WB_CHECK(require(ctx, p + "qkvW", G, F, C, C + 2 * KV, &L.qkv));
            WB_CHECK(require(ctx, p + "qkvB", R, R, 1, C + 2 * KV, &L.qkvb));
        } else {
            WB_CHECK(require(ctx, p + "qW", G, F, C, C, &L.q));
            WB_CHECK(require(ctx, p + "kW", G, F, C, KV, &L.k));
            WB_CHECK(require(ctx, p + "vW", G, F, C, KV, &L.v));
            WB_CHECK(require(ctx, p + "qB", R, R, 1, C, &L.qb));
            WB_CHECK(require(ctx, p + "kB", R, R, 1, KV, &L.kb));
            WB_CHECK(require(ctx, p + "vB", R, R, 1, KV, &L.vb));
        }
        WB_CHECK(require(ctx, p + "oW", G, F, C, C, &L.o));
        if (find(ctx, p + "gateUpW") >= 0) {
            WB_CHECK(require(ctx, p + "gateUpW", G, F, C, 2 * I, &L.gate_up));
        } else {
            WB_CHECK(require(ctx, p + "gateW", G, F, C, I, &L.gate));
            WB_CHECK(require(ctx, p + "upW", G, F, C, I, &L.up));
        }
        WB_CHECK(require(ctx, p + "downW", G, F, I, C, &L.down));
        if ((L.qkv >= 0) != (m->layers[0].qkv >= 0) || (L.gate_up >= 0) != (m->layers[0].gate_up >= 0))
            return fail(WB_ERR_BAD_ARG, "layers must all use fused projections or none");
    }
    // residency owned by the model: KV cache, rope table, decode state (taken from the weight slab, handed back by
    // wb_qwen_destroy when nothing was allocated after it)
    m->carve_mark = ctx->arena[WB_ARENA_WEIGHTS].used;
    const int rc = [&]() -> int {
        const uint64_t cache_bytes = (uint64_t)cfg->n_layer * cfg->max_t * KV * kv_elem(m.get());
        WB_CHECK(carve(ctx, WB_ARENA_WEIGHTS, cache_bytes, (void **)&m->k_cache));
        WB_CHECK(carve(ctx, WB_ARENA_WEIGHTS, cache_bytes, (void **)&m->v_cache));
        WB_CUDA(cudaMemsetAsync(m->k_cache, 0, cache_bytes, ctx->stream));
        WB_CUDA(cudaMemsetAsync(m->v_cache, 0, cache_bytes, ctx->stream));
        const int half = m->D / 2;
        std::vector<float> cs((size_t)cfg->max_t * half * 2);
        for (int pos = 0; pos < cfg->max_t; pos++)
            for (int i = 0; i < half; i++) {
                // ropeHalfRef: angle = pos * base^(-(2i)/D), evaluated in double (src/reference/qwen-ref.ts:49-53)
                const double angle = (double)pos * pow((double)cfg->rope_theta, -((double)(2 * i) / (double)m->D));
                cs[((size_t)pos * half + i) * 2] = (float)cos(angle);
                cs[((size_t)pos * half + i) * 2 + 1] = (float)sin(angle);
            }
        WB_CHECK(carve_t(ctx, WB_ARENA_WEIGHTS, cs.size(), &m->cs_table));
        WB_CUDA(cudaMemcpyAsync(m->cs_table, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
        WB_CHECK(alloc_bufs(m.get(), WB_ARENA_WEIGHTS, 1, 1, &m->dec));
        m->history_cap = cfg->max_t;
        m->host_pin_cap = (size_t)cfg->max_t;
        WB_CUDA(cudaHostAlloc((void **)&m->host_pin, m->host_pin_cap * sizeof(uint32_t), cudaHostAllocDefault));
        WB_CHECK(carve_t(ctx, WB_ARENA_WEIGHTS, (uint64_t)m->history_cap, &m->d_history));
        WB_CHECK(carve_t(ctx, WB_ARENA_WEIGHTS, 64, &m->d_cache_len));
        m->d_step = m->d_cache_len + 1;
        WB_CHECK(carve_t(ctx, WB_ARENA_WEIGHTS, 128, &m->d_bval));
        WB_CHECK(carve_t(ctx, WB_ARENA_WEIGHTS, 128, &m->d_bidx));
        WB_CUDA(cudaMemsetAsync(m->d_cache_len, 0, 64 * sizeof(int), ctx->stream));
        WB_CHECK(carve_t(ctx, WB_ARENA_WEIGHTS, (uint64_t)op_attention_decode_scratch_floats(m->H, m->D), &m->att_scratch));
        WB_CHECK(carve_t(ctx, WB_ARENA_WEIGHTS, (uint64_t)m->H, &m->att_counters));
        WB_CUDA(cudaMemsetAsync(m->att_counters, 0, (size_t)m->H * sizeof(unsigned), ctx->stream));
        WB_CUDA(cudaStreamSynchronize(ctx->stream));  // `cs` is read by the copy until here
        return WB_OK;
    }();
    if (rc != WB_OK) {
        cudaStreamSynchronize(ctx->stream);
        if (m->host_pin) cudaFreeHost(m->host_pin);
        ctx->arena[WB_ARENA_WEIGHTS].used = m->carve_mark;
        return rc;
    }
    m->carve_top = ctx->arena[WB_ARENA_WEIGHTS].used;
    *out = m.release();
    return WB_OK;
}

int wb_qwen_destroy(wb_qwen *m)
{
    if (!m) return WB_OK;
    cudaSetDevice(m->ctx->device);
    cudaStreamSynchronize(m->ctx->stream);
    drop_graph(m);
    // the model's carve is handed back when it still is the top of the weight arena
    ArenaState &wa = m->ctx->arena[WB_ARENA_WEIGHTS];
    if (wa.used == m->carve_top) wa.used = m->carve_mark;
    if (m->host_pin) cudaFreeHost(m->host_pin);
    delete m;
    return WB_OK;
}

int wb_qwen_reset_cache(wb_qwen *m)
{
    WB_MODEL(m);
    m->cache_len = 0;
    return WB_OK;
}

int wb_qwen_cache_len(wb_qwen *m, int64_t *len)
{
    WB_MODEL(m);
    *len = m->cache_len;
    return WB_OK;
}

int wb_qwen_set_exact(wb_qwen *m, int exact)
{
    WB_MODEL(m);
    m->exact = exact ? 1 : 0;
    return WB_OK;
}

static int check_tokens(const wb_qwen *m, const uint32_t *tokens, int64_t n)
{
    if (!tokens) return fail(WB_ERR_BAD_ARG, "tokens is NULL");
    for (int64_t i = 0; i < n; i++)
        if (tokens[i] >= (uint32_t)m->V) return fail(WB_ERR_BAD_ARG, "token id %u at %lld is outside the vocabulary of %d", tokens[i], (long long)i, m->V);
    return WB_OK;
}

static int run_eager(wb_qwen *m, const uint32_t *tokens, int64_t M, int64_t B, int64_t T, int64_t past, bool use_cache,
                     bool last_only, uint64_t *logits_offset)
{
    wb_context *ctx = m->ctx;
    WB_CHECK(check_tokens(m, tokens, M));
    WB_CHECK(wb_arena_reset(ctx, WB_ARENA_ACT));  // runForward: this.arena.reset() (src/model/qwen.ts:359)
    Bufs b{};
    WB_CHECK(alloc_bufs(m, WB_ARENA_ACT, M, last_only ? 1 : M, &b));
    WB_CUDA(cudaMemcpyAsync(b.tokens, tokens, (size_t)M * 4, cudaMemcpyHostToDevice, ctx->stream));
    WB_CHECK(forward_impl(m, b, M, B, T, past, nullptr, use_cache, last_only));
    if (use_cache) m->cache_len = past + M;
    if (logits_offset) *logits_offset = (uint64_t)((char *)b.logits - ctx->arena[WB_ARENA_ACT].base);
    return WB_OK;
}

int wb_qwen_forward(wb_qwen *m, const uint32_t *tokens, int64_t B, int64_t T, uint64_t *logits_offset)
{
    WB_MODEL(m);
    WB_NOT_RECORDING(m->ctx, "wb_qwen_forward");
    if (B <= 0 || T <= 0) return fail(WB_ERR_BAD_ARG, "forward: B and T must be positive");
    if (T > m->cfg.max_t) return fail(WB_ERR_BAD_ARG, "T=%lld 超过 blockSize=%d", (long long)T, m->cfg.max_t);
    return run_eager(m, tokens, B * T, B, T, 0, false, false, logits_offset);
}

int wb_qwen_prefill(wb_qwen *m, const uint32_t *tokens, int64_t n, int last_only, uint64_t *logits_offset)
{
    WB_MODEL(m);
    WB_NOT_RECORDING(m->ctx, "wb_qwen_prefill");
    if (m->cache_len != 0) return fail(WB_ERR_BAD_ARG, "prefill 前请先 resetCache()（当前 cacheLen=%lld）", (long long)m->cache_len);
    if (n <= 0) return fail(WB_ERR_BAD_ARG, "prefill: tokens 不能为空");
    if (n > m->cfg.max_t) return fail(WB_ERR_BAD_ARG, "上下文长度 %lld 超过 blockSize=%d", (long long)n, m->cfg.max_t);
    return run_eager(m, tokens, n, 1, n, 0, true, last_only != 0, logits_offset);
}

int wb_qwen_decode_step(wb_qwen *m, uint32_t token, uint64_t *logits_offset)
{
    WB_MODEL(m);
    WB_NOT_RECORDING(m->ctx, "wb_qwen_decode_step");
    if (m->cache_len == 0) return fail(WB_ERR_BAD_ARG, "decodeStep 前请先调用 prefill()");
    if (m->cache_len + 1 > m->cfg.max_t)
        return fail(WB_ERR_BAD_ARG, "上下文长度 %lld 超过 blockSize=%d", (long long)(m->cache_len + 1), m->cfg.max_t);
    return run_eager(m, &token, 1, 1, 1, m->cache_len, true, true, logits_offset);
}

__global__ void set_decode_state_kernel(int *cache_len, int *step, uint32_t *tokens, int len, uint32_t first_token)
{
    *cache_len = len, *step = 0, *tokens = first_token;
}

// One decode step on the persistent M = 1 buffers, positions read from device memory, followed by the
// on-device argmax that also appends the token and bumps the cache length.
static int enqueue_graph_step(wb_qwen *m)
{
    WB_CHECK(forward_impl(m, m->dec, 1, 1, 1, 0, m->d_cache_len, true, true));
    return op_argmax(m->ctx, m->dec.logits, m->V, m->d_bval, m->d_bidx, m->dec.tokens, m->d_history, m->d_step, m->d_cache_len);
}

int wb_qwen_decode_greedy(wb_qwen *m, uint32_t first_token, int64_t n_steps, uint32_t *out_tokens)
{
    WB_MODEL(m);
    WB_NOT_RECORDING(m->ctx, "wb_qwen_decode_greedy");
    wb_context *ctx = m->ctx;
    if (m->cache_len == 0) return fail(WB_ERR_BAD_ARG, "decodeStep 前请先调用 prefill()");
    if (n_steps <= 0 || !out_tokens) return fail(WB_ERR_BAD_ARG, "decode_greedy: n_steps must be positive");
    if (m->cache_len + n_steps > m->cfg.max_t)
        return fail(WB_ERR_BAD_ARG, "上下文长度 %lld 超过 blockSize=%d", (long long)(m->cache_len + n_steps), m->cfg.max_t);
    WB_CHECK(check_tokens(m, &first_token, 1));
    // the decode state (cache length, step counter, first token) goes to the device as the arguments of one tiny kernel:
    // no staging of pageable host memory on the per-token path
    auto set_state = [&]() -> int {
        set_decode_state_kernel<<<1, 1, 0, ctx->stream>>>(m->d_cache_len, m->d_step, m->dec.tokens, (int)m->cache_len, first_token);
        ctx->launches++;
        WB_CUDA(cudaGetLastError());
        return WB_OK;
    };
    WB_CHECK(set_state());
    if (m->graph && (m->graph_stream != ctx->stream || m->graph_exact != m->exact)) drop_graph(m);
    if (!m->graph) {
        // Warm-up step outside capture (sets kernel attributes, counts the step's kernels), then restore the
        // state it advanced.
        const uint64_t launches_warm = ctx->launches;
        WB_CHECK(enqueue_graph_step(m));
        m->graph_launches = ctx->launches - launches_warm;
        WB_CHECK(set_state());
        WB_CUDA(cudaStreamSynchronize(ctx->stream));
        cudaGraph_t g = nullptr;
        WB_CUDA(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
        const uint64_t launches_before = ctx->launches;
        int rc = enqueue_graph_step(m);
        cudaError_t e = cudaStreamEndCapture(ctx->stream, &g);
        if (rc != WB_OK) {
            if (g) cudaGraphDestroy(g);
            return rc;
        }
        WB_CUDA(e);
        ctx->launches = launches_before;  // capture enqueues nothing
        e = cudaGraphInstantiate(&m->graph, g, 0);
        cudaGraphDestroy(g);
        WB_CUDA(e);
        m->graph_stream = ctx->stream;
        m->graph_exact = m->exact;
    }
    const uint64_t per_step = m->graph_launches;  // kernels per replayed step, for wb_launch_count
    for (int64_t s = 0; s < n_steps; s++) WB_CUDA(cudaGraphLaunch(m->graph, ctx->stream));
    ctx->launches += per_step * (uint64_t)n_steps;
    // the sampled ids come back through pinned memory (a pageable destination would be staged by the driver)
    uint32_t *back = n_steps <= (int64_t)m->host_pin_cap ? m->host_pin : out_tokens;
    WB_CUDA(cudaMemcpyAsync(back, m->d_history, (size_t)n_steps * 4, cudaMemcpyDeviceToHost, ctx->stream));
    WB_CHECK(wb_synchronize(ctx));
    if (back != out_tokens) memcpy(out_tokens, back, (size_t)n_steps * 4);
    m->cache_len += n_steps;
    return WB_OK;
}

int wb_qwen_last_logits(wb_qwen *m, float *out)
{
    WB_MODEL(m);
    WB_NOT_RECORDING(m->ctx, "wb_qwen_last_logits");
    if (!out) return fail(WB_ERR_BAD_ARG, "out is NULL");
    WB_CUDA(cudaMemcpyAsync(out, m->dec.logits, (size_t)m->V * 4, cudaMemcpyDeviceToHost, m->ctx->stream));
    return wb_synchronize(m->ctx);
}

}  // extern "C"
