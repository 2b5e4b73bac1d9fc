// Internal layout of the Qwen2 model object (qwen_model.cu).
#pragma once
#include "qwen_ops.cuh"

namespace wbq {

struct LayerW {
    int in_norm = -1, post_norm = -1;
    int q = -1, k = -1, v = -1, o = -1, gate = -1, up = -1, down = -1;
    int qb = -1, kb = -1, vb = -1;
    int qkv = -1, qkvb = -1, gate_up = -1;  // fused variants
};

// Activation buffers of one forward call (all f32).
struct Bufs {
    uint32_t *tokens;
    float *x, *xa, *n, *q, *k, *v, *att, *proj, *gu, *act, *logits;
    __half *h16;  // fp16 copy of whichever activation feeds the next tensor-core GEMM ([M, max(C, I)]; M > 8 only)
    int ldq, ldk, ldv, ld_gu;
};

}  // namespace wbq

struct wb_qwen {
    wb_context *ctx = nullptr;
    wb_qwen_config cfg{};
    int C = 0, H = 0, KVH = 0, D = 0, KV = 0, I = 0, V = 0;
    int embed = -1, final_norm = -1;
    std::vector<wbq::LayerW> layers;
    char *k_cache = nullptr, *v_cache = nullptr;  // [n_layer][max_t][KV] of kv_dtype
    float *cs_table = nullptr;                    // [max_t][D/2][2] cos, sin
    int64_t cache_len = 0;
    int exact = 0;
    // device-resident decode state and M = 1 buffers (stable addresses for the captured graph)
    wbq::Bufs dec{};
    int *d_cache_len = nullptr, *d_step = nullptr, *d_bidx = nullptr;
    float *d_bval = nullptr, *att_scratch = nullptr;
    unsigned *att_counters = nullptr;
    uint32_t *host_pin = nullptr;  // pinned host buffer the sampled ids come back through
    size_t host_pin_cap = 0;
    uint32_t *d_history = nullptr;
    int64_t history_cap = 0;
    cudaGraphExec_t graph = nullptr;
    cudaStream_t graph_stream = nullptr;
    int graph_exact = -1;
    uint64_t graph_launches = 0;    // kernels in one captured decode step
    uint64_t carve_mark = 0, carve_top = 0;  // weight-arena `used` before and after the model's own allocations
};
