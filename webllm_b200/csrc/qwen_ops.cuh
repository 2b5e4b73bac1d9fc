// Host entry points of the non-linear Qwen2 forward steps (qwen_ops.cu).
#pragma once
#include "common.cuh"

namespace wb {

int op_embed(wb_context *ctx, const __half *table, const uint32_t *tokens, float *x, int M, int C, int vocab);
// y = rmsnorm(x + delta) * w; when delta != nullptr the sum is also stored to x_out (residual stream).
// y16 != nullptr: y is not written, the result goes to y16 as fp16 (input of a tensor-core GEMM).
int op_rmsnorm(wb_context *ctx, const float *x, const float *delta, float *x_out, const float *w, float *y, int M, int D, float eps,
               __half *y16 = nullptr);
int op_add(wb_context *ctx, const float *a, const float *b, float *out, int64_t n);
int op_silu_mul(wb_context *ctx, const float *gate, const float *up, float *out, int M, int I, int ld, __half *out16 = nullptr);
// Rotates q in place and k (into the cache when k_cache != nullptr, else in place); copies v to the cache.
// The position offset is read from pos_ptr when it is not null (graph replay), else pos_imm.
int op_rope_kv(wb_context *ctx, float *q, float *k, const float *v, void *k_cache, void *v_cache, int kv_f16,
               const float *cs_table, int M, int H, int KVH, int D, int T, const int *pos_ptr, int pos_imm, int ldq,
               int ldk, int ldv);
int op_attention(wb_context *ctx, const float *q, const void *kmem, const void *vmem, int kv_f16, float *out, int M, int H,
                 int KVH, int D, int T, const int *past_ptr, int past_imm, int use_cache, int max_keys, int ldq, int kv_ld);
// The same for M >= 16 rows against the KV cache on the tensor cores (attention_prefill.cu): fp16 operands, f32 softmax
// and accumulation; head size 64 or 128. Used by the default mode; the fp32-activation mode keeps op_attention.
bool op_attention_prefill_supported(int M, int H, int KVH, int D, int ldq, int kv_ld);
int op_attention_prefill(wb_context *ctx, const float *q, const void *kmem, const void *vmem, int kv_f16, float *out, int M, int H,
                         int KVH, int D, const int *past_ptr, int past_imm, int ldq, int kv_ld, __half *out16 = nullptr);
// One query row against the cache, keys split over several CTAs per head; scratch holds the per-slice
// softmax state (op_attention_decode_scratch_floats floats), counters one zeroed word per head.
// With k_raw / v_raw / cs_table set, q, k_raw and v_raw are the un-rotated projection outputs: the kernel applies the
// rotary embedding and appends the new key and value to the cache itself (no op_rope_kv before it). early_kv: the kernel
// reads the cache and the position before it waits for the kernel in front of it (see the kernel).
int op_attention_decode(wb_context *ctx, const float *q, void *kmem, void *vmem, int kv_f16, float *out, float *scratch,
                        unsigned *counters, int H, int KVH, int D, const int *past_ptr, int past_imm, int max_keys, int kv_ld,
                        const float *k_raw = nullptr, const float *v_raw = nullptr, const float *cs_table = nullptr,
                        int early_kv = 0);
int op_attention_decode_scratch_floats(int H, int D);
// Dynamic shared memory of the decode attention kernel for up to max_keys keys (it stages a split's V rows).
size_t op_attention_decode_smem(int D, int max_keys, int kv_f16);
int op_argmax(wb_context *ctx, const float *logits, int V, float *bval, int *bidx, uint32_t *token_out, uint32_t *history,
              int *step_counter, int *cache_len);

}  // namespace wb
