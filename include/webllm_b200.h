/*
 * webllm_b200 — C ABI of the B200 (sm_100a) implementation of webllm's quantized-linear path.
 *
 * This header is the whole drop-in boundary: plain pointers, sizes and integer handles, no C++ or
 * framework types. A TypeScript host binds it through N-API / FFI, a Python host through ctypes.
 * Each entry point names the function of the reference (intplusplus/webllm, TypeScript) whose job it
 * takes over.
 *
 * Conventions
 *   - Every function returns a wb_status (0 = ok, negative = error class). The text of the last error
 *     on the calling thread is wb_last_error(); where the reference throws with a message, the text
 *     is the reference's. Nothing throws or aborts across this boundary.
 *   - One context per GPU. Calls on one context are not re-entrant; different contexts may be driven
 *     from different threads.
 *   - Tensors are addressed as (arena, byte offset), offsets 256-byte aligned — the reference's Tensor
 *     {buffer, offset, length, shape} (src/gpu/buffer.ts:11-18, ALIGN = 256 at :3-9).
 *   - All device work is ordered on the context's stream (this replaces the reference's passBreak(),
 *     src/model/qwen.ts:551-559). wb_synchronize and wb_download are the only blocking calls.
 *   - Host pointers are borrowed for the duration of the call only.
 */
#ifndef WEBLLM_B200_H
#define WEBLLM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define WB_API __attribute__((visibility("default")))

typedef struct wb_context wb_context;
typedef struct wb_qwen wb_qwen;
typedef struct wb_batch wb_batch;
typedef int32_t wb_handle; /* index of a registered weight; < 0 = none */

typedef enum {
    WB_OK = 0,
    WB_ERR_BAD_ARG = -1,     /* validation failure (the reference's `throw new Error`) */
    WB_ERR_OOM = -2,         /* arena or device memory exhausted */
    WB_ERR_CUDA = -3,        /* a CUDA runtime / driver call failed */
    WB_ERR_NCCL = -4,
    WB_ERR_TIMEOUT = -5,     /* a bounded device-side wait ran out */
    WB_ERR_NOT_FOUND = -6,   /* unknown weight name ("缺少 f16 权重") */
    WB_ERR_EXISTS = -7,      /* duplicate weight name ("权重已存在") */
    WB_ERR_UNSUPPORTED = -8
} wb_status;

typedef enum { WB_F32 = 0, WB_F16 = 1 } wb_dtype;
typedef enum { WB_ARENA_WEIGHTS = 0, WB_ARENA_ACT = 1 } wb_arena;

/* Which kernel a linear call uses (see wb_plan_query). */
typedef enum {
    WB_KERNEL_GEMV_MMA = 1,   /* M <= 32: weights streamed once, register unpack, warp-level MMA, split-K. The planner's
                                 choice up to M = 8 (up to 12 / 16 with fp16 / f32 activations on short-K, wide-N shapes) */
    WB_KERNEL_GEMM_TC = 2,    /* tcgen05 / TMEM GEMM, TMA-fed, dequant in shared memory; f32 activations are rounded to
                                 fp16 first (as the reference's tiled GEMM stages them), never in exact mode */
    WB_KERNEL_GENERIC = 3,    /* shape-agnostic CUDA kernel for ragged sizes (K%8, N%4, group%32 != 0) */
    WB_KERNEL_DENSE_GEMV = 4, /* fp16 [N,K] weight, M <= 8 */
    WB_KERNEL_GEMV_STREAM = 5, /* M <= 4 on bandwidth-bound shapes (whole 128-k chunks, N % 32 == 0, >= 20 chunks per K
                                  slice): same arithmetic as GEMV_MMA, weights straight into registers, persistent CTAs */
    WB_KERNEL_GEMM_TC_PAIR = 6 /* the tcgen05 GEMM on CTA pairs (cta_group::2): GPTQ weights, M >= 128, N >= 256; each CTA
                                  of a pair unpacks 128 weight columns and loads half of the activation tile */
} wb_kernel_kind;

typedef struct {
    int32_t kernel;      /* wb_kernel_kind */
    int32_t split_k;     /* number of K slices (1 = unsplit); the planGemvSplit analogue */
    int32_t grid_x, grid_y, grid_z;
    int32_t block;       /* threads per block */
    int32_t tile_m, tile_n; /* GEMM_TC: tokens x output columns per CTA; otherwise 0 */
    int32_t launches;    /* kernels this call enqueues */
    uint64_t scratch_bytes; /* split-K partial sums / fp16 staging taken from the context workspace */
} wb_plan;

/* ---- library ---------------------------------------------------------------------------------- */
WB_API const char *wb_last_error(void);
WB_API int wb_version(void);

/* ---- context: one per GPU. Replaces initGpu (src/gpu/device.ts:40-98). ------------------------- */
WB_API int wb_context_create(int device, wb_context **out);
WB_API int wb_context_destroy(wb_context *ctx);
/* Use a caller-owned cudaStream_t (e.g. the host framework's current stream); NULL restores the
 * context's own stream. */
WB_API int wb_set_stream(wb_context *ctx, void *cuda_stream);
WB_API int wb_get_stream(wb_context *ctx, void **cuda_stream);
WB_API int wb_synchronize(wb_context *ctx);
/* Number of kernels this context has launched since creation (profilers rebuild the launch list from
 * wb_plan_query, as the reference's decode profiler does from planGemvSplit,
 * src/tests/perf/profile-decode.ts:55-82). */
WB_API int wb_launch_count(wb_context *ctx, uint64_t *count);

/* ---- arenas. Replaces Arena / alignTo (src/gpu/arena.ts:17-59, src/gpu/buffer.ts:3-9). ---------- */
/* One slab per arena, either allocated here or adopted from the caller (no copy, not freed here). */
WB_API int wb_arena_create(wb_context *ctx, int arena, uint64_t bytes);
WB_API int wb_arena_adopt(wb_context *ctx, int arena, void *device_ptr, uint64_t bytes);
/* Arena.allocFloat32 generalised to bytes: returns a 256-byte-aligned offset. */
WB_API int wb_arena_alloc(wb_context *ctx, int arena, uint64_t bytes, uint64_t *offset);
/* Arena.reset(): everything allocated since the last reset is recycled. The weight arena refuses
 * while weights are registered. */
WB_API int wb_arena_reset(wb_context *ctx, int arena);
WB_API int wb_arena_used(wb_context *ctx, int arena, uint64_t *used, uint64_t *capacity);
/* Partial reset: hands back everything allocated after the point where `used` was `mark`. */
WB_API int wb_arena_rewind(wb_context *ctx, int arena, uint64_t mark);
WB_API int wb_arena_base(wb_context *ctx, int arena, void **device_ptr);
/* queue.writeBuffer / readbackF32 (src/gpu/buffer.ts:37-52,123-145). */
WB_API int wb_upload(wb_context *ctx, int arena, uint64_t offset, const void *host, uint64_t bytes);
WB_API int wb_download(wb_context *ctx, int arena, uint64_t offset, void *host, uint64_t bytes);

/* ---- weights. Replaces QwenGpt.allocF16 / writeF16Chunk / uploadF16 / uploadF32
 *      (src/model/qwen.ts:247-276) and the GPTQ half of loadQwenWeights
 *      (src/weights/qwen-loader.ts:55-67). Names are the reference's ("L3.qW", "embed", ...). ------- */

/* Takes the three GPTQ tensors as they sit in the checkpoint and keeps them packed on the device:
 *   qweight  bytes of I32 [ceil(K/8), N]    nibble j of word [r,n] = input channel 8r+j
 *   qzeros   bytes of I32 [ceil(K/g), ceil(N/8)] or NULL (symmetric, zero point 8); stored value is zero-1
 *   scales   fp16 bits [ceil(K/g), N]
 * Validates exactly what dequantizeGptqInt4 validates (src/weights/quant.ts:46-79): bits == 4,
 * group > 0, in/out > 0, byte lengths, group % 8 == 0. */
WB_API int wb_gptq_register(wb_context *ctx, const char *name, const void *qweight, uint64_t qweight_bytes,
                            const void *qzeros, uint64_t qzeros_bytes, const uint16_t *scales_f16,
                            uint64_t scales_len, int64_t in_features, int64_t out_features, int64_t group_size,
                            int bits, wb_handle *out);
/* Registers the column slice [col_begin, col_begin+col_count) of a GPTQ linear (output-column
 * sharding across GPUs). col_begin and col_count must be multiples of 8 so no zero word is split.
 * No counterpart in the reference, which has one device. */
WB_API int wb_gptq_register_cols(wb_context *ctx, const char *name, const void *qweight, uint64_t qweight_bytes,
                                 const void *qzeros, uint64_t qzeros_bytes, const uint16_t *scales_f16,
                                 uint64_t scales_len, int64_t in_features, int64_t out_features,
                                 int64_t group_size, int bits, int64_t col_begin, int64_t col_count,
                                 wb_handle *out);
/* allocF16(name, length) with the logical shape [rows, cols] (rows*cols == length). */
WB_API int wb_f16_alloc(wb_context *ctx, const char *name, int64_t rows, int64_t cols, wb_handle *out);
/* writeF16Chunk: f32 -> fp16 round-to-nearest-even with the reference's edge rules
 * (f32ToF16Bits, src/gpu/buffer.ts:57-100: NaN -> 0x7e00, |x| < 2^-24 -> +-0). */
WB_API int wb_f16_write_chunk(wb_context *ctx, wb_handle h, int64_t elem_offset, const float *data, int64_t n);
/* Same, from fp16 bits as stored in a safetensors file (no f32 round trip). */
WB_API int wb_f16_write_bits(wb_context *ctx, wb_handle h, int64_t elem_offset, const uint16_t *bits, int64_t n);
/* uploadF32(name, data): norm weights and biases. */
WB_API int wb_f32_upload(wb_context *ctx, const char *name, const float *data, int64_t n, wb_handle *out);
WB_API int wb_weight_lookup(wb_context *ctx, const char *name, wb_handle *out);
/* Drops the most recently registered weight and returns its arena space (stack order). Lets a host
 * implement the pure function dequantizeGptqInt4(params) -> array as register / export / pop. */
WB_API int wb_weight_pop(wb_context *ctx);
/* readWeightF16Bytes (src/model/qwen.ts:527-531): raw fp16 bits of a dense fp16 weight. */
WB_API int wb_read_weight_f16(wb_context *ctx, wb_handle h, int64_t elem_offset, int64_t n, uint16_t *out_bits);
/* weightBytes (src/model/qwen.ts:222-242): device bytes held by registered weights. */
WB_API int wb_weight_bytes(wb_context *ctx, uint64_t *bytes);

/* ---- dequant export. Replaces dequantizeGptqInt4 (src/weights/quant.ts:42-118) and its fp16 device
 *      copy (writeF16, src/gpu/buffer.ts:103-120). Output [N, K] row-major in the activation arena:
 *      f32 equal to the reference's Float32Array bit for bit, fp16 equal to f32ToF16Bits of it. ---- */
WB_API int wb_gptq_dequant_f32(wb_context *ctx, wb_handle h, uint64_t out_offset);
WB_API int wb_gptq_dequant_f16(wb_context *ctx, wb_handle h, uint64_t out_offset);

/* ---- linear. Replaces QwenGpt.gemm (src/model/qwen.ts:568-618) and the four WGSL kernels behind it
 *      (gemm_gemv_f16, gemm_gemv_split_f16, gemm_gemv_split_reduce, gemm_nt_f16_from_f32).
 *      C[M,N] = A[M,K] . W[N,K]^T (+ bias[N]); A at a_offset and C at c_offset in the activation
 *      arena, row-major, dense; bias is an f32 weight handle or -1 and is added once, after the full-K
 *      sum. act_dtype / out_dtype are wb_dtype. `exact` != 0 asks for the fp32-activation mode: f32
 *      activations keep ~22 bits through the tensor-core paths (hi/lo split) instead of being rounded
 *      to fp16 as the reference's tiled GEMM does (gemm_nt_f16_from_f32.wgsl:58-62). ---------------- */
WB_API int wb_linear(wb_context *ctx, wb_handle weight, uint64_t a_offset, uint64_t c_offset, wb_handle bias,
                     int64_t M, int act_dtype, int out_dtype, int exact);
/* ---- output-column shards over several GPUs, one process and one context per GPU. No counterpart in the
 *      reference, which has one device; the call keeps QwenGpt.gemm's meaning (src/model/qwen.ts:568-618) for the
 *      full [M, n_total] result. `weight` holds this GPU's columns [col_begin, col_begin + N) of the full matrix
 *      (wb_gptq_register_cols). The product is stored at those columns of the [M, n_total] row-major tensor at
 *      c_offset in this context's activation slab AND at the same offset in every peer slab: the all-gather is
 *      the kernel's own stores over NVLink, issued tile by tile by the tensor-core kernel while other tiles are
 *      still being multiplied (decode-size calls write a dense piece to the scratch tensor at tmp_offset,
 *      [M, N], and one small launch spreads it). The call is stream-ordered like wb_linear and does NOT wait for
 *      the peers: before any rank reads its full tensor, every rank's call must have completed (a barrier across
 *      the ranks after the call: wb_peer_barrier below, or any collective on the same streams), and no rank may still
 *      be reading the tensor when the next call writes it.
 *      wb_arena_ipc_export writes WB_IPC_HANDLE_BYTES bytes that another process on the same node passes to
 *      wb_peer_open to map this context's slab (only a slab made by wb_arena_create); wb_peer_close unmaps it. */
#define WB_IPC_HANDLE_BYTES 64
WB_API int wb_linear_gather(wb_context *ctx, wb_handle weight, uint64_t a_offset, uint64_t c_offset, uint64_t tmp_offset,
                            wb_handle bias, int64_t M, int act_dtype, int out_dtype, int64_t n_total,
                            int64_t col_begin, void *const *peer_bases, int n_peers);
WB_API int wb_arena_ipc_export(wb_context *ctx, int arena, void *handle_out);
WB_API int wb_peer_open(wb_context *ctx, const void *handle, void **base_out);
WB_API int wb_peer_close(wb_context *ctx, void *base);
/* The barrier that wb_linear_gather needs, done by a kernel of this library instead of a collective (no counterpart in
 * the reference). `flags_offset` names WB_PEER_FLAG_BYTES bytes of the activation slab, the same offset on every rank;
 * `rank` is this process's index among the n_peers + 1 ranks. wb_peer_barrier_init zeroes the flags and the epoch
 * counter kept beside them on the device: every rank calls it once, and the ranks must meet on the host (any host-side
 * barrier) between the last init and the first wb_peer_barrier. wb_peer_barrier is stream-ordered: the kernel stores an increasing epoch word
 * into slot `rank` of every peer's flags (behind a system-scope fence, so everything this stream stored into the peers
 * before it is visible first) and waits until every other slot of its own flags has reached the epoch. The wait is
 * bounded: after timeout_us (0 = 2 s) the kernel records a code and returns, and the next wb_synchronize / wb_download
 * returns WB_ERR_TIMEOUT; nothing hangs when a peer never arrives. Every rank must issue the same sequence of barriers.
 * Both calls may be recorded into a command batch (the epoch advances on the device with every replay).
 * wb_linear_gather_barrier is wb_linear_gather followed by that barrier; for decode-size calls the copy into the peers
 * and the barrier are one launch. */
#define WB_PEER_FLAG_BYTES 256
WB_API int wb_peer_barrier_init(wb_context *ctx, uint64_t flags_offset);
WB_API int wb_peer_barrier(wb_context *ctx, uint64_t flags_offset, int rank, void *const *peer_bases, int n_peers,
                           uint32_t timeout_us);
WB_API int wb_linear_gather_barrier(wb_context *ctx, wb_handle weight, uint64_t a_offset, uint64_t c_offset,
                                    uint64_t tmp_offset, wb_handle bias, int64_t M, int act_dtype, int out_dtype,
                                    int64_t n_total, int64_t col_begin, void *const *peer_bases, int n_peers,
                                    uint64_t flags_offset, int rank, uint32_t timeout_us);
/* The same exchange as an NCCL all-gather over NVLink (no counterpart in the reference). NCCL is loaded with dlopen
 * when one of these is first called (WEBLLM_B200_NCCL_LIB names the file, else libnccl.so.2), so the library links
 * only the CUDA runtime. wb_comm_unique_id fills WB_COMM_ID_BYTES bytes on one rank; the host hands them to the
 * others (any channel) and every rank calls wb_comm_init(rank, nranks, id). Creation is polled on the host for at most
 * timeout_ms (<= 0: 30 s): if a rank never joins, the others get WB_ERR_TIMEOUT and the half-built communicator is
 * aborted. wb_linear_colshard: `weight` holds this rank's N columns (wb_gptq_register_cols, equal widths on all
 * ranks); the local [M, N] product goes to scratch_offset, the all-gather of the pieces to c_offset as rank-major
 * [nranks, M, N] (for M == 1 that IS the row [1, nranks * N]); with row_major != 0 and M > 1 the pieces are gathered
 * into the scratch and a kernel of this library rearranges them to row-major [M, nranks * N] at c_offset. Scratch
 * size: align256(M * N * elem) bytes, plus nranks * M * N * elem when rearranging. Stream-ordered like wb_linear;
 * cannot be recorded into a command batch. */
#define WB_COMM_ID_BYTES 128
WB_API int wb_comm_unique_id(void *id_out);
WB_API int wb_comm_init(wb_context *ctx, int rank, int nranks, const void *unique_id, int timeout_ms);
WB_API int wb_comm_destroy(wb_context *ctx);
WB_API int wb_linear_colshard(wb_context *ctx, wb_handle weight, uint64_t a_offset, uint64_t c_offset,
                              uint64_t scratch_offset, wb_handle bias, int64_t M, int act_dtype, int out_dtype,
                              int row_major);
/* Diagnostic with no counterpart in the reference: one kernel of `ctas` x 256 threads reads `bytes` of a slab once
 * (128-bit streaming loads) and computes nothing. It measures the rate that any single pass over that many bytes
 * reaches when launched like the int4 GEMV, the figure that kernel's bandwidth is compared with. */
WB_API int wb_read_sweep(wb_context *ctx, int arena, uint64_t offset, uint64_t bytes, int ctas);
/* planGemvSplit (src/model/qwen.ts:61-74) generalised: which kernel, how many K slices, what grid. */
WB_API int wb_plan_query(wb_context *ctx, wb_handle weight, int64_t M, int act_dtype, int exact, wb_plan *out);
/* Forces a kernel (wb_kernel_kind) and/or split for the next wb_linear calls; 0 = planner's choice. A forced kind
 * means that kernel and no other (WB_KERNEL_GEMV_MMA never falls through to GEMV_STREAM and vice versa; a shape or split
 * the kernel does not take is refused with WB_ERR_UNSUPPORTED).
 * Used by tests to cover every path at every shape, as the reference's tests drive the split kernel with
 * explicit S (src/tests/kernels.ts:1378-1400). */
WB_API int wb_plan_override(wb_context *ctx, int kernel, int split_k);
/* Tells the next wb_linear call which weight a LATER call will stream (< 0 = none): a decode-size call (the int4
 * GEMV) then also asks the L2 to fetch that weight (up to 32 MiB of it) while it runs, so the later call finds its
 * first chunks in L2 instead of paying the HBM latency on its critical path. The hint is consumed by the next
 * wb_linear whatever kernel it picks; results never depend on it. No counterpart in the reference (WebGPU offers
 * no cache control); the Qwen decode step sets it for its own sequence of projections. */
WB_API int wb_linear_hint_next(wb_context *ctx, wb_handle next_weight);

/* ---- command batches. Replaces CommandBatch (src/gpu/pipeline.ts:55-117): every wb_linear /
 *      wb_gptq_dequant call between begin and end is recorded instead of run; wb_batch_submit enqueues
 *      the whole recording in one go and may be repeated. Transfers and wb_synchronize are not allowed
 *      while recording. Offsets and handles are baked in: keep the tensors alive while the batch is. ---- */
WB_API int wb_batch_begin(wb_context *ctx);
WB_API int wb_batch_end(wb_context *ctx, wb_batch **out);
WB_API int wb_batch_submit(wb_batch *batch);
WB_API int wb_batch_destroy(wb_batch *batch);

/* ---- Qwen2 forward. Replaces QwenGpt (src/model/qwen.ts:124-531) for the quantized-linear path and the
 *      decode loop of generateQwen (src/infer/qwen-generate.ts:29-84). Weights are looked up by the
 *      reference's names: "embed" (fp16 [V,C], tied lm_head), "finalNorm", and per layer i "L{i}.inNorm",
 *      "L{i}.postNorm" (f32), "L{i}.qW/kW/vW/oW/gateW/upW/downW" (GPTQ or dense fp16), "L{i}.qB/kB/vB" (f32).
 *      A layer may instead provide the fused projections "L{i}.qkvW" (+ "L{i}.qkvB") and "L{i}.gateUpW"
 *      (output columns concatenated), which the reference already runs in shared passes
 *      (src/model/qwen.ts:407-414,462-466). ---------------------------------------------------------- */
typedef struct {
    int32_t vocab_size, n_layer, n_head, n_kv_head, n_embd, intermediate; /* QwenConfig, src/model/qwen-config.ts:12-28 */
    int32_t max_t;    /* context limit = KV cache rows (the reference's blockSize) */
    int32_t kv_dtype; /* WB_F32 (the reference's cache, src/model/qwen.ts:200-205) or WB_F16 */
    float rms_eps, rope_theta;
} wb_qwen_config;

WB_API int wb_qwen_create(wb_context *ctx, const wb_qwen_config *cfg, wb_qwen **out);
WB_API int wb_qwen_destroy(wb_qwen *model);
/* resetCache() */
WB_API int wb_qwen_reset_cache(wb_qwen *model);
WB_API int wb_qwen_cache_len(wb_qwen *model, int64_t *len);
/* `exact` != 0: fp32-activation mode for every linear (see wb_linear). */
WB_API int wb_qwen_set_exact(wb_qwen *model, int exact);
/* forward(tokens, B, T): no KV cache, logits [B*T, V] f32 at *logits_offset in the activation arena
 * (the arena is reset first, as runForward does, src/model/qwen.ts:359). */
WB_API int wb_qwen_forward(wb_qwen *model, const uint32_t *tokens, int64_t B, int64_t T, uint64_t *logits_offset);
/* prefill(tokens): fills the cache; last_only != 0 computes only the last row of logits ([1, V]),
 * which is all generateQwen reads (src/infer/qwen-generate.ts:53-57); else [n, V]. */
WB_API int wb_qwen_prefill(wb_qwen *model, const uint32_t *tokens, int64_t n, int last_only, uint64_t *logits_offset);
/* decodeStep(token): logits [1, V]. */
WB_API int wb_qwen_decode_step(wb_qwen *model, uint32_t token, uint64_t *logits_offset);
/* Greedy decoding kept on the device: feeds `first_token`, then n_steps times (forward one token, argmax
 * with the reference's first-strict-maximum rule, src/infer/sampler.ts:30-36, append). The step is captured
 * in a CUDA graph on first use and replayed; out_tokens receives the n_steps sampled tokens. Replaces the
 * per-token logits readback of generateQwen (src/infer/qwen-generate.ts:66-74). */
WB_API int wb_qwen_decode_greedy(wb_qwen *model, uint32_t first_token, int64_t n_steps, uint32_t *out_tokens);
/* Logits of the last step run by wb_qwen_decode_greedy, [V] f32, copied to the host. */
WB_API int wb_qwen_last_logits(wb_qwen *model, float *out);

/* ---- allocation-free GEMV. No counterpart in the reference (its split-K scratch comes from the arena,
 *      src/model/qwen.ts:584); added for hosts that may not allocate device memory where they run the
 *      kernel: a real-time loop or driver callback where the allocator is off limits, a sandboxed plugin
 *      that was handed its buffers up front, an application that owns every byte of the GPU and passes a
 *      plugin only input and output pointers. It needs no context and calls no cudaMalloc / cudaFree or
 *      any allocating routine: the split-K partial sums and arrival counters live in a 4 MiB + 16 KiB
 *      array inside the library image (held by every GPU that loads the library until the process exits).
 *
 *      y[M,N] = x[M,K] . W[N,K]^T (+ bias) for one GPTQ linear given as raw DEVICE pointers in the
 *      checkpoint layout (see wb_gptq_register; qzeros and bias may be NULL), on the current device and the
 *      given cudaStream_t (NULL = default stream). split_k <= 0 picks a split automatically.
 *      Limits: M <= 32, K % 8 == 0, N % 4 == 0, group % 128 == 0, N <= 131072 * (1, 2 or 4 for M <= 2, 4, 32),
 *      and split_k * M * N * 4 bytes <= 4 MiB; anything beyond is refused with WB_ERR_UNSUPPORTED and a
 *      message, never truncated.
 *      Alignment of the caller's pointers (a view into the middle of a larger buffer may break it): qweight, x and
 *      y 16 bytes, scales_f16 8 bytes, qzeros and bias 4 bytes; anything else is refused with WB_ERR_BAD_ARG
 *      before any launch. The kernel is ordered behind everything enqueued earlier on the stream (it is launched
 *      without programmatic stream serialization), so a kernel of the caller that writes the tensors may
 *      directly precede the call.
 *      The first call on a device looks up the array's device address (cudaGetSymbolAddress): make that
 *      call before any stream capture. All calls on a device share the array, which keeps the previous
 *      call's contents; each call re-zeroes the counters it uses on its stream, so calls that run one after
 *      another are safe, while calls that overlap on the GPU (different streams) race on it. ------------ */
WB_API int wb_gptq_gemv_static(const void *qweight, const void *qzeros, const void *scales_f16, const void *x, void *y,
                               const float *bias, int64_t in_features, int64_t out_features, int64_t group_size,
                               int64_t M, int act_dtype, int out_dtype, int split_k, void *cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* WEBLLM_B200_H */
