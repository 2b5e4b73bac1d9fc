// Context, arenas, weight registry and host<->device transfers behind the C ABI.
#include <cuda.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "common.cuh"

namespace wb {

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
}

int fail(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
    return code;
}

int check_range(wb_context *ctx, int arena, uint64_t off, uint64_t bytes, const char *what)
{
    if (arena != WB_ARENA_WEIGHTS && arena != WB_ARENA_ACT) return fail(WB_ERR_BAD_ARG, "%s: bad arena %d", what, arena);
    const ArenaState &a = ctx->arena[arena];
    if (!a.base) return fail(WB_ERR_BAD_ARG, "%s: arena %d has no slab", what, arena);
    if (off > a.capacity || bytes > a.capacity - off)
        return fail(WB_ERR_BAD_ARG, "%s: range [%llu, +%llu) outside arena of %llu bytes", what,
                    (unsigned long long)off, (unsigned long long)bytes, (unsigned long long)a.capacity);
    return WB_OK;
}

int get_weight(wb_context *ctx, wb_handle h, Weight **out)
{
    if (h < 0 || (size_t)h >= ctx->weights.size()) return fail(WB_ERR_NOT_FOUND, "bad weight handle %d", h);
    *out = &ctx->weights[h];
    return WB_OK;
}

static int arena_alloc(wb_context *ctx, int arena, uint64_t bytes, uint64_t *off)
{
    ArenaState &a = ctx->arena[arena];
    if (!a.base) return fail(WB_ERR_BAD_ARG, "arena %d has no slab (call wb_arena_create first)", arena);
    uint64_t need = align_up(bytes ? bytes : 4);
    if (need > a.capacity - a.used)
        return fail(WB_ERR_OOM, "arena %d exhausted: need %llu, free %llu", arena, (unsigned long long)need,
                    (unsigned long long)(a.capacity - a.used));
    *off = a.used;
    a.used += need;
    return WB_OK;
}

static int add_weight(wb_context *ctx, Weight &&w, wb_handle *out)
{
    int idx = (int)ctx->weights.size();
    w.arena_top = ctx->arena[WB_ARENA_WEIGHTS].used;
    ctx->by_name[w.name] = idx;
    ctx->weights.push_back(std::move(w));
    if (out) *out = idx;
    return WB_OK;
}

static int check_new_name(wb_context *ctx, const char *name)
{
    if (!name || !*name) return fail(WB_ERR_BAD_ARG, "weight name is empty");
    if (ctx->by_name.count(name)) return fail(WB_ERR_EXISTS, "权重已存在: %s", name);
    return WB_OK;
}

__global__ void f32_to_f16_ref_kernel(const float *__restrict__ in, unsigned short *__restrict__ out, int64_t n)
{
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) out[i] = f32_to_f16_bits_ref(in[i]);
}

int launch_f32_to_f16_ref(wb_context *ctx, const float *in, __half *out, int64_t n)
{
    if (n <= 0) return WB_OK;
    int blocks = (int)((n + 255) / 256);
    if (blocks > ctx->sm_count * 16) blocks = ctx->sm_count * 16;
    f32_to_f16_ref_kernel<<<blocks, 256, 0, ctx->stream>>>(in, (unsigned short *)out, n);
    ctx->launches++;
    WB_CUDA(cudaGetLastError());
    return WB_OK;
}

}  // namespace wb

using namespace wb;

#define WB_CTX(ctx)                                                        \
    do {                                                                   \
        if (!(ctx)) return wb::fail(WB_ERR_BAD_ARG, "context is NULL");   \
        WB_CUDA(cudaSetDevice((ctx)->device));                             \
    } while (0)

namespace wb {
// Reads a byte range once and does nothing else (an XOR that is never stored): the rate that ANY single pass over that
// many bytes can reach when launched like the GEMV, which is what its roofline fraction is read against.
__global__ void __launch_bounds__(256) read_sweep_kernel(const uint4 *__restrict__ src, size_t n16, uint32_t *sink)
{
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint32_t acc = 0;
    for (; i + 3 * stride < n16; i += 4 * stride) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; u++) v[u] = ldg_stream_v4(reinterpret_cast<const uint32_t *>(src + i + u * stride));
#pragma unroll
        for (int u = 0; u < 4; u++) acc ^= v[u].x ^ v[u].y ^ v[u].z ^ v[u].w;
    }
    for (; i < n16; i += stride) {
        const uint4 v = ldg_stream_v4(reinterpret_cast<const uint32_t *>(src + i));
        acc ^= v.x ^ v.y ^ v.z ^ v.w;
    }
    if (acc == 0x9e3779b9u) *sink = acc;  // keeps the loads alive; practically never true
}
}  // namespace wb

extern "C" {

const char *wb_last_error(void) { return g_error; }
int wb_version(void) { return 100; }

int wb_context_create(int device, wb_context **out)
{
    if (!out) return fail(WB_ERR_BAD_ARG, "out is NULL");
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return fail(WB_ERR_CUDA, "no CUDA device is visible (%s); this library has no CPU path",
                    cudaGetErrorString(e));
    if (device < 0 || device >= count) return fail(WB_ERR_BAD_ARG, "device %d out of range (0..%d)", device, count - 1);
    WB_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    WB_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(WB_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", device,
                    prop.major, prop.minor);
    wb_context *ctx = new wb_context();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    const int rc = [&]() -> int {
        WB_CUDA(cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking));
        ctx->stream = ctx->own_stream;
        WB_CUDA(cudaMalloc(&ctx->workspace, kWorkspaceBytes));
        WB_CUDA(cudaMalloc(&ctx->counters, kMaxCounters * sizeof(unsigned)));
        WB_CUDA(cudaMemset(ctx->counters, 0, kMaxCounters * sizeof(unsigned)));
        WB_CUDA(cudaHostAlloc(&ctx->status_host, sizeof(int), cudaHostAllocMapped));
        *ctx->status_host = 0;
        WB_CUDA(cudaHostGetDevicePointer(&ctx->status_word, ctx->status_host, 0));
        cudaDriverEntryPointQueryResult qres;
        WB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ctx->tmap_encode, cudaEnableDefault, &qres));
        if (qres != cudaDriverEntryPointSuccess || !ctx->tmap_encode)
            return fail(WB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
        return WB_OK;
    }();
    if (rc != WB_OK) {
        wb_context_destroy(ctx);  // frees whatever was built; keeps the error text
        return rc;
    }
    *out = ctx;
    return WB_OK;
}

int wb_context_destroy(wb_context *ctx)
{
    if (!ctx) return WB_OK;
    cudaSetDevice(ctx->device);
    if (ctx->stream) cudaStreamSynchronize(ctx->stream);
    comm_release(ctx);
    for (int i = 0; i < 2; i++)
        if (ctx->arena[i].owned && ctx->arena[i].base) cudaFree(ctx->arena[i].base);
    if (ctx->workspace) cudaFree(ctx->workspace);
    if (ctx->counters) cudaFree(ctx->counters);
    if (ctx->status_host) cudaFreeHost(ctx->status_host);
    if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
    delete ctx;
    return WB_OK;
}

int wb_set_stream(wb_context *ctx, void *cuda_stream)
{
    WB_CTX(ctx);
    ctx->stream = cuda_stream ? (cudaStream_t)cuda_stream : ctx->own_stream;
    return WB_OK;
}

int wb_get_stream(wb_context *ctx, void **cuda_stream)
{
    WB_CTX(ctx);
    *cuda_stream = (void *)ctx->stream;
    return WB_OK;
}

int wb_synchronize(wb_context *ctx)
{
    WB_CTX(ctx);
    WB_NOT_RECORDING(ctx, "wb_synchronize");
    WB_CUDA(cudaStreamSynchronize(ctx->stream));
    if (*ctx->status_host != 0) {
        int code = *ctx->status_host;
        *ctx->status_host = 0;
        return fail(WB_ERR_TIMEOUT, "a device-side bounded wait gave up (code %d)", code);
    }
    return WB_OK;
}

int wb_launch_count(wb_context *ctx, uint64_t *count)
{
    WB_CTX(ctx);
    *count = ctx->launches;
    return WB_OK;
}

// ------------------------------------------------------------------ arenas

int wb_arena_create(wb_context *ctx, int arena, uint64_t bytes)
{
    WB_CTX(ctx);
    if (arena != 0 && arena != 1) return fail(WB_ERR_BAD_ARG, "bad arena %d", arena);
    if (ctx->arena[arena].base) return fail(WB_ERR_EXISTS, "arena %d already has a slab", arena);
    uint64_t cap = align_up(bytes ? bytes : kAlign);
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, cap);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(WB_ERR_OOM, "cudaMalloc(%llu) failed: %s", (unsigned long long)cap, cudaGetErrorString(e));
    }
    ctx->arena[arena] = {(char *)p, cap, 0, true};
    return WB_OK;
}

int wb_arena_adopt(wb_context *ctx, int arena, void *device_ptr, uint64_t bytes)
{
    WB_CTX(ctx);
    if (arena != 0 && arena != 1) return fail(WB_ERR_BAD_ARG, "bad arena %d", arena);
    if (ctx->arena[arena].base) return fail(WB_ERR_EXISTS, "arena %d already has a slab", arena);
    if (!device_ptr || ((uintptr_t)device_ptr % kAlign) != 0)
        return fail(WB_ERR_BAD_ARG, "adopted slab must be a non-NULL, 256-byte aligned device pointer");
    ctx->arena[arena] = {(char *)device_ptr, bytes / kAlign * kAlign, 0, false};
    return WB_OK;
}

int wb_arena_alloc(wb_context *ctx, int arena, uint64_t bytes, uint64_t *offset)
{
    WB_CTX(ctx);
    if (arena != 0 && arena != 1) return fail(WB_ERR_BAD_ARG, "bad arena %d", arena);
    if (!offset) return fail(WB_ERR_BAD_ARG, "offset is NULL");
    return arena_alloc(ctx, arena, bytes, offset);
}

int wb_arena_reset(wb_context *ctx, int arena)
{
    WB_CTX(ctx);
    if (arena != 0 && arena != 1) return fail(WB_ERR_BAD_ARG, "bad arena %d", arena);
    if (arena == WB_ARENA_WEIGHTS && !ctx->weights.empty())
        return fail(WB_ERR_BAD_ARG, "weight arena holds %zu registered weights; destroy the context to drop them",
                    ctx->weights.size());
    ctx->arena[arena].used = 0;
    return WB_OK;
}

int wb_arena_used(wb_context *ctx, int arena, uint64_t *used, uint64_t *capacity)
{
    WB_CTX(ctx);
    if (arena != 0 && arena != 1) return fail(WB_ERR_BAD_ARG, "bad arena %d", arena);
    if (used) *used = ctx->arena[arena].used;
    if (capacity) *capacity = ctx->arena[arena].capacity;
    return WB_OK;
}

int wb_arena_rewind(wb_context *ctx, int arena, uint64_t mark)
{
    WB_CTX(ctx);
    if (arena != WB_ARENA_ACT) return fail(WB_ERR_BAD_ARG, "only the activation arena can be rewound");
    if (mark > ctx->arena[arena].used || mark % kAlign)
        return fail(WB_ERR_BAD_ARG, "wb_arena_rewind: mark %llu is not an earlier allocation point", (unsigned long long)mark);
    ctx->arena[arena].used = mark;
    return WB_OK;
}

int wb_arena_base(wb_context *ctx, int arena, void **device_ptr)
{
    WB_CTX(ctx);
    if (arena != 0 && arena != 1) return fail(WB_ERR_BAD_ARG, "bad arena %d", arena);
    *device_ptr = ctx->arena[arena].base;
    return WB_OK;
}

int wb_upload(wb_context *ctx, int arena, uint64_t offset, const void *host, uint64_t bytes)
{
    WB_CTX(ctx);
    WB_NOT_RECORDING(ctx, "wb_upload");
    WB_CHECK(check_range(ctx, arena, offset, bytes, "wb_upload"));
    if (bytes == 0) return WB_OK;
    if (!host) return fail(WB_ERR_BAD_ARG, "wb_upload: host pointer is NULL");
    WB_CUDA(cudaMemcpyAsync(arena_ptr(ctx, arena, offset), host, bytes, cudaMemcpyHostToDevice, ctx->stream));
    // The host buffer is borrowed for the call only: pageable copies are already staged when
    // cudaMemcpyAsync returns; pinned ones are not, so wait.
    WB_CUDA(cudaStreamSynchronize(ctx->stream));
    return WB_OK;
}

int wb_download(wb_context *ctx, int arena, uint64_t offset, void *host, uint64_t bytes)
{
    WB_CTX(ctx);
    WB_NOT_RECORDING(ctx, "wb_download");
    WB_CHECK(check_range(ctx, arena, offset, bytes, "wb_download"));
    if (bytes == 0) return WB_OK;
    if (!host) return fail(WB_ERR_BAD_ARG, "wb_download: host pointer is NULL");
    WB_CUDA(cudaMemcpyAsync(host, arena_ptr(ctx, arena, offset), bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return wb_synchronize(ctx);
}

// ------------------------------------------------------------------ weights

static int gptq_register_impl(wb_context *ctx, const char *name, const void *qweight, uint64_t qweight_bytes,
                              const void *qzeros, uint64_t qzeros_bytes, const uint16_t *scales, uint64_t scales_len,
                              int64_t inF, int64_t outF, int64_t group, int bits, int64_t col_begin,
                              int64_t col_count, wb_handle *out)
{
    WB_NOT_RECORDING(ctx, "wb_gptq_register");
    WB_CHECK(check_new_name(ctx, name));
    // The validation list and message texts of dequantizeGptqInt4 (src/weights/quant.ts:46-79).
    if (bits != 4) return fail(WB_ERR_BAD_ARG, "GPTQ: 当前仅支持 4bit，收到 bits=%d", bits);
    if (group <= 0) return fail(WB_ERR_BAD_ARG, "GPTQ: groupSize 必须为正");
    if (inF <= 0 || outF <= 0) return fail(WB_ERR_BAD_ARG, "GPTQ: in/out 必须为正");
    const int64_t pack = 8;
    const int64_t pack_rows = (inF + pack - 1) / pack;
    const int64_t pack_cols = (outF + pack - 1) / pack;
    const int64_t groups = (inF + group - 1) / group;
    if (!qweight || (int64_t)qweight_bytes < pack_rows * outF * 4)
        return fail(WB_ERR_BAD_ARG, "GPTQ: qweight 字节不足，需要 %lld，实际 %lld", (long long)(pack_rows * outF * 4),
                    (long long)qweight_bytes);
    if (!scales || (int64_t)scales_len < groups * outF)
        return fail(WB_ERR_BAD_ARG, "GPTQ: scales 数量不足，需要 %lld，实际 %lld", (long long)(groups * outF),
                    (long long)scales_len);
    if (qzeros && (int64_t)qzeros_bytes < groups * pack_cols * 4)
        return fail(WB_ERR_BAD_ARG, "GPTQ: qzeros 字节不足，需要 %lld，实际 %lld",
                    (long long)(groups * pack_cols * 4), (long long)qzeros_bytes);
    if (group % pack != 0)
        return fail(WB_ERR_BAD_ARG, "GPTQ: groupSize=%lld 必须是 packFactor=%lld 的整数倍", (long long)group,
                    (long long)pack);
    if (col_begin < 0 || col_count <= 0 || col_begin + col_count > outF)
        return fail(WB_ERR_BAD_ARG, "GPTQ: column slice [%lld, +%lld) outside out=%lld", (long long)col_begin,
                    (long long)col_count, (long long)outF);
    const bool sliced = !(col_begin == 0 && col_count == outF);
    if (sliced && (col_begin % 8 != 0 || col_count % 8 != 0))
        return fail(WB_ERR_BAD_ARG, "GPTQ: a column slice must start and end on a multiple of 8 (a qzeros word)");

    Weight w;
    w.name = name;
    w.kind = WeightKind::Gptq;
    w.K = inF;
    w.N = col_count;
    w.group = group;
    w.pack_rows = pack_rows;
    w.groups = groups;
    w.zcols = (col_count + 7) / 8;
    w.has_zeros = qzeros != nullptr;
    const uint64_t qw_bytes = (uint64_t)pack_rows * col_count * 4;
    const uint64_t qz_bytes = (uint64_t)groups * w.zcols * 4;
    const uint64_t sc_bytes = (uint64_t)groups * col_count * 2;
    w.bytes = align_up(qw_bytes) + align_up(sc_bytes) + (w.has_zeros ? align_up(qz_bytes) : 0);

    // The device keeps the checkpoint's own packing: qweight rows are already contiguous along the
    // output dimension, which is what both the streaming kernel (128-bit loads of 4 columns) and the
    // TMA box of the tensor-core kernel want. A column slice is a strided 2-D copy.
    const uint64_t mark = ctx->arena[WB_ARENA_WEIGHTS].used;
    const int rc = [&]() -> int {
        WB_CHECK(arena_alloc(ctx, WB_ARENA_WEIGHTS, qw_bytes, &w.off_main));
        WB_CHECK(arena_alloc(ctx, WB_ARENA_WEIGHTS, sc_bytes, &w.off_scales));
        if (w.has_zeros) WB_CHECK(arena_alloc(ctx, WB_ARENA_WEIGHTS, qz_bytes, &w.off_zeros));
        char *base = ctx->arena[WB_ARENA_WEIGHTS].base;
        WB_CUDA(cudaMemcpy2DAsync(base + w.off_main, (size_t)col_count * 4, (const char *)qweight + col_begin * 4,
                                  (size_t)outF * 4, (size_t)col_count * 4, (size_t)pack_rows, cudaMemcpyHostToDevice,
                                  ctx->stream));
        WB_CUDA(cudaMemcpy2DAsync(base + w.off_scales, (size_t)col_count * 2, (const char *)scales + col_begin * 2,
                                  (size_t)outF * 2, (size_t)col_count * 2, (size_t)groups, cudaMemcpyHostToDevice,
                                  ctx->stream));
        if (w.has_zeros)
            WB_CUDA(cudaMemcpy2DAsync(base + w.off_zeros, (size_t)w.zcols * 4, (const char *)qzeros + col_begin / 8 * 4,
                                      (size_t)pack_cols * 4, (size_t)w.zcols * 4, (size_t)groups, cudaMemcpyHostToDevice,
                                      ctx->stream));
        WB_CUDA(cudaStreamSynchronize(ctx->stream));
        return WB_OK;
    }();
    if (rc != WB_OK) {
        ctx->arena[WB_ARENA_WEIGHTS].used = mark;  // a failed registration leaves the arena as it found it
        return rc;
    }
    return add_weight(ctx, std::move(w), out);
}

int wb_gptq_register(wb_context *ctx, const char *name, const void *qweight, uint64_t qweight_bytes,
                     const void *qzeros, uint64_t qzeros_bytes, const uint16_t *scales_f16, uint64_t scales_len,
                     int64_t in_features, int64_t out_features, int64_t group_size, int bits, wb_handle *out)
{
    WB_CTX(ctx);
    return gptq_register_impl(ctx, name, qweight, qweight_bytes, qzeros, qzeros_bytes, scales_f16, scales_len,
                              in_features, out_features, group_size, bits, 0, out_features, out);
}

int wb_gptq_register_cols(wb_context *ctx, const char *name, const void *qweight, uint64_t qweight_bytes,
                          const void *qzeros, uint64_t qzeros_bytes, const uint16_t *scales_f16, uint64_t scales_len,
                          int64_t in_features, int64_t out_features, int64_t group_size, int bits, int64_t col_begin,
                          int64_t col_count, wb_handle *out)
{
    WB_CTX(ctx);
    return gptq_register_impl(ctx, name, qweight, qweight_bytes, qzeros, qzeros_bytes, scales_f16, scales_len,
                              in_features, out_features, group_size, bits, col_begin, col_count, out);
}

int wb_f16_alloc(wb_context *ctx, const char *name, int64_t rows, int64_t cols, wb_handle *out)
{
    WB_CTX(ctx);
    WB_CHECK(check_new_name(ctx, name));
    if (rows <= 0 || cols <= 0) return fail(WB_ERR_BAD_ARG, "wb_f16_alloc: rows/cols must be positive");
    Weight w;
    w.name = name;
    w.kind = WeightKind::DenseF16;
    w.N = rows;
    w.K = cols;
    w.bytes = align_up((uint64_t)rows * cols * 2);
    WB_CHECK(arena_alloc(ctx, WB_ARENA_WEIGHTS, (uint64_t)rows * cols * 2, &w.off_main));
    return add_weight(ctx, std::move(w), out);
}

static int dense_f16_target(wb_context *ctx, wb_handle h, int64_t elem_offset, int64_t n, Weight **w)
{
    WB_CHECK(get_weight(ctx, h, w));
    if ((*w)->kind != WeightKind::DenseF16) return fail(WB_ERR_NOT_FOUND, "缺少 f16 权重: %s", (*w)->name.c_str());
    if (elem_offset < 0 || n < 0 || elem_offset + n > (*w)->N * (*w)->K)
        return fail(WB_ERR_BAD_ARG, "f16 weight %s: range [%lld, +%lld) outside %lld elements", (*w)->name.c_str(),
                    (long long)elem_offset, (long long)n, (long long)((*w)->N * (*w)->K));
    return WB_OK;
}

int wb_f16_write_chunk(wb_context *ctx, wb_handle h, int64_t elem_offset, const float *data, int64_t n)
{
    WB_CTX(ctx);
    WB_NOT_RECORDING(ctx, "wb_f16_write_chunk");
    Weight *w;
    WB_CHECK(dense_f16_target(ctx, h, elem_offset, n, &w));
    if (n == 0) return WB_OK;
    if (!data) return fail(WB_ERR_BAD_ARG, "wb_f16_write_chunk: data is NULL");
    // Stage the f32 chunk in the workspace and convert on the device, piece by piece.
    const int64_t piece = (int64_t)(kWorkspaceBytes / 4);
    __half *dst = (__half *)(ctx->arena[WB_ARENA_WEIGHTS].base + w->off_main) + elem_offset;
    for (int64_t done = 0; done < n; done += piece) {
        int64_t cur = n - done < piece ? n - done : piece;
        WB_CUDA(cudaMemcpyAsync(ctx->workspace, data + done, (size_t)cur * 4, cudaMemcpyHostToDevice, ctx->stream));
        WB_CHECK(launch_f32_to_f16_ref(ctx, (const float *)ctx->workspace, dst + done, cur));
        WB_CUDA(cudaStreamSynchronize(ctx->stream));
    }
    return WB_OK;
}

int wb_f16_write_bits(wb_context *ctx, wb_handle h, int64_t elem_offset, const uint16_t *bits, int64_t n)
{
    WB_CTX(ctx);
    WB_NOT_RECORDING(ctx, "wb_f16_write_bits");
    Weight *w;
    WB_CHECK(dense_f16_target(ctx, h, elem_offset, n, &w));
    if (n == 0) return WB_OK;
    if (!bits) return fail(WB_ERR_BAD_ARG, "wb_f16_write_bits: bits is NULL");
    char *dst = ctx->arena[WB_ARENA_WEIGHTS].base + w->off_main + elem_offset * 2;
    WB_CUDA(cudaMemcpyAsync(dst, bits, (size_t)n * 2, cudaMemcpyHostToDevice, ctx->stream));
    WB_CUDA(cudaStreamSynchronize(ctx->stream));
    return WB_OK;
}

int wb_f32_upload(wb_context *ctx, const char *name, const float *data, int64_t n, wb_handle *out)
{
    WB_CTX(ctx);
    WB_NOT_RECORDING(ctx, "wb_f32_upload");
    WB_CHECK(check_new_name(ctx, name));
    if (n <= 0 || !data) return fail(WB_ERR_BAD_ARG, "wb_f32_upload: empty data");
    Weight w;
    w.name = name;
    w.kind = WeightKind::F32;
    w.N = n;
    w.K = 1;
    w.bytes = align_up((uint64_t)n * 4);
    const uint64_t mark = ctx->arena[WB_ARENA_WEIGHTS].used;
    WB_CHECK(arena_alloc(ctx, WB_ARENA_WEIGHTS, (uint64_t)n * 4, &w.off_main));
    cudaError_t e = cudaMemcpyAsync(ctx->arena[WB_ARENA_WEIGHTS].base + w.off_main, data, (size_t)n * 4,
                                    cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) ctx->arena[WB_ARENA_WEIGHTS].used = mark;
    WB_CUDA(e);
    return add_weight(ctx, std::move(w), out);
}

int wb_weight_lookup(wb_context *ctx, const char *name, wb_handle *out)
{
    WB_CTX(ctx);
    if (!name) return fail(WB_ERR_BAD_ARG, "name is NULL");
    auto it = ctx->by_name.find(name);
    if (it == ctx->by_name.end()) return fail(WB_ERR_NOT_FOUND, "缺少权重: %s", name);
    *out = it->second;
    return WB_OK;
}

int wb_weight_pop(wb_context *ctx)
{
    WB_CTX(ctx);
    WB_NOT_RECORDING(ctx, "wb_weight_pop");
    if (ctx->weights.empty()) return fail(WB_ERR_NOT_FOUND, "no weight is registered");
    const Weight &w = ctx->weights.back();
    // A weight's pieces were the last allocations of the weight arena when it was registered. If anything was taken
    // from the arena since (a model's KV cache and decode buffers, a raw wb_arena_alloc), rewinding would hand that
    // memory to the next registration while it is still in use.
    if (ctx->arena[WB_ARENA_WEIGHTS].used != w.arena_top)
        return fail(WB_ERR_BAD_ARG, "wb_weight_pop: %llu bytes were taken from the weight arena after %s was registered "
                                    "(a model created on this context?); the weight cannot be dropped",
                    (unsigned long long)(ctx->arena[WB_ARENA_WEIGHTS].used - w.arena_top), w.name.c_str());
    WB_CUDA(cudaStreamSynchronize(ctx->stream));
    ctx->arena[WB_ARENA_WEIGHTS].used = w.off_main;
    ctx->by_name.erase(w.name);
    ctx->weights.pop_back();
    return WB_OK;
}

int wb_read_weight_f16(wb_context *ctx, wb_handle h, int64_t elem_offset, int64_t n, uint16_t *out_bits)
{
    WB_CTX(ctx);
    Weight *w;
    WB_NOT_RECORDING(ctx, "wb_read_weight_f16");
    WB_CHECK(dense_f16_target(ctx, h, elem_offset, n, &w));
    if (n == 0) return WB_OK;
    WB_CUDA(cudaMemcpyAsync(out_bits, ctx->arena[WB_ARENA_WEIGHTS].base + w->off_main + elem_offset * 2,
                            (size_t)n * 2, cudaMemcpyDeviceToHost, ctx->stream));
    WB_CUDA(cudaStreamSynchronize(ctx->stream));
    return WB_OK;
}

int wb_weight_bytes(wb_context *ctx, uint64_t *bytes)
{
    WB_CTX(ctx);
    uint64_t total = 0;
    for (const Weight &w : ctx->weights) total += w.bytes;
    *bytes = total;
    return WB_OK;
}

// ------------------------------------------------------------------ dequant export + linear

static int dequant_common(wb_context *ctx, wb_handle h, uint64_t out_offset, bool f16)
{
    Weight *w;
    WB_CHECK(get_weight(ctx, h, &w));
    if (w->kind != WeightKind::Gptq) return fail(WB_ERR_BAD_ARG, "%s is not a GPTQ weight", w->name.c_str());
    WB_CHECK(check_range(ctx, WB_ARENA_ACT, out_offset, (uint64_t)w->N * w->K * (f16 ? 2 : 4), "wb_gptq_dequant"));
    if (out_offset % kAlign) return fail(WB_ERR_BAD_ARG, "offsets must be 256-byte aligned");
    return launch_dequant(ctx, *w, arena_ptr(ctx, WB_ARENA_ACT, out_offset), f16);
}

int wb_gptq_dequant_f32(wb_context *ctx, wb_handle h, uint64_t out_offset)
{
    WB_CTX(ctx);
    return dequant_common(ctx, h, out_offset, false);
}

int wb_gptq_dequant_f16(wb_context *ctx, wb_handle h, uint64_t out_offset)
{
    WB_CTX(ctx);
    return dequant_common(ctx, h, out_offset, true);
}

static int linear_args(wb_context *ctx, wb_handle weight, int64_t M, int act_dtype, int out_dtype, Weight **w)
{
    WB_CHECK(get_weight(ctx, weight, w));
    if ((*w)->kind == WeightKind::F32) return fail(WB_ERR_NOT_FOUND, "缺少 f16 权重: %s", (*w)->name.c_str());
    if (M <= 0) return fail(WB_ERR_BAD_ARG, "wb_linear: M must be positive");
    if ((act_dtype != WB_F32 && act_dtype != WB_F16) || (out_dtype != WB_F32 && out_dtype != WB_F16))
        return fail(WB_ERR_BAD_ARG, "wb_linear: dtype must be WB_F32 or WB_F16");
    return WB_OK;
}

int wb_linear(wb_context *ctx, wb_handle weight, uint64_t a_offset, uint64_t c_offset, wb_handle bias, int64_t M,
              int act_dtype, int out_dtype, int exact)
{
    WB_CTX(ctx);
    Weight *w;
    WB_CHECK(linear_args(ctx, weight, M, act_dtype, out_dtype, &w));
    if (a_offset % kAlign || c_offset % kAlign) return fail(WB_ERR_BAD_ARG, "offsets must be 256-byte aligned");
    WB_CHECK(check_range(ctx, WB_ARENA_ACT, a_offset, (uint64_t)M * w->K * (act_dtype == WB_F16 ? 2 : 4), "wb_linear A"));
    WB_CHECK(check_range(ctx, WB_ARENA_ACT, c_offset, (uint64_t)M * w->N * (out_dtype == WB_F16 ? 2 : 4), "wb_linear C"));
    const float *bias_ptr = nullptr;
    if (bias >= 0) {
        Weight *b;
        WB_CHECK(get_weight(ctx, bias, &b));
        if (b->kind != WeightKind::F32) return fail(WB_ERR_NOT_FOUND, "缺少 f32 权重: %s", b->name.c_str());
        if (b->N != w->N) return fail(WB_ERR_BAD_ARG, "bias %s has %lld elements, N=%lld", b->name.c_str(),
                                      (long long)b->N, (long long)w->N);
        bias_ptr = (const float *)(ctx->arena[WB_ARENA_WEIGHTS].base + b->off_main);
    }
    return launch_linear(ctx, *w, arena_ptr(ctx, WB_ARENA_ACT, a_offset), arena_ptr(ctx, WB_ARENA_ACT, c_offset),
                         bias_ptr, M, act_dtype, out_dtype, exact);
}

// `sync` != nullptr: the call also runs the peer barrier (wb_linear_gather_barrier).
struct GatherSync {
    uint64_t flags_offset;
    int rank;
    uint32_t timeout_us;
};

static int linear_gather_impl(wb_context *ctx, wb_handle weight, uint64_t a_offset, uint64_t c_offset, uint64_t tmp_offset,
                              wb_handle bias, int64_t M, int act_dtype, int out_dtype, int64_t n_total, int64_t col_begin,
                              void *const *peer_bases, int n_peers, const GatherSync *sync)
{
    WB_CTX(ctx);
    Weight *w;
    WB_CHECK(linear_args(ctx, weight, M, act_dtype, out_dtype, &w));
    if (n_peers < 0 || n_peers > kMaxGatherDst - 1 || (n_peers > 0 && !peer_bases))
        return fail(WB_ERR_BAD_ARG, "wb_linear_gather: at most %d peers", kMaxGatherDst - 1);
    if (col_begin < 0 || n_total <= 0 || col_begin + w->N > n_total)
        return fail(WB_ERR_BAD_ARG, "wb_linear_gather: columns [%lld, %lld) do not fit a row of %lld", (long long)col_begin,
                    (long long)(col_begin + w->N), (long long)n_total);
    const uint64_t esz = out_dtype == WB_F16 ? 2 : 4;
    if (a_offset % kAlign || c_offset % kAlign || tmp_offset % kAlign) return fail(WB_ERR_BAD_ARG, "offsets must be 256-byte aligned");
    WB_CHECK(check_range(ctx, WB_ARENA_ACT, a_offset, (uint64_t)M * w->K * (act_dtype == WB_F16 ? 2 : 4), "wb_linear_gather A"));
    WB_CHECK(check_range(ctx, WB_ARENA_ACT, c_offset, (uint64_t)M * n_total * esz, "wb_linear_gather C"));
    const float *bias_ptr = nullptr;
    if (bias >= 0) {
        Weight *b;
        WB_CHECK(get_weight(ctx, bias, &b));
        if (b->kind != WeightKind::F32) return fail(WB_ERR_NOT_FOUND, "缺少 f32 权重: %s", b->name.c_str());
        if (b->N != w->N) return fail(WB_ERR_BAD_ARG, "bias %s has %lld elements, N=%lld", b->name.c_str(),
                                      (long long)b->N, (long long)w->N);
        bias_ptr = (const float *)(ctx->arena[WB_ARENA_WEIGHTS].base + b->off_main);
    }
    OutPlace pl;
    pl.ld = n_total, pl.col0 = (int)col_begin, pl.n_dst = 1 + n_peers, pl.elem_bytes = (int)esz;
    pl.dst[0] = arena_ptr(ctx, WB_ARENA_ACT, c_offset);
    for (int g = 0; g < n_peers; g++) {
        if (!peer_bases[g]) return fail(WB_ERR_BAD_ARG, "wb_linear_gather: peer %d is NULL", g);
        pl.dst[1 + g] = (char *)peer_bases[g] + c_offset;
    }
    ctx->place = pl;  // the planner prices the stores to the peers
    wb_plan plan;
    int rc = plan_linear(ctx, *w, M, act_dtype, 0, &plan);
    ctx->place = OutPlace();
    WB_CHECK(rc);
    const void *A = arena_ptr(ctx, WB_ARENA_ACT, a_offset);
    bool barrier_done = false;
    if (plan.kernel == WB_KERNEL_GEMM_TC || plan.kernel == WB_KERNEL_GEMM_TC_PAIR) {
        // the tensor-core kernel (and its split-K reduce) stores every output tile straight to all destinations
        ctx->place = pl;
        rc = launch_linear(ctx, *w, A, pl.dst[0], bias_ptr, M, act_dtype, out_dtype, 0);
        ctx->place = OutPlace();
    } else {
        // decode-size kernels write a dense [M, N] piece to the scratch tensor; one small launch spreads it (and, with
        // `sync`, signals and waits for the peers in that same launch while the piece is small enough for one CTA)
        WB_CHECK(check_range(ctx, WB_ARENA_ACT, tmp_offset, (uint64_t)M * w->N * esz, "wb_linear_gather scratch"));
        void *tmp = arena_ptr(ctx, WB_ARENA_ACT, tmp_offset);
        rc = launch_linear(ctx, *w, A, tmp, bias_ptr, M, act_dtype, out_dtype, 0);
        if (rc == WB_OK) {
            ctx->place = pl;
            if (sync && (uint64_t)M * w->N * esz <= (256u << 10)) {
                rc = launch_scatter_barrier(ctx, tmp, M, w->N, out_dtype == WB_F16, sync->flags_offset, sync->rank, peer_bases,
                                            n_peers, sync->timeout_us);
                barrier_done = true;
            } else {
                rc = launch_scatter_cols(ctx, tmp, M, w->N, out_dtype == WB_F16);
            }
            ctx->place = OutPlace();
        }
    }
    if (rc == WB_OK && sync && !barrier_done)
        rc = wb_peer_barrier(ctx, sync->flags_offset, sync->rank, peer_bases, n_peers, sync->timeout_us);
    return rc;
}

int wb_linear_gather(wb_context *ctx, wb_handle weight, uint64_t a_offset, uint64_t c_offset, uint64_t tmp_offset,
                     wb_handle bias, int64_t M, int act_dtype, int out_dtype, int64_t n_total, int64_t col_begin,
                     void *const *peer_bases, int n_peers)
{
    return linear_gather_impl(ctx, weight, a_offset, c_offset, tmp_offset, bias, M, act_dtype, out_dtype, n_total, col_begin,
                              peer_bases, n_peers, nullptr);
}

int wb_linear_gather_barrier(wb_context *ctx, wb_handle weight, uint64_t a_offset, uint64_t c_offset, uint64_t tmp_offset,
                             wb_handle bias, int64_t M, int act_dtype, int out_dtype, int64_t n_total, int64_t col_begin,
                             void *const *peer_bases, int n_peers, uint64_t flags_offset, int rank, uint32_t timeout_us)
{
    const GatherSync sync{flags_offset, rank, timeout_us};
    return linear_gather_impl(ctx, weight, a_offset, c_offset, tmp_offset, bias, M, act_dtype, out_dtype, n_total, col_begin,
                              peer_bases, n_peers, &sync);
}

int wb_arena_ipc_export(wb_context *ctx, int arena, void *handle_out)
{
    WB_CTX(ctx);
    if (arena != 0 && arena != 1) return fail(WB_ERR_BAD_ARG, "bad arena %d", arena);
    if (!handle_out) return fail(WB_ERR_BAD_ARG, "handle_out is NULL");
    if (!ctx->arena[arena].base || !ctx->arena[arena].owned)
        return fail(WB_ERR_BAD_ARG, "only a slab that the library allocated itself (wb_arena_create) can be exported");
    static_assert(sizeof(cudaIpcMemHandle_t) == WB_IPC_HANDLE_BYTES, "handle size");
    cudaIpcMemHandle_t h;
    WB_CUDA(cudaIpcGetMemHandle(&h, ctx->arena[arena].base));
    memcpy(handle_out, &h, sizeof h);
    return WB_OK;
}

int wb_peer_open(wb_context *ctx, const void *handle, void **base_out)
{
    WB_CTX(ctx);
    if (!handle || !base_out) return fail(WB_ERR_BAD_ARG, "wb_peer_open: NULL argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof h);
    void *p = nullptr;
    WB_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *base_out = p;
    return WB_OK;
}

int wb_peer_close(wb_context *ctx, void *base)
{
    WB_CTX(ctx);
    if (!base) return WB_OK;
    WB_CUDA(cudaIpcCloseMemHandle(base));
    return WB_OK;
}

int wb_read_sweep(wb_context *ctx, int arena, uint64_t offset, uint64_t bytes, int ctas)
{
    WB_CTX(ctx);
    if (arena != 0 && arena != 1) return fail(WB_ERR_BAD_ARG, "bad arena %d", arena);
    if (offset % 16 || bytes % 16 || bytes == 0 || ctas <= 0) return fail(WB_ERR_BAD_ARG, "wb_read_sweep: 16-byte units, ctas > 0");
    if (!ctx->arena[arena].base || offset + bytes > ctx->arena[arena].capacity)
        return fail(WB_ERR_BAD_ARG, "wb_read_sweep: range outside the slab");
    read_sweep_kernel<<<ctas, 256, 0, ctx->stream>>>((const uint4 *)(ctx->arena[arena].base + offset), bytes / 16,
                                                     (uint32_t *)ctx->counters + (kMaxCounters - 1));
    ctx->launches++;
    WB_CUDA(cudaGetLastError());
    return WB_OK;
}

int wb_plan_query(wb_context *ctx, wb_handle weight, int64_t M, int act_dtype, int exact, wb_plan *out)
{
    WB_CTX(ctx);
    Weight *w;
    WB_CHECK(linear_args(ctx, weight, M, act_dtype, WB_F32, &w));
    if (!out) return fail(WB_ERR_BAD_ARG, "out is NULL");
    return plan_linear(ctx, *w, M, act_dtype, exact, out);
}

int wb_plan_override(wb_context *ctx, int kernel, int split_k)
{
    WB_CTX(ctx);
    if (kernel < 0 || kernel > WB_KERNEL_GEMM_TC_PAIR || split_k < 0)
        return fail(WB_ERR_BAD_ARG, "wb_plan_override: bad kernel %d / split %d", kernel, split_k);
    ctx->force_kernel = kernel;
    ctx->force_split = split_k;
    return WB_OK;
}

int wb_linear_hint_next(wb_context *ctx, wb_handle next_weight)
{
    WB_CTX(ctx);
    if (next_weight < 0) {
        ctx->prefetch_weight = -1;
        return WB_OK;
    }
    Weight *w = nullptr;
    WB_CHECK(get_weight(ctx, next_weight, &w));
    ctx->prefetch_weight = (int)(w - ctx->weights.data());
    return WB_OK;
}

}  // extern "C"
