// Command batches: record many linear / dequant calls once, submit them together, replay at will.
// Replaces CommandBatch (src/gpu/pipeline.ts:55-117), which packs every dispatch of a forward pass into
// one command encoder and one submit to avoid ~110 us of CPU cost per dispatch. Here a batch is a CUDA
// graph captured from the context's stream; ordering inside it is stream order (the reference's endPass).
#include "common.cuh"

struct wb_batch {
    wb_context *ctx = nullptr;
    cudaGraphExec_t exec = nullptr;
    uint64_t launches = 0;  // kernels per replay
};

using namespace wb;

extern "C" {

int wb_batch_begin(wb_context *ctx)
{
    if (!ctx) return fail(WB_ERR_BAD_ARG, "context is NULL");
    WB_CUDA(cudaSetDevice(ctx->device));
    if (ctx->capturing) return fail(WB_ERR_BAD_ARG, "a batch is already being recorded on this context");
    WB_CUDA(cudaStreamSynchronize(ctx->stream));
    WB_CUDA(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    ctx->capturing = true;
    ctx->launches_at_capture = ctx->launches;
    return WB_OK;
}

int wb_batch_end(wb_context *ctx, wb_batch **out)
{
    if (!ctx || !out) return fail(WB_ERR_BAD_ARG, "wb_batch_end: NULL argument");
    WB_CUDA(cudaSetDevice(ctx->device));
    if (!ctx->capturing) return fail(WB_ERR_BAD_ARG, "wb_batch_end without wb_batch_begin");
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &g);
    ctx->capturing = false;
    const uint64_t recorded = ctx->launches - ctx->launches_at_capture;
    ctx->launches = ctx->launches_at_capture;  // recording launches nothing
    WB_CUDA(e);
    wb_batch *b = new wb_batch();
    b->ctx = ctx;
    b->launches = recorded;
    e = cudaGraphInstantiate(&b->exec, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) {
        delete b;
        WB_CUDA(e);
    }
    *out = b;
    return WB_OK;
}

int wb_batch_submit(wb_batch *b)
{
    if (!b) return fail(WB_ERR_BAD_ARG, "batch is NULL");
    WB_CUDA(cudaSetDevice(b->ctx->device));
    WB_CUDA(cudaGraphLaunch(b->exec, b->ctx->stream));
    b->ctx->launches += b->launches;
    return WB_OK;
}

int wb_batch_destroy(wb_batch *b)
{
    if (!b) return WB_OK;
    cudaSetDevice(b->ctx->device);
    cudaStreamSynchronize(b->ctx->stream);
    if (b->exec) cudaGraphExecDestroy(b->exec);
    delete b;
    return WB_OK;
}

}  // extern "C"
