// Exchange step of the output-column-sharded linear: one process and one context per GPU of a node.
//
// The reference has a single device (src/gpu/device.ts:40-98), so nothing here replaces reference code; the
// call keeps QwenGpt.gemm's meaning (src/model/qwen.ts:568-618) for the full [M, N] result while every rank
// holds N / G of the output columns. Two exchanges are offered:
//
//   * wb_comm_init / wb_linear_colshard: the local product followed by an NCCL all-gather on the context's
//     stream. NCCL is loaded with dlopen on first use, so the library itself links only the CUDA runtime and
//     single-GPU hosts never need NCCL installed. The communicator is created non-blocking and polled with
//     a host-side time limit: a rank that never joins costs the others that limit, not a hang.
//   * wb_linear_gather (context.cu) + wb_peer_barrier: the product's own stores go to every peer slab, and
//     this file's barrier kernel replaces a collective as the "everyone has stored" signal. Each rank writes
//     an increasing epoch word into slot `rank` of every peer's flag array (after a system-scope fence, so
//     the data stores are visible first) and then polls its own array until every other slot has reached the
//     epoch. The epoch counter lives on the device, so the barrier can be recorded into a command batch. The
//     poll is bounded by wall time on the device: when it runs out the kernel writes a code to the context's
//     status word and returns, and wb_synchronize reports WB_ERR_TIMEOUT. Plain peer stores and loads of this
//     GPU's own memory only: no multimem, no multicast, no kernel reads a peer's memory.
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <thread>

#include "common.cuh"

namespace wb {

namespace {

struct NcclApi {
    void *lib = nullptr;
    decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
    decltype(&ncclCommInitRankConfig) CommInitRankConfig = nullptr;
    decltype(&ncclCommGetAsyncError) CommGetAsyncError = nullptr;
    decltype(&ncclCommAbort) CommAbort = nullptr;
    decltype(&ncclCommDestroy) CommDestroy = nullptr;
    decltype(&ncclAllGather) AllGather = nullptr;
    decltype(&ncclGetErrorString) GetErrorString = nullptr;
};

NcclApi g_nccl;

// WEBLLM_B200_NCCL_LIB names the library file; otherwise the usual sonames. A process that already has NCCL
// loaded (e.g. through a framework) gets that copy back from dlopen.
int nccl_load()
{
    if (g_nccl.lib) return WB_OK;
    const char *names[3] = {getenv("WEBLLM_B200_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    void *lib = nullptr;
    for (const char *n : names) {
        if (n && *n && (lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL)) != nullptr) break;
    }
    if (!lib) return fail(WB_ERR_NCCL, "NCCL is not available: dlopen(libnccl.so.2) failed (%s); set WEBLLM_B200_NCCL_LIB", dlerror());
    NcclApi a;
    a.lib = lib;
#define WB_SYM(field, name)                                                                  \
    a.field = (decltype(a.field))dlsym(lib, name);                                           \
    if (!a.field) return fail(WB_ERR_NCCL, "NCCL library lacks the symbol %s", name)
    WB_SYM(GetUniqueId, "ncclGetUniqueId");
    WB_SYM(CommInitRankConfig, "ncclCommInitRankConfig");
    WB_SYM(CommGetAsyncError, "ncclCommGetAsyncError");
    WB_SYM(CommAbort, "ncclCommAbort");
    WB_SYM(CommDestroy, "ncclCommDestroy");
    WB_SYM(AllGather, "ncclAllGather");
    WB_SYM(GetErrorString, "ncclGetErrorString");
#undef WB_SYM
    g_nccl = a;
    return WB_OK;
}

int nccl_fail(const char *what, ncclResult_t r)
{
    return fail(WB_ERR_NCCL, "%s: %s", what, g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "NCCL error");
}

// Waits (on the host, bounded) until a call on a non-blocking communicator has left the in-progress state.
int nccl_settle(ncclComm_t comm, ncclResult_t r, int timeout_ms, const char *what)
{
    const auto t0 = std::chrono::steady_clock::now();
    while (r == ncclInProgress) {
        const auto waited = std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count();
        if (waited > (long long)timeout_ms * 1000)
            return fail(WB_ERR_TIMEOUT, "%s did not complete within %d ms (a rank that never joined?)", what, timeout_ms);
        // an enqueue settles within microseconds: poll closely at first, back off for the long waits (creation)
        if (waited > 200) std::this_thread::sleep_for(std::chrono::microseconds(waited > 20000 ? 500 : 20));
        ncclResult_t q = g_nccl.CommGetAsyncError(comm, &r);
        if (q != ncclSuccess) return nccl_fail(what, q);
    }
    if (r != ncclSuccess) return nccl_fail(what, r);
    return WB_OK;
}

// ---- kernels ---------------------------------------------------------------------------------------------------

// Layout of the WB_PEER_FLAG_BYTES flag area of a slab: word r (r < 8) is written by rank r's barrier kernel with
// that rank's epoch; word 8 is this GPU's own epoch counter. The counter lives on the device and the kernel advances
// it, so a recorded barrier (command batch, CUDA graph) takes a new epoch on every replay.
constexpr int kEpochWord = 8;

struct PeerSync {
    unsigned *own_flags;                    // this GPU's flag area
    unsigned *peer_flags[kMaxGatherDst];    // the same area in every peer slab
    int n_peers, rank, nranks;
    unsigned long long limit_ns;
    int *status;
};

__device__ __forceinline__ unsigned long long global_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Signal and wait; called by the first warp of ONE CTA after a __syncthreads() that follows the CTA's stores. Thread 0
// alone issues the system-scope fence (the barrier before it orders the other threads' stores in front of the fence,
// and one fence is far cheaper than one per thread) and then publishes the epoch; threads 0 .. nranks - 1 (but
// `rank`) wait. What the peers stored into this GPU's memory before their flag is seen by the kernels that follow
// in the stream (kernel boundary), so the waiting side needs no fence of its own.
__device__ __forceinline__ void peer_signal_and_wait(const PeerSync &ps)
{
    const int t = threadIdx.x;
    // every rank issues the same sequence of barriers, so the local counters agree on the epoch
    const unsigned epoch = ps.own_flags[kEpochWord] + 1u;
    __syncwarp();
    if (t == 0) {
        ps.own_flags[kEpochWord] = epoch;
        __threadfence_system();
#pragma unroll
        for (int g = 0; g < kMaxGatherDst - 1; g++)
            if (g < ps.n_peers) *(volatile unsigned *)(ps.peer_flags[g] + ps.rank) = epoch;
    }
    if (t < ps.nranks && t != ps.rank) {
        const unsigned long long t0 = global_ns();
        const volatile unsigned *flag = ps.own_flags + t;
        bool ok = false;
        for (unsigned it = 0; it < (1u << 28); it++) {
            if ((int)(*flag - epoch) >= 0) {
                ok = true;
                break;
            }
            __nanosleep(32);
            if ((it & 15u) == 15u && global_ns() - t0 > ps.limit_ns) break;
        }
        if (!ok) *(volatile int *)ps.status = 7;  // the peer barrier gave up
    }
}

// Both kernels are launched with programmatic stream serialization: their CTA becomes resident under the tail of the
// kernel before them and waits there (pdl_sync) until that kernel has completed and its stores are visible.
__global__ void __launch_bounds__(32) peer_barrier_kernel(const PeerSync ps)
{
    pdl_sync();
    peer_signal_and_wait(ps);
}

// Decode-size column-sharded call: copies the dense local [M, N] piece to its columns of every destination and
// runs the barrier in the same launch (one CTA: the signal must follow ALL of the copy's stores).
__global__ void __launch_bounds__(1024) scatter_barrier_kernel(const void *__restrict__ src, const OutPlace pl, int64_t M, int N,
                                                                int esz, const PeerSync ps)
{
    pdl_sync();
    const int row_bytes = N * esz;
    const bool vec = (row_bytes & 15) == 0 && ((pl.ld * esz) & 15) == 0 && ((pl.col0 * esz) & 15) == 0;
    if (vec) {
        const int per_row = row_bytes >> 4;
        for (int64_t i = threadIdx.x; i < M * per_row; i += blockDim.x) {
            const int64_t m = i / per_row;
            const int64_t off = (m * pl.ld + pl.col0) * esz + (i - m * per_row) * 16;
            const uint4 v = *(const uint4 *)((const char *)src + i * 16);
#pragma unroll
            for (int g = 0; g < kMaxGatherDst; g++)
                if (g < pl.n_dst) *(uint4 *)((char *)pl.dst[g] + off) = v;
        }
    } else {
        for (int64_t i = threadIdx.x; i < M * N; i += blockDim.x) {
            const int64_t m = i / N;
            const int64_t o = m * pl.ld + pl.col0 + (i - m * N);
#pragma unroll
            for (int g = 0; g < kMaxGatherDst; g++) {
                if (g < pl.n_dst) {
                    if (esz == 2) ((__half *)pl.dst[g])[o] = ((const __half *)src)[i];
                    else ((float *)pl.dst[g])[o] = ((const float *)src)[i];
                }
            }
        }
    }
    __syncthreads();
    if (threadIdx.x < 32) peer_signal_and_wait(ps);
}

// [G][M][Nl] (what an all-gather delivers) -> row-major [M][G * Nl], 16-byte pieces (Nl * esz % 16 == 0)
__global__ void __launch_bounds__(256) rank_major_to_row_major_kernel(const uint4 *__restrict__ in, uint4 *__restrict__ out,
                                                                      int64_t M, int G, int per_piece_row)
{
    const int64_t total = (int64_t)G * M * per_piece_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t g = i / (M * per_piece_row), r = i - g * M * per_piece_row;
        const int64_t m = r / per_piece_row, c = r - m * per_piece_row;
        out[(m * G + g) * per_piece_row + c] = in[i];
    }
}

}  // namespace

void comm_release(wb_context *ctx)
{
    if (ctx->nccl_comm && g_nccl.CommDestroy) g_nccl.CommDestroy((ncclComm_t)ctx->nccl_comm);
    ctx->nccl_comm = nullptr;
    ctx->comm_rank = 0, ctx->comm_size = 1;
}

static int fill_sync(wb_context *ctx, uint64_t flags_offset, int rank, void *const *peer_bases, int n_peers, uint32_t timeout_us,
                     PeerSync *ps)
{
    if (n_peers < 0 || n_peers > kMaxGatherDst - 1 || (n_peers > 0 && !peer_bases))
        return fail(WB_ERR_BAD_ARG, "peer barrier: at most %d peers", kMaxGatherDst - 1);
    if (rank < 0 || rank > n_peers) return fail(WB_ERR_BAD_ARG, "peer barrier: rank %d outside 0..%d", rank, n_peers);
    if (flags_offset % kAlign) return fail(WB_ERR_BAD_ARG, "offsets must be 256-byte aligned");
    WB_CHECK(check_range(ctx, WB_ARENA_ACT, flags_offset, WB_PEER_FLAG_BYTES, "peer barrier flags"));
    ps->own_flags = (unsigned *)arena_ptr(ctx, WB_ARENA_ACT, flags_offset);
    for (int g = 0; g < kMaxGatherDst; g++) ps->peer_flags[g] = nullptr;
    for (int g = 0; g < n_peers; g++) {
        if (!peer_bases[g]) return fail(WB_ERR_BAD_ARG, "peer barrier: peer %d is NULL", g);
        ps->peer_flags[g] = (unsigned *)((char *)peer_bases[g] + flags_offset);
    }
    ps->n_peers = n_peers, ps->rank = rank, ps->nranks = n_peers + 1;
    ps->limit_ns = (unsigned long long)(timeout_us ? timeout_us : 2000000u) * 1000ull;
    ps->status = ctx->status_word;
    return WB_OK;
}

// Used by wb_linear_gather_barrier for decode-size calls (ctx->place holds the destinations).
int launch_scatter_barrier(wb_context *ctx, const void *src, int64_t M, int64_t N, bool f16, uint64_t flags_offset, int rank,
                           void *const *peer_bases, int n_peers, uint32_t timeout_us)
{
    PeerSync ps;
    WB_CHECK(fill_sync(ctx, flags_offset, rank, peer_bases, n_peers, timeout_us, &ps));
    const cudaError_t e = launch_pdl(scatter_barrier_kernel, dim3(1), dim3(1024), 0, ctx->stream, src, ctx->place, M, (int)N,
                                     f16 ? 2 : 4, ps);
    ctx->launches++;
    WB_CUDA(e);
    return WB_OK;
}

}  // namespace wb

using namespace wb;

extern "C" {

int wb_comm_unique_id(void *id_out)
{
    if (!id_out) return fail(WB_ERR_BAD_ARG, "id_out is NULL");
    WB_CHECK(nccl_load());
    static_assert(sizeof(ncclUniqueId) == WB_COMM_ID_BYTES, "unique id size");
    ncclUniqueId id;
    const ncclResult_t r = g_nccl.GetUniqueId(&id);
    if (r != ncclSuccess) return nccl_fail("ncclGetUniqueId", r);
    memcpy(id_out, &id, sizeof id);
    return WB_OK;
}

int wb_comm_init(wb_context *ctx, int rank, int nranks, const void *unique_id, int timeout_ms)
{
    if (!ctx) return fail(WB_ERR_BAD_ARG, "context is NULL");
    WB_CUDA(cudaSetDevice(ctx->device));
    WB_NOT_RECORDING(ctx, "wb_comm_init");
    if (!unique_id || nranks < 1 || nranks > kMaxGatherDst || rank < 0 || rank >= nranks)
        return fail(WB_ERR_BAD_ARG, "wb_comm_init: rank %d of %d (at most %d ranks) or NULL id", rank, nranks, kMaxGatherDst);
    if (ctx->nccl_comm) return fail(WB_ERR_EXISTS, "this context already has a communicator");
    WB_CHECK(nccl_load());
    if (timeout_ms <= 0) timeout_ms = 30000;
    ncclUniqueId id;
    memcpy(&id, unique_id, sizeof id);
    ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
    cfg.blocking = 0;  // the calls return at once; completion is polled below with a time limit
    ncclComm_t comm = nullptr;
    ncclResult_t r = g_nccl.CommInitRankConfig(&comm, nranks, id, rank, &cfg);
    if (r != ncclSuccess && r != ncclInProgress) return nccl_fail("ncclCommInitRankConfig", r);
    const int rc = nccl_settle(comm, ncclInProgress, timeout_ms, "NCCL communicator creation");
    if (rc != WB_OK) {
        if (comm) g_nccl.CommAbort(comm);  // frees what the unfinished creation holds
        return rc;
    }
    ctx->nccl_comm = comm, ctx->comm_rank = rank, ctx->comm_size = nranks;
    return WB_OK;
}

int wb_comm_destroy(wb_context *ctx)
{
    if (!ctx) return fail(WB_ERR_BAD_ARG, "context is NULL");
    WB_CUDA(cudaSetDevice(ctx->device));
    WB_NOT_RECORDING(ctx, "wb_comm_destroy");
    WB_CUDA(cudaStreamSynchronize(ctx->stream));
    comm_release(ctx);
    return WB_OK;
}

int wb_linear_colshard(wb_context *ctx, wb_handle weight, uint64_t a_offset, uint64_t c_offset, uint64_t scratch_offset,
                       wb_handle bias, int64_t M, int act_dtype, int out_dtype, int row_major)
{
    if (!ctx) return fail(WB_ERR_BAD_ARG, "context is NULL");
    WB_CUDA(cudaSetDevice(ctx->device));
    WB_NOT_RECORDING(ctx, "wb_linear_colshard");
    if (!ctx->nccl_comm) return fail(WB_ERR_BAD_ARG, "wb_linear_colshard needs wb_comm_init first");
    Weight *w;
    WB_CHECK(get_weight(ctx, weight, &w));
    if (w->kind == WeightKind::F32) return fail(WB_ERR_NOT_FOUND, "缺少 f16 权重: %s", w->name.c_str());
    if (M <= 0) return fail(WB_ERR_BAD_ARG, "wb_linear_colshard: M must be positive");
    if ((act_dtype != WB_F32 && act_dtype != WB_F16) || (out_dtype != WB_F32 && out_dtype != WB_F16))
        return fail(WB_ERR_BAD_ARG, "wb_linear_colshard: dtype must be WB_F32 or WB_F16");
    const int G = ctx->comm_size;
    const uint64_t esz = out_dtype == WB_F16 ? 2 : 4;
    const uint64_t piece = (uint64_t)M * w->N * esz;
    const bool rearrange = row_major && M > 1 && G > 1;
    if (rearrange && (w->N * esz) % 16 != 0) return fail(WB_ERR_UNSUPPORTED, "row-major gather needs N/G * element size %% 16 == 0");
    if (a_offset % kAlign || c_offset % kAlign || scratch_offset % kAlign) return fail(WB_ERR_BAD_ARG, "offsets must be 256-byte aligned");
    WB_CHECK(check_range(ctx, WB_ARENA_ACT, a_offset, (uint64_t)M * w->K * (act_dtype == WB_F16 ? 2 : 4), "wb_linear_colshard A"));
    WB_CHECK(check_range(ctx, WB_ARENA_ACT, c_offset, piece * G, "wb_linear_colshard C"));
    const uint64_t gathered_off = align_up(piece);
    WB_CHECK(check_range(ctx, WB_ARENA_ACT, scratch_offset, gathered_off + (rearrange ? piece * G : 0), "wb_linear_colshard scratch"));
    const float *bias_ptr = nullptr;
    if (bias >= 0) {
        Weight *b;
        WB_CHECK(get_weight(ctx, bias, &b));
        if (b->kind != WeightKind::F32) return fail(WB_ERR_NOT_FOUND, "缺少 f32 权重: %s", b->name.c_str());
        if (b->N != w->N) return fail(WB_ERR_BAD_ARG, "bias %s has %lld elements, N=%lld", b->name.c_str(), (long long)b->N, (long long)w->N);
        bias_ptr = (const float *)(ctx->arena[WB_ARENA_WEIGHTS].base + b->off_main);
    }
    char *local = arena_ptr(ctx, WB_ARENA_ACT, scratch_offset);
    char *out = arena_ptr(ctx, WB_ARENA_ACT, c_offset);
    char *gathered = rearrange ? local + gathered_off : out;
    WB_CHECK(launch_linear(ctx, *w, arena_ptr(ctx, WB_ARENA_ACT, a_offset), local, bias_ptr, M, act_dtype, out_dtype, 0));
    ncclComm_t comm = (ncclComm_t)ctx->nccl_comm;
    const ncclResult_t r = g_nccl.AllGather(local, gathered, piece, ncclUint8, comm, ctx->stream);
    if (r != ncclSuccess && r != ncclInProgress) return nccl_fail("ncclAllGather", r);
    WB_CHECK(nccl_settle(comm, r, 30000, "ncclAllGather (enqueue)"));
    ctx->launches++;
    if (rearrange) {
        const int per_piece_row = (int)(w->N * esz / 16);
        const int64_t total = (int64_t)G * M * per_piece_row;
        int blocks = (int)std::min<int64_t>((total + 255) / 256, (int64_t)ctx->sm_count * 8);
        rank_major_to_row_major_kernel<<<blocks, 256, 0, ctx->stream>>>((const uint4 *)gathered, (uint4 *)out, M, G, per_piece_row);
        ctx->launches++;
        WB_CUDA(cudaGetLastError());
    }
    return WB_OK;
}

int wb_peer_barrier_init(wb_context *ctx, uint64_t flags_offset)
{
    if (!ctx) return fail(WB_ERR_BAD_ARG, "context is NULL");
    WB_CUDA(cudaSetDevice(ctx->device));
    WB_NOT_RECORDING(ctx, "wb_peer_barrier_init");
    if (flags_offset % kAlign) return fail(WB_ERR_BAD_ARG, "offsets must be 256-byte aligned");
    WB_CHECK(check_range(ctx, WB_ARENA_ACT, flags_offset, WB_PEER_FLAG_BYTES, "peer barrier flags"));
    WB_CUDA(cudaMemsetAsync(arena_ptr(ctx, WB_ARENA_ACT, flags_offset), 0, WB_PEER_FLAG_BYTES, ctx->stream));
    WB_CUDA(cudaStreamSynchronize(ctx->stream));
    return WB_OK;
}

int wb_peer_barrier(wb_context *ctx, uint64_t flags_offset, int rank, void *const *peer_bases, int n_peers, uint32_t timeout_us)
{
    if (!ctx) return fail(WB_ERR_BAD_ARG, "context is NULL");
    WB_CUDA(cudaSetDevice(ctx->device));
    PeerSync ps;
    WB_CHECK(fill_sync(ctx, flags_offset, rank, peer_bases, n_peers, timeout_us, &ps));
    const cudaError_t e = launch_pdl(peer_barrier_kernel, dim3(1), dim3(32), 0, ctx->stream, ps);
    ctx->launches++;
    WB_CUDA(e);
    return WB_OK;
}

}  // extern "C"
