// Shared declarations of the webllm_b200 CUDA library: context layout, error plumbing, device helpers.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/webllm_b200.h"

namespace wb {

// ---------------------------------------------------------------- errors
void set_error(const char *fmt, ...);
int fail(int code, const char *fmt, ...);

#define WB_CUDA(expr)                                                                         \
    do {                                                                                      \
        cudaError_t _e = (expr);                                                              \
        if (_e != cudaSuccess)                                                                \
            return wb::fail(WB_ERR_CUDA, "CUDA error %s at %s:%d: %s", cudaGetErrorName(_e), \
                            __FILE__, __LINE__, cudaGetErrorString(_e));                      \
    } while (0)

#define WB_CHECK(expr)          \
    do {                        \
        int _s = (expr);        \
        if (_s != WB_OK) return _s; \
    } while (0)

// Transfers, registrations and anything else that blocks on the stream are refused while a command batch is being
// recorded (the stream is capturing: they would fail inside CUDA and invalidate the recording).
#define WB_NOT_RECORDING(ctx, what)                                                                              \
    do {                                                                                                         \
        if ((ctx)->capturing)                                                                                    \
            return wb::fail(WB_ERR_BAD_ARG, "%s is not allowed while a command batch is being recorded "         \
                                            "(between wb_batch_begin and wb_batch_end)", what);                 \
    } while (0)

// ---------------------------------------------------------------- weights
enum class WeightKind : int { Gptq = 1, DenseF16 = 2, F32 = 3 };

// A CUtensorMap (128 bytes, 64-byte aligned) encoded on first use and kept with the weight it describes.
struct TmapSlot {
    alignas(64) unsigned char bytes[128];
    bool ok = false;
};

struct Weight {
    std::string name;
    WeightKind kind;
    int64_t K = 0, N = 0;     // in_features, out_features (DenseF16: cols, rows; F32: N = length)
    int64_t group = 0;        // GPTQ group size
    int64_t pack_rows = 0;    // ceil(K/8)
    int64_t groups = 0;       // ceil(K/group)
    int64_t zcols = 0;        // ceil(N/8)
    uint64_t off_main = 0;    // qweight / fp16 matrix / f32 vector (byte offset in the weight arena)
    uint64_t off_zeros = 0;   // qzeros (valid if has_zeros)
    uint64_t off_scales = 0;  // fp16 scales
    bool has_zeros = false;
    uint64_t bytes = 0;
    uint64_t arena_top = 0;   // `used` of the weight arena right after this registration (what wb_weight_pop checks)
    // tensor maps of the weight operand of the tensor-core GEMM, for 128 and 256 output columns per CTA
    mutable TmapSlot tmap_tc[2];
};

struct ArenaState {
    char *base = nullptr;
    uint64_t capacity = 0, used = 0;
    bool owned = false;
};

constexpr uint64_t kAlign = 256;
inline uint64_t align_up(uint64_t n, uint64_t a = kAlign) { return (n + a - 1) / a * a; }

// Split-K partial sums, fp16 staging of activations and arrival counters live here; sized at context
// creation so that no linear call allocates.
constexpr uint64_t kWorkspaceBytes = 96ull << 20;
constexpr int kMaxCounters = 16384;

// Where a linear's result goes when the output columns are sharded over GPUs (wb_linear_gather): element (m, n) of
// the local [M, N] product is stored at dst[g] + (m * ld + col0 + n) elements for every g < n_dst. dst[0] is this
// GPU's own slab, the others are peers' slabs mapped into this process (plain stores over NVLink).
constexpr int kMaxGatherDst = 8;
struct OutPlace {
    int64_t ld = 0;
    int col0 = 0;
    int n_dst = 0;  // 0: not a gather call
    int elem_bytes = 4;  // size of an output element (what the planner needs to price the stores to the peers)
    void *dst[kMaxGatherDst] = {};
};

}  // namespace wb

struct wb_context {
    int device = 0;
    int sm_count = 148;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;
    wb::ArenaState arena[2];
    std::vector<wb::Weight> weights;
    std::unordered_map<std::string, int> by_name;
    char *workspace = nullptr;       // kWorkspaceBytes of scratch
    unsigned *counters = nullptr;    // kMaxCounters arrival counters, zero between calls
    int *status_word = nullptr;      // device-side error flag for bounded waits (mapped pinned host memory)
    int *status_host = nullptr;
    uint64_t launches = 0;
    int force_kernel = 0, force_split = 0;
    int prefetch_weight = -1;        // index of the weight the next linear should pull into L2 (-1: none)
    void *tmap_encode = nullptr;     // cuTensorMapEncodeTiled, resolved at context creation
    wb::OutPlace place;              // set for the duration of one wb_linear_gather call (n_dst > 0)
    bool capturing = false;          // a command batch is being recorded (batch.cu)
    uint64_t launches_at_capture = 0;
    void *nccl_comm = nullptr;       // ncclComm_t of the column-sharded group (comm.cu); nullptr until wb_comm_init
    int comm_rank = 0, comm_size = 1;
};

namespace wb {

inline char *arena_ptr(wb_context *ctx, int arena, uint64_t off) { return ctx->arena[arena].base + off; }
int check_range(wb_context *ctx, int arena, uint64_t off, uint64_t bytes, const char *what);
int get_weight(wb_context *ctx, wb_handle h, Weight **out);

// kernels' host entry points (one per .cu file)
int launch_dequant(wb_context *ctx, const Weight &w, void *out, bool f16);
int launch_f32_to_f16_ref(wb_context *ctx, const float *in, __half *out, int64_t n);
int plan_linear(wb_context *ctx, const Weight &w, int64_t M, int act_dtype, int exact, wb_plan *plan);
int launch_scatter_cols(wb_context *ctx, const void *src, int64_t M, int64_t N, bool f16);  // uses ctx->place
// comm.cu: the same copy with the peer barrier in the same launch (one CTA), and the release of the communicator
int launch_scatter_barrier(wb_context *ctx, const void *src, int64_t M, int64_t N, bool f16, uint64_t flags_offset, int rank,
                           void *const *peer_bases, int n_peers, uint32_t timeout_us);
void comm_release(wb_context *ctx);
// Work a decode-size int4 projection can do on its input while staging it (see GemvPrologue in gemv_core.cuh):
// kind 1 = rmsnorm(x + delta) * norm_w with x + delta stored to x_out, kind 2 = silu(x) * up with row pitch ld.
struct LinearFusion {
    int kind = 0;
    const float *delta = nullptr;
    float *x_out = nullptr;
    const float *norm_w = nullptr;
    float eps = 0.f;
    const float *up = nullptr;
    int ld = 0;
};
// True when launch_linear would run this weight at M rows of f32 activations through the kernel that fuses.
bool linear_fusion_supported(wb_context *ctx, const Weight &w, int64_t M);
int launch_linear(wb_context *ctx, const Weight &w, const void *A, void *C, const float *bias, int64_t M,
                  int act_dtype, int out_dtype, int exact, const LinearFusion *fusion = nullptr);

// ---------------------------------------------------------------- device helpers
#ifdef __CUDACC__

// f32 -> fp16 bits with the rules of the reference's f32ToF16Bits (src/gpu/buffer.ts:57-100):
// IEEE round-to-nearest-even, except NaN -> 0x7e00 and |x| < 2^-24 -> signed zero.
__device__ __forceinline__ unsigned short f32_to_f16_bits_ref(float f)
{
    if (f != f) return 0x7e00;
    unsigned short h = __half_as_ushort(__float2half_rn(f));
    if (fabsf(f) < 5.9604644775390625e-8f) h &= 0x8000;
    return h;
}

// Weights are read once per token and are far larger than the L2 (458 MB per decode step against 126 MB): they are
// loaded with an evict-first L2 policy so that they do not push out what IS reused between kernels and steps
// (activations, the KV cache, the rotary table, norm weights), which then stays an L2 hit.
__device__ __forceinline__ uint64_t l2_evict_first_policy()
{
    uint64_t pol;
    asm("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

__device__ __forceinline__ uint4 ldg_stream_v4(const void *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p), "l"(l2_evict_first_policy()));
    return v;
}

// ---- programmatic dependent launch -------------------------------------------------------------------------
// Kernels of the decode step are launched so that the next one may become resident while the previous one is
// still running. A kernel first does whatever touches only constant data (index arithmetic, requesting its
// first weight chunks), then calls pdl_sync(): it blocks until every kernel before it in the stream has
// completed and its writes are visible, and only THEN lets its own successor start the same way. Nothing that an
// earlier kernel writes or reads may be touched before pdl_sync(). The order matters: with the trigger in front of
// the wait every kernel released its successor the moment it started, so a chain of kernels several deep sat
// resident and waiting behind the one that ran; releasing the successor after the wait keeps exactly one kernel
// ahead (its prologue overlaps the whole of this kernel) and took the 125-launch decode step from 0.577 to 0.550 ms.
// Without the launch attribute both instructions return at once.
__device__ __forceinline__ void pdl_sync()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
// The two halves, for kernels whose roles reach the dependence at different points (a producer that requests constant
// weights first, warps that only ever touch shared memory, an epilogue that must not store before its predecessor is done).
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// WEBLLM_B200_NO_PDL=1 in the environment launches every kernel fully serialised (for A/B timing).
inline bool pdl_enabled()
{
    static const bool on = [] {
        const char *e = getenv("WEBLLM_B200_NO_PDL");
        return !(e && e[0] == '1');
    }();
    return on;
}

// `cluster_y` > 1 launches thread-block clusters of (1, cluster_y, 1) CTAs (grid.y must be a multiple of it).
// `pdl` = false launches fully serialised behind the stream's earlier work: for entry points that read caller-owned
// buffers which the caller's previous kernel on that stream may still be writing (a kernel launched with the
// attribute requests its weights BEFORE it waits for its predecessor).
template <typename... P, typename... A>
inline cudaError_t launch_cluster_ex(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     unsigned cluster_y, bool pdl, A &&...args)
{
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    unsigned n = 0;
    if (pdl && pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        n++;
    }
    if (cluster_y > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 1, attr[n].val.clusterDim.y = cluster_y, attr[n].val.clusterDim.z = 1;
        n++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, P(args)...);
}

template <typename... P, typename... A>
inline cudaError_t launch_pdl_cluster(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                      unsigned cluster_y, A &&...args)
{
    return launch_cluster_ex(kernel, grid, block, smem, stream, cluster_y, true, static_cast<A &&>(args)...);
}

template <typename... P, typename... A>
inline cudaError_t launch_pdl(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A &&...args)
{
    return launch_pdl_cluster(kernel, grid, block, smem, stream, 1u, static_cast<A &&>(args)...);
}

// ---- thread-block clusters: distributed shared memory and the cluster barrier --------------------------------
__device__ __forceinline__ uint32_t cluster_cta_rank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Address of `smem_ptr` (a pointer into this CTA's shared memory) in the shared memory of CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t cluster_map_shared(const void *smem_ptr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"((uint32_t)__cvta_generic_to_shared(smem_ptr)), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_store_f32(uint32_t addr, float v)
{
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
// Every thread of every CTA of the cluster must reach this; stores made before it (also remote ones) are visible after.
__device__ __forceinline__ void cluster_barrier()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---- merge through an mbarrier in the cluster's first CTA instead of a second cluster barrier ----
// The senders write their values with st.async (the store itself reports its bytes to the barrier) and leave; the first
// CTA waits on the barrier's phase, bounded. The barrier is initialised at the top of the kernel and made known with one
// relaxed cluster barrier there, off the critical path: what the closing barrier.cluster.arrive.release cost the senders
// and the receiver (a fence at cluster scope, then a round trip) no longer follows the last partial sum.
constexpr int kStatusClusterMergeTimeout = 31;
__device__ __forceinline__ void cluster_merge_init(uint64_t *bar, uint32_t expect_bytes, bool receiver)
{
    if (receiver && threadIdx.x == 0) {
        const uint32_t a = (uint32_t)__cvta_generic_to_shared(bar);
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(a));
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(a), "r"(expect_bytes) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();  // the .aligned forms want the warp converged
    asm volatile("barrier.cluster.arrive.relaxed.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// remote_addr, remote_bar: shared::cluster addresses (cluster_map_shared) in the receiving CTA
__device__ __forceinline__ void cluster_send_f32(uint32_t remote_addr, float v, uint32_t remote_bar)
{
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.f32 [%0], %1, [%2];" ::"r"(remote_addr), "f"(v), "r"(remote_bar)
                 : "memory");
}
// Every thread of the receiver that reads the merged values calls this. False (and `status` set) when the bytes did not
// arrive within ~2^20 polls; the caller carries on with what it has, the host sees the code at its next synchronize.
__device__ __forceinline__ bool cluster_merge_wait(uint64_t *bar, int *status)
{
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(bar);
    for (uint32_t it = 0; it < (1u << 20); it++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(a)
            : "memory");
        if (ok) return true;
    }
    if (status) *(volatile int *)status = kStatusClusterMergeTimeout;
    return false;
}

#endif  // __CUDACC__

}  // namespace wb
