// Device-side pieces shared by the tcgen05 GEMM kernels: mbarrier / TMA / tensor-memory wrappers, the shared-memory
// matrix and instruction descriptors, the kernel parameter block and the transposing epilogue stores.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace wb {

namespace tc {

constexpr int BN = 128;       // output columns per accumulator (UMMA M); a CTA holds NH = 1 or 2 of them
constexpr int BK = 64;        // k per stage: one 128-byte swizzle atom of fp16
constexpr int UNPACK_WARPS = 16;
// Warp roles, shared by the three kernels. The thread that issues the MMAs paces a kernel with its own instruction
// latency (a wait, four to eight tcgen05.mma, a commit per k-block), and a warp scheduler serves the warps with the same
// id % 4: so the scheduler of the issuing warp carries no unpack warp. Warp 1 = MMA issuer, 5 = TMA producer, 9 / 13 / 17
// have no part in the k-loop; the sixteen warps 0 .. 20 with id % 4 != 1 unpack. Measured on the 7B-class gate
// projection at M = 4096 (CTA-pair kernel): 383 us with the unpack warps spread over all four schedulers, 337 us so.
constexpr int MMA_WARP = 1, TMA_WARP = 5;
constexpr int WARPS = 21;             // the one-tile kernel: every warp takes part in the epilogue
constexpr int THREADS = 32 * WARPS;
__device__ __forceinline__ bool is_unpack_warp(int warp) { return (warp & 3) != 1 && warp <= 20; }
// 0 .. 15 for the unpack warps in warp-id order
__device__ __forceinline__ int unpack_index(int warp) { return (warp >> 2) * 3 + ((warp & 3) == 0 ? 0 : (warp & 3) - 1); }
constexpr uint32_t SPIN_LIMIT = 1u << 20;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait. Returns false when it gave up or another role already aborted.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *status, int code)
{
    for (uint32_t it = 0; it < SPIN_LIMIT; it++) {
        if (mbar_try(bar, parity)) return true;
        if ((it & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    if (status) *(volatile int *)status = code;
    return false;
}

// The same for a warp that waits through a whole k-loop (the persistent kernel's epilogue): it sleeps between polls so
// that it does not take issue slots from the unpack warps. 2^18 polls of >= 64 ns bound the wait at some tens of ms.
__device__ __forceinline__ bool mbar_wait_idle(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *status, int code)
{
    for (uint32_t it = 0; it < (1u << 18); it++) {
        if (mbar_try(bar, parity)) return true;
        __nanosleep(64);
        if ((it & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1;
    if (status) *(volatile int *)status = code;
    return false;
}


__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t *dst_smem, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major operand tile stored as 8-row x 128-byte swizzle atoms
// (rows 128 bytes apart, atoms 1024 bytes apart): start address >> 4, leading byte offset 1 (unused with
// a swizzle), stride byte offset 1024 >> 4, descriptor version 1 (sm_100), layout type 2 = 128-byte swizzle.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr)
{
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

// Instruction descriptor, kind::f16: D = f32 (bits 4-5 = 1), A = B = fp16 (0), both K-major (bits 15, 16 = 0),
// N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t idesc_f16(int m, int n)
{
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

struct Params {
    const uint32_t *qz;   // nullable
    const __half *sc;     // GPTQ scales; nullptr for a dense fp16 weight
    void *out;
    const float *bias;    // nullable
    int *status;
    int M, N, K;
    int zcols, group_blocks;  // group / 64
    int out_f16;
    int kb_per_slice;     // k-blocks per grid.z slice (split-K); the whole K when gridDim.z == 1
    float *partial;       // [slices][M][N] f32 partial sums when gridDim.z > 1
    // Placement of the result of a column-sharded call (GATHER instantiation; n_dst = 0 otherwise): element (m, n)
    // goes to dst[g] + m * ld_out + col0 + n for every g < n_dst, this GPU's slab first, then its peers' (the
    // all-gather is these stores, issued tile by tile while other tiles are still being multiplied).
    int64_t ld_out;
    int col0, n_dst;
    void *dst[kMaxGatherDst];
};


// ---- epilogue stores. After tcgen05.ld a lane holds ONE output column (its TMEM lane) of 16 token rows, so a plain
// store instruction writes 2 or 4 bytes per lane, 64 or 128 bytes of one row per warp. Measured on the 0.5B gate
// projection at M = 2048, those stores cost as much as the whole k-loop (20 MB of fp16 output left at ~1 TB/s, and
// the same time for f32: the cost is per store instruction, not per byte). So the lanes first transpose among
// themselves with shuffles (xor 1, 2, 4) until each holds 16 bytes of consecutive columns of one row: 2 (fp16) or 4
// (f32) store instructions per 16 rows instead of 16.
struct StoreDst {
    void *dst[kMaxGatherDst];
    int n_dst;
    int64_t ld;   // row pitch in elements
    int col0;     // column of the tile's column 0 in the destination row
};

template <bool MULTI>
__device__ __forceinline__ void store_u4(const StoreDst &d, int64_t off_bytes, const uint4 &v)
{
    *(uint4 *)((char *)d.dst[0] + off_bytes) = v;
    if constexpr (MULTI) {
        if (d.n_dst > 1) {
#pragma unroll
            for (int g = 1; g < kMaxGatherDst; g++)  // static indices: a run-time index would move the array to local memory
                if (g < d.n_dst) *(uint4 *)((char *)d.dst[g] + off_bytes) = v;
        }
    }
}

// r: this lane's column n_warp + lane, token rows m_base .. m_base + 15 (f32 bits); bias already per lane.
template <bool MULTI>
__device__ __forceinline__ void store_block16_f16(const StoreDst &d, const uint32_t (&r)[16], float bias, int m_base, int M,
                                                  int n_warp, int N, int lane)
{
    const bool b = lane & 1, c = lane & 2, e = lane & 4;
    uint32_t h[8];  // h[i]: columns (n & ~1, + 1) of row 2 i + b
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float v0 = __uint_as_float(r[2 * i]) + bias, v1 = __uint_as_float(r[2 * i + 1]) + bias;
        const float got = __shfl_xor_sync(0xffffffffu, b ? v0 : v1, 1);
        const __half2 pr = b ? __floats2half2_rn(got, v1) : __floats2half2_rn(v0, got);
        h[i] = *(const uint32_t *)&pr;
    }
    uint2 o[4];  // o[k]: four consecutive columns of row 4 k + 2 c + b
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const uint32_t got = __shfl_xor_sync(0xffffffffu, c ? h[2 * k] : h[2 * k + 1], 2);
        o[k] = c ? make_uint2(got, h[2 * k + 1]) : make_uint2(h[2 * k], got);
    }
    const int n8 = n_warp + (lane >> 3) * 8;
#pragma unroll
    for (int k = 0; k < 2; k++) {  // eight consecutive columns of row 8 k + (lane & 7)
        const uint2 snd = e ? o[2 * k] : o[2 * k + 1];
        const uint32_t gx = __shfl_xor_sync(0xffffffffu, snd.x, 4), gy = __shfl_xor_sync(0xffffffffu, snd.y, 4);
        const uint4 f = e ? make_uint4(gx, gy, o[2 * k + 1].x, o[2 * k + 1].y) : make_uint4(o[2 * k].x, o[2 * k].y, gx, gy);
        const int m = m_base + 8 * k + (lane & 7);
        if (m < M && n8 < N) store_u4<MULTI>(d, ((int64_t)m * d.ld + d.col0 + n8) * 2, f);
    }
}

template <bool MULTI>
__device__ __forceinline__ void store_block16_f32(const StoreDst &d, const uint32_t (&r)[16], float bias, int m_base, int M,
                                                  int n_warp, int N, int lane)
{
    const bool b = lane & 1, c = lane & 2;
    float2 pr[8];  // pr[i]: columns (n & ~1, + 1) of row 2 i + b
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float v0 = __uint_as_float(r[2 * i]) + bias, v1 = __uint_as_float(r[2 * i + 1]) + bias;
        const float got = __shfl_xor_sync(0xffffffffu, b ? v0 : v1, 1);
        pr[i] = b ? make_float2(got, v1) : make_float2(v0, got);
    }
    const int n4 = n_warp + (lane >> 2) * 4;
#pragma unroll
    for (int k = 0; k < 4; k++) {  // four consecutive columns of row 4 k + (lane & 3)
        const float2 snd = c ? pr[2 * k] : pr[2 * k + 1];
        const float gx = __shfl_xor_sync(0xffffffffu, snd.x, 2), gy = __shfl_xor_sync(0xffffffffu, snd.y, 2);
        const float4 f = c ? make_float4(gx, gy, pr[2 * k + 1].x, pr[2 * k + 1].y) : make_float4(pr[2 * k].x, pr[2 * k].y, gx, gy);
        const int m = m_base + 4 * k + (lane & 3);
        if (m < M && n4 < N)
            store_u4<MULTI>(d, ((int64_t)m * d.ld + d.col0 + n4) * 4,
                            make_uint4(__float_as_uint(f.x), __float_as_uint(f.y), __float_as_uint(f.z), __float_as_uint(f.w)));
    }
}

// One 16-row block of a warp's 32 columns to its destination(s): transposed 16-byte stores where rows and column
// groups are 16-byte aligned (N, pitch and column offset multiples of 8), else one element per lane.
template <bool MULTI>
__device__ __forceinline__ void store_block16(const StoreDst &d, bool f16, bool vec, const uint32_t (&r)[16], float bias, int m_base,
                                              int M, int n_warp, int N, int lane)
{
    if (vec) {
        if (f16) store_block16_f16<MULTI>(d, r, bias, m_base, M, n_warp, N, lane);
        else store_block16_f32<MULTI>(d, r, bias, m_base, M, n_warp, N, lane);
        return;
    }
    const int n = n_warp + lane;
    if (n >= N) return;
#pragma unroll
    for (int j = 0; j < 16; j++) {
        const int m = m_base + j;
        if (m < M) {
            const float v = __uint_as_float(r[j]) + bias;
            const int64_t o = (int64_t)m * d.ld + d.col0 + n;
            if (f16) {
                const __half hv = __float2half_rn(v);
                ((__half *)d.dst[0])[o] = hv;
                if constexpr (MULTI) {
#pragma unroll
                    for (int g = 1; g < kMaxGatherDst; g++)
                        if (g < d.n_dst) ((__half *)d.dst[g])[o] = hv;
                }
            } else {
                ((float *)d.dst[0])[o] = v;
                if constexpr (MULTI) {
#pragma unroll
                    for (int g = 1; g < kMaxGatherDst; g++)
                        if (g < d.n_dst) ((float *)d.dst[g])[o] = v;
                }
            }
        }
    }
}
}  // namespace tc

}  // namespace wb
