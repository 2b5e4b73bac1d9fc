// Inner loop of the fused int4 GEMV (gemv.cu): fetch of one 128-k chunk, and its unpack + MMA.
//
// Instruction budget: at HBM speed a warp consumes one 512-byte load (32 lanes x 128 bits = 1024 weights) every
// ~47 ns per SM sub-partition, so the loop has to stay within a few dozen issue slots per load; see compute_chunk.
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

namespace wb {

// Launch parameters of the streaming GEMV; the chunk functions below read the weight pointers and sizes.
struct GemvParams {
    const uint32_t *qw;
    const uint32_t *qz;  // nullable
    const __half *sc;
    const void *x;
    void *out;
    const float *bias;  // nullable
    float *partial;
    unsigned *counters;
    int M, N, K;
    int pack_rows, zcols;
    int chunks;         // ceil(pack_rows / 16)
    int chunks_per_split;
    int group_chunks;   // group / 128
    int S;
    int wn, wk;         // warps across columns / across k
    int x_f16, out_f16;
    int xs_stride;      // uint4 per staged activation row
    int stages;         // depth of the per-thread cp.async ring
    int ring_off;       // byte offset of the ring in dynamic shared memory
    int red_off;        // byte offset of the cross-warp reduction buffer
    int direct;         // 1: every warp holds at most one chunk of one tile: it is loaded straight into registers
    int cluster;        // 1: the S slices of a column tile are one thread-block cluster and merge through its shared memory
    int cl_off;         // byte offset of the [S][M * tile columns] merge buffer (used in the cluster's first CTA)
    int cl_async;       // 1: the slices send their partial tiles with st.async to an mbarrier of the first CTA (one tile per CTA)
    int *status;        // error word of the context (bounded waits)
    const char *pf_ptr;   // weight of a later call to pull into L2 while this one runs (nullable)
    unsigned pf_bytes;    // multiple of 16
    // Optional work fused in front of the projection (f32 activations, M <= 8); see GemvPrologue.
    int prologue;
    const float *delta;   // RmsNorm: x_in = x + delta (nullable)
    float *x_out;         // RmsNorm with delta: where CTA (0, 0) stores x_in, [M, K]
    const float *norm_w;  // RmsNorm: weight [K]
    float eps;
    const float *up;      // SiluMul: the second factor; rows of x and up are `ld_x` floats apart
    int ld_x;
};

// What the GEMV does to its input while staging it:
//   RmsNorm  the operand is rmsnorm(x + delta) * norm_w (rmsNormRef, src/reference/qwen-ref.ts:12-29, after the
//            residual add of vec_add.wgsl); every CTA needs the whole row for the mean square, so K is not split
//            for the statistic, only for the staging.
//   SiluMul  the operand is silu(x) * up (siluMulRef, src/reference/qwen-ref.ts:119-123).
enum GemvPrologue : int { kPrologueNone = 0, kPrologueRmsNorm = 1, kPrologueSiluMul = 2 };

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }


struct ChunkRegs {
    uint4 w[4];     // packed words: rows 4*st + t of the chunk, columns c .. c+3
    uint2 s;        // four fp16 scales
    uint32_t z;     // four stored zero nibbles in bits 0..15
};

__device__ __forceinline__ void fetch_chunk(const GemvParams &p, int ch, int t, int c, bool col_ok, ChunkRegs &r)
{
    const uint4 zero4 = make_uint4(0, 0, 0, 0);
    const uint32_t *base = p.qw + (int64_t)(ch * 16 + t) * p.N + c;
    const int64_t step = (int64_t)4 * p.N;
    if (ch * 16 + 16 <= p.pack_rows) {  // whole chunk inside the matrix (all but possibly the last one)
#pragma unroll
        for (int st = 0; st < 4; st++) r.w[st] = col_ok ? ldg_stream_v4(base + st * step) : zero4;
    } else {
#pragma unroll
        for (int st = 0; st < 4; st++)
            r.w[st] = (col_ok && ch * 16 + st * 4 + t < p.pack_rows) ? ldg_stream_v4(base + st * step) : zero4;
    }
    const int G = p.group_chunks == 1 ? ch : ch / p.group_chunks;
    r.s = make_uint2(0u, 0u);
    r.z = 0x7777u;  // stored zero 7 -> zero point 8 when the checkpoint has no qzeros
    if (col_ok) {
        r.s = *reinterpret_cast<const uint2 *>(p.sc + (int64_t)G * p.N + c);
        if (p.qz) r.z = p.qz[(int64_t)G * p.zcols + (c >> 3)] >> ((c & 7) * 4);
    }
}

// ---- asynchronous fetch: the same chunk, copied global -> shared by cp.async into a slot that belongs to
// this thread alone (80 bytes: 4 x 16 words, 8 scales, 4 zeros). A thread only ever reads back what it copied
// itself, so there are no bank conflicts and no barriers, and several chunks can be in flight per thread
// without holding a register: this is what keeps enough bytes in flight to cover the HBM latency.
constexpr int kSlotBytes = 80;

// 16-byte copy of packed weights. Without an L2 cache-policy operand: the copy with an evict-first policy
// (cp.async ... L2::cache_hint) made a decode step ~3 % faster while every projection used this ring, but the kernel
// raised "illegal instruction" twice with it, in different instances and only in some builds (512 threads at M = 16;
// 256 threads with K slices as a cluster at M = 1); reading did not show why, and nothing else in the ring path takes a
// register operand that can be invalid, so no copy carries the policy any more. The register path's plain loads keep it.
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void *src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_8(uint32_t dst, const void *src)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void *src)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait(int pending)
{
    switch (pending) {  // the instruction takes an immediate
    case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    }
}

__device__ __forceinline__ void fetch_chunk_async(const GemvParams &p, int ch, int t, int c, bool col_ok, unsigned char *slot)
{
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(slot);
    const uint32_t *base = p.qw + (int64_t)(ch * 16 + t) * p.N + c;
    const int64_t step = (int64_t)4 * p.N;
    const uint4 zero4 = make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int st = 0; st < 4; st++) {
        if (col_ok && ch * 16 + st * 4 + t < p.pack_rows) cp_async_16(dst + st * 16, base + st * step);
        else *reinterpret_cast<uint4 *>(slot + st * 16) = zero4;
    }
    const int G = p.group_chunks == 1 ? ch : ch / p.group_chunks;
    if (col_ok) {
        cp_async_8(dst + 64, p.sc + (int64_t)G * p.N + c);
        if (p.qz) cp_async_4(dst + 72, p.qz + (int64_t)G * p.zcols + (c >> 3));
        else *reinterpret_cast<uint32_t *>(slot + 72) = 0x77777777u;  // stored zero 7 -> zero point 8
    } else {
        *reinterpret_cast<uint2 *>(slot + 64) = make_uint2(0u, 0u);
        *reinterpret_cast<uint32_t *>(slot + 72) = 0x77777777u;
    }
}

__device__ __forceinline__ void read_slot(const unsigned char *slot, int c, ChunkRegs &r)
{
#pragma unroll
    for (int st = 0; st < 4; st++) r.w[st] = *reinterpret_cast<const uint4 *>(slot + st * 16);
    r.s = *reinterpret_cast<const uint2 *>(slot + 64);
    r.z = *reinterpret_cast<const uint32_t *>(slot + 72) >> ((c & 7) * 4);
}

// ---- unpack + MMA of one chunk ------------------------------------------------------------------------------
// A nibble masked in place is already an fp16 number: bits 0-3 of a 16-bit lane are the subnormal q * 2^-24,
// bits 4-7 are 16 q * 2^-24. So (w & 0x000f000f) is the half2 (q0, q4) * 2^-24 and (w & 0x00f000f0) is
// (q1, q5) * 2^-20, the same for w >> 8: one shift and four single-constant ANDs per word, no conversion at
// all. The tensor core multiplies subnormals exactly and accumulates in f32, so
//     sum_k x_k q_k = 2^24 (acc_even + acc_odd / 16)          exactly up to f32 accumulation,
// and the zero point comes off once per chunk through the chunk's activation sum S:
//     sum_k x_k (q_k - z) = 2^24 (acc_even + acc_odd / 16) - z S.
// The staged activation row holds (x0,x4)(x2,x6)(x1,x5)(x3,x7): .x/.y feed the even-nibble MMA, .z/.w the odd
// one. With f32 activations (EXACT) a second row holds the fp16 remainders x - fp16(x) and doubles the MMAs.
// xsum[m * chunks_cta + chunk] = sum of that chunk of row m.
template <int MB, bool EXACT>
__device__ __forceinline__ void compute_chunk(const GemvParams &p, const ChunkRegs &r, int rl0, int g, int t, const uint4 *xs_hi,
                                              const uint4 *xs_lo, const float *xsum, int chunk_local, int chunks_cta,
                                              float (&tot)[MB][2][4])
{
    float ae[MB][2][4], ao[MB][2][4];
#pragma unroll
    for (int mb = 0; mb < MB; mb++)
#pragma unroll
        for (int s = 0; s < 2; s++)
#pragma unroll
            for (int i = 0; i < 4; i++) ae[mb][s][i] = 0.f, ao[mb][s][i] = 0.f;
#pragma unroll
    for (int st = 0; st < 4; st++) {
        const int rl = rl0 + st * 4;
        uint32_t e0[4], e1[4], o0[4], o1[4];  // per column j: (q0,q4) (q2,q6) and 16 x (q1,q5) (q3,q7), in units of 2^-24
        const uint32_t wv[4] = {r.w[st].x, r.w[st].y, r.w[st].z, r.w[st].w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t w8 = wv[j] >> 8;
            e0[j] = wv[j] & 0x000f000fu;
            o0[j] = wv[j] & 0x00f000f0u;
            e1[j] = w8 & 0x000f000fu;
            o1[j] = w8 & 0x00f000f0u;
        }
#pragma unroll
        for (int mb = 0; mb < MB; mb++) {
            const int m = min(mb * 8 + g, p.M);  // row M is a staged row of zeros; so are rows past the k-slice
            const uint4 xb = xs_hi[m * p.xs_stride + rl];
            mma_16816(ae[mb][0], e0[0], e0[1], e1[0], e1[1], xb.x, xb.y);
            mma_16816(ao[mb][0], o0[0], o0[1], o1[0], o1[1], xb.z, xb.w);
            mma_16816(ae[mb][1], e0[2], e0[3], e1[2], e1[3], xb.x, xb.y);
            mma_16816(ao[mb][1], o0[2], o0[3], o1[2], o1[3], xb.z, xb.w);
            if constexpr (EXACT) {
                const uint4 xl = xs_lo[m * p.xs_stride + rl];
                mma_16816(ae[mb][0], e0[0], e0[1], e1[0], e1[1], xl.x, xl.y);
                mma_16816(ao[mb][0], o0[0], o0[1], o1[0], o1[1], xl.z, xl.w);
                mma_16816(ae[mb][1], e0[2], e0[3], e1[2], e1[3], xl.x, xl.y);
                mma_16816(ao[mb][1], o0[2], o0[3], o1[2], o1[3], xl.z, xl.w);
            }
        }
    }
    const float2 s01 = __half22float2(u32_as_h2(r.s.x)), s23 = __half22float2(u32_as_h2(r.s.y));
    const float scale[4] = {s01.x, s01.y, s23.x, s23.y};
    float sz[4];  // scale * zero point
#pragma unroll
    for (int j = 0; j < 4; j++) sz[j] = scale[j] * (float)(((r.z >> (4 * j)) & 15u) + 1u);
#pragma unroll
    for (int mb = 0; mb < MB; mb++) {
        // this thread's accumulator columns are the activation rows m = mb*8 + 2t, 2t+1
        float sx[2];
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int m = mb * 8 + 2 * t + i;
            sx[i] = m < p.M ? xsum[m * chunks_cta + chunk_local] : 0.f;
        }
#pragma unroll
        for (int s = 0; s < 2; s++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int col = 2 * s + (i >> 1);  // accumulator rows g / g+8 of set s are columns c+2s / c+2s+1
                const float v = fmaf(ao[mb][s][i], 0.0625f, ae[mb][s][i]) * 16777216.f;
                tot[mb][s][i] = fmaf(scale[col], v, fmaf(-sz[col], sx[i & 1], tot[mb][s][i]));
            }
    }
}

}  // namespace wb
