// Streaming int4 GEMV for the bandwidth-bound shapes: 1 <= M <= 4 rows, whole 128-k chunks, N % 32 == 0.
//
// Same arithmetic as gptq_gemv_mma_kernel (gemv.cu): packed words straight from the checkpoint layout, nibbles used
// in place as fp16 subnormals, warp-level m16n8k16 MMA with the weight tile as the 16-row operand, zero point applied
// through the per-chunk activation sums, scales in f32 per group. What differs is everything around the MMAs, because
// at HBM speed an SM has ~120 issue slots per scheduler for each 2 KB chunk and the general kernel spends 450:
//   * no bounds: the host only picks this kernel when every chunk is whole and every column tile is full, so the
//     loop has no predicates and no zero filling;
//   * f32 activations cost no extra MMAs: only batch rows occupy the 8 columns of the activation operand, so the hi
//     and lo fp16 halves of row j sit in columns 2j and 2j + 1 of the SAME operand and one MMA produces both partial
//     sums, which land in one thread (accumulator elements 2t, 2t + 1) and are added there;
//   * weights go from global memory into registers with 128-bit streaming loads, two chunks ahead (issuing a plain
//     load costs a third of a cp.async to shared memory, and nothing has to be read back from a ring);
//   * accumulators start from the zero register instead of being cleared, and the per-chunk epilogue touches the four
//     outputs a thread owns, not sixteen;
//   * CTAs are persistent over column tiles (two CTAs per SM, one wave): the activations are staged once per CTA and the
//     register prefetch runs on across tile boundaries, so the loads never drain between tiles.
// A TMA-fed variant of this kernel (one elected thread copying [16 rows x 32 columns] boxes into a ring of shared-memory
// slots, persistent over column tiles) was built and measured slower (16.7 us against 14.0 us on K = 3584, N = 18944),
// so the loads stay per thread.
#include "common.cuh"
#include "gemv_core.cuh"

namespace wb {

namespace {

// D = A * B (C = 0): starts an accumulator without a clearing pass.
__device__ __forceinline__ void mma_16816_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

struct StreamRegs {
    uint4 w[4];  // packed words: rows 4 * st + t of the chunk, columns c .. c + 3
    uint2 s;     // four fp16 scales
    uint32_t z;  // the zero word of columns c .. c + 7 (or 0x77777777)
};

__device__ __forceinline__ void stream_fetch(const GemvParams &p, const uint32_t *wbase, int64_t row_step, int ch, int c, StreamRegs &r)
{
    const uint32_t *src = wbase + (int64_t)ch * 16 * p.N;
#pragma unroll
    for (int st = 0; st < 4; st++) r.w[st] = ldg_stream_v4(src + st * row_step);
    const int G = p.group_chunks == 1 ? ch : ch / p.group_chunks;
    r.s = *reinterpret_cast<const uint2 *>(p.sc + (int64_t)G * p.N + c);
    r.z = p.qz ? p.qz[(int64_t)G * p.zcols + (c >> 3)] : 0x77777777u;
}

}  // namespace

// grid (resident CTAs walking the column tiles of 32, K slices); block 256 = 8 warps over the chunks of the slice.
// HAS_LO: f32 activations.
template <bool HAS_LO>
__global__ void __launch_bounds__(256, 2) gptq_gemv_stream_kernel(const GemvParams p)
{
    extern __shared__ uint4 smem_u4[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int ch_begin = blockIdx.y * p.chunks_per_split;
    const int ch_end = min(p.chunks, ch_begin + p.chunks_per_split);
    const int chunks_cta = ch_end - ch_begin;
    const int rows_pad = chunks_cta * 16, row_begin = ch_begin * 16;
    // Column tiles are persistent: this CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ... so the activations are
    // staged once per CTA and the prefetch runs on across tile boundaries.
    const int col_tiles = p.N >> 5;
    const int tiles_cta = (int)blockIdx.x < col_tiles ? (col_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;

    // operand rows: hi of batch row j at index j, lo at M + j, then one row of zeros
    const int n_rows = HAS_LO ? 2 * p.M : p.M;
    uint4 *xs = smem_u4;
    float *xsum = reinterpret_cast<float *>(smem_u4 + (size_t)(n_rows + 1) * p.xs_stride);  // [M][chunks_cta]
    float *red = xsum + ((p.M * chunks_cta + 3) & ~3);                                       // [8 warps][32 lanes][4]

    // This warp's work is the sequence (tile j, chunk ch_begin + warp + 8 i); `pf` is the position of the next request.
    // The first three chunks are requested before anything else (and before the wait on the previous kernel), so that
    // three are in flight while the activations are staged; in the loop two are in flight behind the one in use.
    const uint32_t *wrow = p.qw + (int64_t)t * p.N + 4 * g;
    const int64_t row_step = (int64_t)4 * p.N;
    const int ch_first = ch_begin + warp;  // every slice holds >= 8 chunks (checked on the host): every warp has one
    auto fetch_at = [&](int j, int ch, StreamRegs &r) {
        const int tile = (int)blockIdx.x + j * (int)gridDim.x;
        stream_fetch(p, wrow + tile * 32, row_step, ch, tile * 32 + 4 * g, r);
    };
    // Three register buffers, used in turn by a loop unrolled three times: a buffer is refilled right after its chunk
    // has been consumed and nothing is ever moved from one buffer to another (a move would wait for the load that it
    // reads), so a warp has two chunks in flight while it computes and three while it waits or stages.
    StreamRegs buf[3];
    int pf_j = 0, pf_ch = ch_first;
    auto pf_advance = [&]() {
        pf_ch += 8;
        if (pf_ch >= ch_end) pf_ch = ch_first, pf_j++;
    };
#pragma unroll
    for (int u = 0; u < 3; u++) {
        if (pf_j < tiles_cta) fetch_at(pf_j, pf_ch, buf[u]);
        pf_advance();
    }
    pdl_sync();

    // ---- stage the activations in the MMA's k-slot order (x0,x4)(x2,x6)(x1,x5)(x3,x7), hi and lo rows ----
    for (int rl = tid; rl < rows_pad; rl += 256) xs[n_rows * p.xs_stride + rl] = make_uint4(0, 0, 0, 0);
    for (int idx = tid; idx < p.M * rows_pad; idx += 256) {
        const int m = idx / rows_pad, rl = idx - m * rows_pad;
        const int64_t k0 = (int64_t)(row_begin + rl) * 8;
        float v[8];
        if (p.x_f16) {
            const uint4 raw = *reinterpret_cast<const uint4 *>((const __half *)p.x + (int64_t)m * p.K + k0);
            const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float2 f = __half22float2(h[j]);
                v[2 * j] = f.x, v[2 * j + 1] = f.y;
            }
        } else {
            const float4 a = *reinterpret_cast<const float4 *>((const float *)p.x + (int64_t)m * p.K + k0);
            const float4 b = *reinterpret_cast<const float4 *>((const float *)p.x + (int64_t)m * p.K + k0 + 4);
            v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
        }
        __half hi[8];
#pragma unroll
        for (int j = 0; j < 8; j++) hi[j] = __float2half_rn(v[j]);
        uint4 o;
        o.x = h2_as_u32(__halves2half2(hi[0], hi[4]));
        o.y = h2_as_u32(__halves2half2(hi[2], hi[6]));
        o.z = h2_as_u32(__halves2half2(hi[1], hi[5]));
        o.w = h2_as_u32(__halves2half2(hi[3], hi[7]));
        xs[m * p.xs_stride + rl] = o;
        // sum of the staged operand values of this 8-k slot, in a fixed order (the zero point multiplies it)
        auto sum8 = [](const __half (&h)[8]) {
            return ((__half2float(h[0]) + __half2float(h[4])) + (__half2float(h[2]) + __half2float(h[6]))) +
                   ((__half2float(h[1]) + __half2float(h[5])) + (__half2float(h[3]) + __half2float(h[7])));
        };
        float sx = sum8(hi);
        if constexpr (HAS_LO) {
            __half lo[8];
#pragma unroll
            for (int j = 0; j < 8; j++) lo[j] = __float2half_rn(v[j] - __half2float(hi[j]));
            o.x = h2_as_u32(__halves2half2(lo[0], lo[4]));
            o.y = h2_as_u32(__halves2half2(lo[2], lo[6]));
            o.z = h2_as_u32(__halves2half2(lo[1], lo[5]));
            o.w = h2_as_u32(__halves2half2(lo[3], lo[7]));
            xs[(p.M + m) * p.xs_stride + rl] = o;
            sx += sum8(lo);
        }
        // per (row m, chunk): the 16 slots of a chunk sit in one half-warp (rows_pad % 16 == 0), so the chunk's sum is
        // a shuffle reduction in this same pass
        const unsigned half_mask = (lane & 16) ? 0xffff0000u : 0x0000ffffu;
#pragma unroll
        for (int o2 = 8; o2 > 0; o2 >>= 1) sx += __shfl_xor_sync(half_mask, sx, o2);
        if ((rl & 15) == 0) xsum[m * chunks_cta + (rl >> 4)] = sx;
    }
    __syncthreads();

    // ---- main loop: this warp's chunks ch_begin + warp, + 8, ... ----
    // operand row of this lane: column n = g of the activation operand is hi (g even) / lo (g odd) of batch row g / 2
    const int bj = g >> 1;
    const int brow = bj < p.M ? ((g & 1) ? (HAS_LO ? p.M + bj : n_rows) : bj) : n_rows;
    const uint4 *xrow = xs + (size_t)brow * p.xs_stride + t;
    const float *xsum_t = xsum + (t < p.M ? t : 0) * chunks_cta;  // this thread's outputs belong to batch row t
    __shared__ int is_last;
    const int zshift = ((4 * g) & 7) * 4;  // nibble of column 4 g in its zero word (tiles start at multiples of 32)

    // one 128-k chunk of one column tile: 16 MMAs, then scale and zero point
    auto chunk_step = [&](const StreamRegs &cur, int ch, float (&tot)[4]) {
        const int rl0 = (ch - ch_begin) * 16;
        float ae[2][4], ao[2][4];
#pragma unroll
        for (int st = 0; st < 4; st++) {
            uint32_t e0[4], e1[4], o0[4], o1[4];
            const uint32_t wv[4] = {cur.w[st].x, cur.w[st].y, cur.w[st].z, cur.w[st].w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t w8 = wv[i] >> 8;
                e0[i] = wv[i] & 0x000f000fu;
                o0[i] = wv[i] & 0x00f000f0u;
                e1[i] = w8 & 0x000f000fu;
                o1[i] = w8 & 0x00f000f0u;
            }
            const uint4 xb = xrow[rl0 + st * 4];
            if (st == 0) {
                mma_16816_zero(ae[0], e0[0], e0[1], e1[0], e1[1], xb.x, xb.y);
                mma_16816_zero(ao[0], o0[0], o0[1], o1[0], o1[1], xb.z, xb.w);
                mma_16816_zero(ae[1], e0[2], e0[3], e1[2], e1[3], xb.x, xb.y);
                mma_16816_zero(ao[1], o0[2], o0[3], o1[2], o1[3], xb.z, xb.w);
            } else {
                mma_16816(ae[0], e0[0], e0[1], e1[0], e1[1], xb.x, xb.y);
                mma_16816(ao[0], o0[0], o0[1], o1[0], o1[1], xb.z, xb.w);
                mma_16816(ae[1], e0[2], e0[3], e1[2], e1[3], xb.x, xb.y);
                mma_16816(ao[1], o0[2], o0[3], o1[2], o1[3], xb.z, xb.w);
            }
        }
        // accumulator elements (0, 1) = (hi, lo) of column c + 2s, (2, 3) of column c + 2s + 1
        const float2 s01 = __half22float2(u32_as_h2(cur.s.x)), s23 = __half22float2(u32_as_h2(cur.s.y));
        const float scale[4] = {s01.x, s01.y, s23.x, s23.y};
        const uint32_t zw = cur.z >> zshift;
        const float sx = xsum_t[ch - ch_begin];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int s = i >> 1, e = (i & 1) * 2;
            const float q = fmaf(ao[s][e], 0.0625f, ae[s][e]) + fmaf(ao[s][e + 1], 0.0625f, ae[s][e + 1]);
            const float zp = (float)(((zw >> (4 * i)) & 15u) + 1u);
            tot[i] = fmaf(scale[i], fmaf(q, 16777216.f, -zp * sx), tot[i]);
        }
    };

    // end of a column tile: reduce over the 8 warps (fixed order), then write / split-K through the workspace
    auto tile_end = [&](int j, const float (&tot)[4]) {
        const int tile = (int)blockIdx.x + j * (int)gridDim.x;
        *reinterpret_cast<float4 *>(red + (warp * 32 + lane) * 4) = make_float4(tot[0], tot[1], tot[2], tot[3]);
        __syncthreads();
        const int n_base = tile * 32;
        const int outputs = p.M * 32;
        if (tid < outputs) {
            const int m = tid >> 5, col = tid & 31;
            const int src = ((col >> 2) * 4 + m) * 4 + (col & 3);
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < 8; w++) v += red[w * 128 + src];
            const int n = n_base + col;
            if (p.S == 1) {
                if (p.bias) v += p.bias[n];
                if (p.out_f16) ((__half *)p.out)[(int64_t)m * p.N + n] = __float2half_rn(v);
                else ((float *)p.out)[(int64_t)m * p.N + n] = v;
            } else {
                p.partial[((int64_t)blockIdx.y * p.M + m) * p.N + n] = v;
            }
        }
        if (p.S > 1) {
            // the last slice to arrive for this tile adds the slices in slice order and the bias once
            __threadfence();
            __syncthreads();
            if (tid == 0) is_last = (atomicAdd(&p.counters[tile], 1u) == (unsigned)(p.S - 1));
            __syncthreads();
            if (is_last) {
                __threadfence();
                if (tid < outputs) {
                    const int m = tid >> 5, n = n_base + (tid & 31);
                    float v = 0.f;
                    for (int s = 0; s < p.S; s++) v += __ldcg(&p.partial[((int64_t)s * p.M + m) * p.N + n]);
                    if (p.bias) v += p.bias[n];
                    if (p.out_f16) ((__half *)p.out)[(int64_t)m * p.N + n] = __float2half_rn(v);
                    else ((float *)p.out)[(int64_t)m * p.N + n] = v;
                }
                if (tid == 0) p.counters[tile] = 0u;
            }
        }
        __syncthreads();  // red and is_last are reused by the next tile
    };

    // Every warp of the CTA meets the same number of tile ends (one per tile), so the barriers inside tile_end match
    // although each warp reaches them from its own place in the unrolled loop.
    int j = 0, ch = ch_first;
    float tot[4] = {0.f, 0.f, 0.f, 0.f};  // columns c .. c + 3 of batch row t
    while (j < tiles_cta) {
#pragma unroll
        for (int u = 0; u < 3; u++) {
            if (j >= tiles_cta) break;
            chunk_step(buf[u], ch, tot);
            if (pf_j < tiles_cta) fetch_at(pf_j, pf_ch, buf[u]);
            pf_advance();
            ch += 8;
            if (ch >= ch_end) {
                tile_end(j, tot);
                tot[0] = tot[1] = tot[2] = tot[3] = 0.f;
                ch = ch_first, j++;
            }
        }
    }
}

// ---- host side -------------------------------------------------------------------------------------------------
// Dynamic shared memory of one CTA: the staged operand rows (hi, lo for f32 activations, one row of zeros), the
// per-chunk activation sums and the cross-warp reduction buffer.
static size_t gemv_stream_smem(int64_t M, int cps, bool has_lo)
{
    const size_t rows = (size_t)(has_lo ? 2 * M : M) + 1;
    return rows * (size_t)(cps * 16 + 4) * 16 + (size_t)((M * cps + 3) & ~3) * 4 + 8 * 32 * 4 * 4;
}

// Whole chunks and tiles only; enough chunks per slice that streaming (not latency) is what matters; every one of
// the 8 warps must own a chunk in EVERY slice, the shorter last one included (a warp without one would prefetch past
// its slice); two CTAs per SM must fit the shared memory; one arrival counter per column tile when K is split.
bool gemv_stream_supports(const Weight &w, int64_t M, int chunks, int S, bool has_lo)
{
    if (w.kind != WeightKind::Gptq || M < 1 || M > 4 || w.K % 128 != 0 || w.N % 32 != 0 || w.group % 128 != 0) return false;
    if (S < 1 || S > chunks) return false;
    const int cps = (chunks + S - 1) / S;
    if ((chunks + cps - 1) / cps != S) return false;  // would leave an empty slice
    const int last = chunks - (S - 1) * cps;
    return cps >= 20 && last >= 8 && w.N / 32 <= kMaxCounters && gemv_stream_smem(M, cps, has_lo) <= 100 * 1024;
}

// Launch grid: what is resident at once (two CTAs per SM), evened out so that every CTA walks the same number of tiles.
int gemv_stream_grid_x(int sm_count, int64_t N, int S)
{
    const int col_tiles = (int)(N / 32);
    int capacity = sm_count * 2 / S;
    if (capacity < 1) capacity = 1;
    const int waves = (col_tiles + capacity - 1) / capacity;
    return (col_tiles + waves - 1) / waves;
}

int launch_gemv_stream(wb_context *ctx, const Weight &w, const GemvParams &gp, bool has_lo)
{
    GemvParams p = gp;
    if (!gemv_stream_supports(w, p.M, p.chunks, p.S, has_lo))
        return fail(WB_ERR_UNSUPPORTED, "the streaming GEMV does not take this shape or split");
    const int cps = p.chunks_per_split;
    p.xs_stride = cps * 16 + 4;
    const size_t smem = gemv_stream_smem(p.M, cps, has_lo);
    dim3 grid((unsigned)gemv_stream_grid_x(ctx->sm_count, w.N, p.S), (unsigned)p.S);
    cudaError_t e;
    if (has_lo) {
        cudaFuncSetAttribute(gptq_gemv_stream_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        e = launch_pdl(gptq_gemv_stream_kernel<true>, grid, dim3(256), smem, ctx->stream, p);
    } else {
        cudaFuncSetAttribute(gptq_gemv_stream_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        e = launch_pdl(gptq_gemv_stream_kernel<false>, grid, dim3(256), smem, ctx->stream, p);
    }
    ctx->launches++;
    WB_CUDA(e);
    return WB_OK;
}

}  // namespace wb
