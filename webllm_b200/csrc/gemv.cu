// Decode-side linear kernels: the fused int4 GEMV / small-batch kernel, the fp16 dense GEMV (tied
// lm_head) and the shape-agnostic kernel for ragged sizes. Together with gemm_tc.cu they replace the four
// WGSL kernels behind QwenGpt.gemm (src/model/qwen.ts:568-618): gemm_gemv_f16.wgsl,
// gemm_gemv_split_f16.wgsl, gemm_gemv_split_reduce.wgsl and gemm_nt_f16_from_f32.wgsl.
#include <algorithm>
#include <atomic>

#include "common.cuh"

namespace wb {

// =====================================================================================================
// Fused int4 GEMV for 1 <= M <= 32  (C[M,N] = A[M,K] . W[N,K]^T + bias)
//
// HBM-bound: every packed word is read exactly once, with 16-byte cp.async copies straight from the
// checkpoint layout qweight[K/8, N] (a warp reads 4 packed rows x 32 columns = four full 128-byte lines per
// copy instruction) into a per-thread ring in shared memory, so that several chunks per thread are in flight
// without holding registers. A scalar-FMA unpack needs >= 3 issue slots per weight, which at 2 weights per
// byte is more than the SMs can issue at HBM speed, so the products run on the warp-level tensor-core MMA
// (m16n8k16, fp16 in, f32 accumulate) with the weight tile as the 16-row operand and up to 8 activation
// rows as the 8-column operand.
//
//   * unpack: none to speak of. w & 0x000f000f is, read as half2, the pair of fp16 SUBNORMALS
//     (q_j, q_{j+4}) * 2^-24, and w & 0x00f000f0 the pair 16 * (q_{j+1}, q_{j+5}) * 2^-24 (the same two masks on
//     w >> 8 give the other four nibbles). The MMA multiplies subnormals exactly; the even and odd nibbles go
//     to separate f32 accumulators and are recombined as 2^24 * (acc_even + acc_odd / 16). The zero point
//     never touches the weights: sum_k (q_k - z) x_k = sum_k q_k x_k - z * sum_k x_k, with the per-chunk
//     activation sums computed once while the activations are staged. Per-group scales are applied in f32 to
//     the group's partial sum, so no product is ever rounded to fp16.
//   * the MMA only needs the two operands to agree on which k sits in which slot, so the nibble order that
//     the masks produce is used as is and the activations are staged in shared memory in the same order:
//     16 bytes per (row m, packed row r) holding (x0,x4)(x2,x6)(x1,x5)(x3,x7) as half2, plus a row of zeros
//     that lanes without a batch row read (no predicates in the loop).
//   * f32 activations are split into hi + lo fp16 halves (two MMAs per tile), which keeps ~22 bits of
//     them: the reference's GEMV reads A as f32 (gemm_gemv_f16.wgsl:45-58). fp16 activations need one.
//   * column tiles are persistent: the grid is what is resident at once and each CTA walks tiles
//     blockIdx.x, blockIdx.x + gridDim.x, ..., the ring running ahead across tile boundaries.
//   * split-K: grid.y slices of whole 128-k chunks. Each slice writes its partial tile to the workspace;
//     the last CTA to arrive for a column tile (arrival counter, no waiting) adds the slices in slice
//     order and the bias once, so the result does not depend on scheduling
//     (cf. gemm_gemv_split_reduce.wgsl:36-38).
//   * decode fusions (M <= 8, f32 activations): the staging step can compute rmsnorm(x + delta) * w or
//     silu(x) * up instead of copying x (GemvPrologue), and one thread per CTA can ask the L2 for the weight
//     of a following call (cp.async.bulk.prefetch.L2) so that call starts on L2 hits.
// =====================================================================================================

}  // namespace wb

#include "gemv_core.cuh"

namespace wb {

// DIRECT (MB == 1 only): every warp holds at most one chunk of one tile and loads it straight into registers with
// 128-bit streaming loads instead of going through the cp.async ring. Issuing six cp.async per thread costs ~0.4 us
// more than plain loads. It needs more registers (122 to 128: two CTAs per SM instead of three), so it is used where the
// launch has at most one CTA per SM: the split-K down projection and, since every kernel releases its successor only
// after its own wait (the prologue then has just one kernel to hide under), the unsplit q|k|v and o projections of a
// decode step (0.541 -> 0.528 ms per step). The 304-CTA gate|up launch needs three CTAs per SM and keeps the ring.
template <int MB, bool EXACT, bool DIRECT>
__global__ void __launch_bounds__(MB == 1 ? 256 : 512, MB == 1 ? (DIRECT ? 2 : 3) : 1) gptq_gemv_mma_kernel(const GemvParams p)
{
    extern __shared__ uint4 smem_u4[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int wn = warp % p.wn, wk = warp / p.wn;
    const int nthreads = blockDim.x;

    const int ch_begin = blockIdx.y * p.chunks_per_split;
    const int ch_end = min(p.chunks, ch_begin + p.chunks_per_split);
    const int row_begin = ch_begin * 16;
    const int rows_cta = max(0, min(p.pack_rows, ch_end * 16) - row_begin);

    uint4 *xs_hi = smem_u4;
    // rows 0..M-1 are the activations, row M is all zeros: lanes whose batch row does not exist read it
    uint4 *xs_lo = smem_u4 + (size_t)(p.M + 1) * p.xs_stride;                           // EXACT only
    float *xsum = reinterpret_cast<float *>(smem_u4 + (size_t)(p.M + 1) * p.xs_stride * (EXACT ? 2 : 1));
    const int chunks_cta = ch_end - ch_begin;

    // Work of this CTA: column tiles blockIdx.x, blockIdx.x + gridDim.x, ... (wn * 32 columns each) of its k-slice.
    // Within a tile a warp owns 32 columns and every wk-th chunk; a thread owns columns c .. c+3 (N % 4 == 0: in
    // or out of the matrix together). The grid is sized to what is resident at once, so no partial second wave.
    const int n_tiles = (p.N + p.wn * 32 - 1) / (p.wn * 32);
    const int tiles_cta = (int)blockIdx.x < n_tiles ? (n_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const int n_i = ch_end > ch_begin + wk ? (ch_end - ch_begin - wk + p.wk - 1) / p.wk : 0;  // this warp's chunks per tile
    auto col_of = [&](int j) { return (((int)blockIdx.x + j * (int)gridDim.x) * p.wn + wn) * 32 + 4 * g; };
    // cp.async ring over the flattened (tile, chunk) sequence of this warp: `stages` slots per thread,
    // stages - 1 chunks requested before the activations are staged and one more per iteration, so that
    // several chunks per thread are always in flight, also across tile boundaries.
    unsigned char *ring = reinterpret_cast<unsigned char *>(smem_u4) + p.ring_off + (size_t)tid * kSlotBytes;
    const size_t stage_stride = (size_t)nthreads * kSlotBytes;
    int rq_tile = 0, rq_i = 0;
    auto request = [&](int slot) {
        if (rq_tile < tiles_cta && n_i > 0) {
            const int cc = col_of(rq_tile);
            fetch_chunk_async(p, ch_begin + wk + rq_i * p.wk, t, cc, cc < p.N, ring + slot * stage_stride);
            if (++rq_i == n_i) rq_i = 0, rq_tile++;
        }
        cp_async_commit();
    };
    ChunkRegs pre;
    if constexpr (DIRECT) {
        if (tiles_cta > 0 && n_i > 0) {
            const int cc = col_of(0);
            fetch_chunk(p, ch_begin + wk, t, cc, cc < p.N, pre);
        }
    } else {
        for (int s = 0; s < p.stages - 1; s++) request(s);
    }
    if (p.pf_bytes && tid == 0) {
        // L2 prefetch of the weight that a following call will stream: each CTA asks for one slice, so the whole
        // matrix is on its way while this kernel (and the small kernels after it) run, and that call finds its
        // first chunks in L2 instead of paying the HBM and page-walk latency on its critical path.
        const unsigned ncta = gridDim.x * gridDim.y, id = blockIdx.y * gridDim.x + blockIdx.x;
        const unsigned slice = ((p.pf_bytes + ncta - 1) / ncta + 15u) & ~15u;
        const unsigned long long off = (unsigned long long)id * slice;
        if (off < p.pf_bytes) {
            const unsigned n = min(slice, (unsigned)(p.pf_bytes - off));
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.pf_ptr + off), "r"(n) : "memory");
        }
    }
    __shared__ uint64_t cl_bar;
    // (cl_async == 2, a test's setting: the barrier is armed for 4 bytes more than are sent, so the receiver's wait runs out)
    if (p.cl_async) cluster_merge_init(&cl_bar, (uint32_t)((p.S - 1) * p.M * p.wn * 32 * 4) + (p.cl_async == 2 ? 4u : 0u), blockIdx.y == 0);
    // The bias is a constant too. A thread's column within a tile is fixed when the block size is a multiple of the tile
    // width; its bias value for the CTA's first tile is requested here, so that the load does not stand in front of the
    // final store (it measured ~0.5 us there on the q|k|v projection of a decode step).
    const int tile_cols_b = p.wn * 32;
    const bool bias_pre_ok = p.bias != nullptr && nthreads % tile_cols_b == 0;
    float bias_pre = 0.f;
    if (bias_pre_ok) {
        const int n = (int)blockIdx.x * tile_cols_b + tid % tile_cols_b;
        if (n < p.N) bias_pre = p.bias[n];
    }
    pdl_sync();  // weights are constant: their first chunks are requested while the previous kernel still runs
    // ---- stage the activations (see the two branches) ----
    const int rows_pad = chunks_cta * 16;
    __shared__ float pro_red[16];
    __shared__ float pro_rstd[8];
    // Decode fast path: one row of activations and at most one packed row (8 values) per thread. Everything a thread
    // needs is loaded once into registers, the rmsnorm statistic is reduced across the CTA (K is not split when the
    // norm is fused), the operand halves go to shared memory and the per-chunk sums come from a half-warp shuffle:
    // one global round trip and two barriers instead of two round trips and four.
    const bool fast = p.M == 1 && rows_pad <= nthreads && (p.prologue != kPrologueRmsNorm || gridDim.y == 1);
    if (fast) {
        const int rl = tid;
        const bool has = rl < rows_pad, real = rl < rows_cta;
        const int64_t k0 = (int64_t)(row_begin + rl) * 8;
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; j++) v[j] = 0.f;
        auto load8 = [&](const float *src, float (&dst)[8]) {
            const float4 a = *reinterpret_cast<const float4 *>(src), b = *reinterpret_cast<const float4 *>(src + 4);
            dst[0] = a.x, dst[1] = a.y, dst[2] = a.z, dst[3] = a.w, dst[4] = b.x, dst[5] = b.y, dst[6] = b.z, dst[7] = b.w;
        };
        if (has) xs_hi[p.xs_stride + rl] = make_uint4(0, 0, 0, 0);  // the zero row (index M = 1)
        if constexpr (EXACT)
            if (has) xs_lo[p.xs_stride + rl] = make_uint4(0, 0, 0, 0);
        if (p.prologue == kPrologueRmsNorm) {
            float w8[8], d8[8];
#pragma unroll
            for (int j = 0; j < 8; j++) w8[j] = 0.f, d8[j] = 0.f;
            if (real) {
                load8((const float *)p.x + k0, v);
                if (p.delta) load8(p.delta + k0, d8);
                load8(p.norm_w + k0, w8);
            }
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < 8; j++) v[j] += d8[j], ss = fmaf(v[j], v[j], ss);
            if (real && p.delta && p.x_out != nullptr && blockIdx.x == 0) {
                *reinterpret_cast<float4 *>(p.x_out + k0) = make_float4(v[0], v[1], v[2], v[3]);
                *reinterpret_cast<float4 *>(p.x_out + k0 + 4) = make_float4(v[4], v[5], v[6], v[7]);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) pro_red[warp] = ss;
            __syncthreads();
            float tsum = 0.f;
            for (int i = 0; i < (nthreads >> 5); i++) tsum += pro_red[i];  // same order in every thread
            const float rstd = rsqrtf(tsum / (float)p.K + p.eps);
#pragma unroll
            for (int j = 0; j < 8; j++) v[j] = v[j] * rstd * w8[j];
        } else if (p.prologue == kPrologueSiluMul) {
            if (real) {
                float u[8];
                load8(p.up + k0, u);
                load8((const float *)p.x + k0, v);
#pragma unroll
                for (int j = 0; j < 8; j++) v[j] = v[j] / (1.f + expf(-v[j])) * u[j];
            }
        } else if (real) {
            if (p.x_f16) {
                const uint4 raw = *reinterpret_cast<const uint4 *>((const __half *)p.x + k0);
                const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float2 f = __half22float2(h[j]);
                    v[2 * j] = f.x;
                    v[2 * j + 1] = f.y;
                }
            } else {
                load8((const float *)p.x + k0, v);
            }
        }
        if (has) {
            auto sum8 = [](const uint4 &o) {
                const float2 a = __half22float2(u32_as_h2(o.x)), b = __half22float2(u32_as_h2(o.y));
                const float2 cc = __half22float2(u32_as_h2(o.z)), d = __half22float2(u32_as_h2(o.w));
                return ((a.x + a.y) + (b.x + b.y)) + ((cc.x + cc.y) + (d.x + d.y));
            };
            __half hi[8];
#pragma unroll
            for (int j = 0; j < 8; j++) hi[j] = __float2half_rn(v[j]);
            uint4 o;
            o.x = h2_as_u32(__halves2half2(hi[0], hi[4]));
            o.y = h2_as_u32(__halves2half2(hi[2], hi[6]));
            o.z = h2_as_u32(__halves2half2(hi[1], hi[5]));
            o.w = h2_as_u32(__halves2half2(hi[3], hi[7]));
            xs_hi[rl] = o;
            float sx = sum8(o);
            if constexpr (EXACT) {
                __half lo[8];
#pragma unroll
                for (int j = 0; j < 8; j++) lo[j] = __float2half_rn(v[j] - __half2float(hi[j]));
                o.x = h2_as_u32(__halves2half2(lo[0], lo[4]));
                o.y = h2_as_u32(__halves2half2(lo[2], lo[6]));
                o.z = h2_as_u32(__halves2half2(lo[1], lo[5]));
                o.w = h2_as_u32(__halves2half2(lo[3], lo[7]));
                xs_lo[rl] = o;
                sx += sum8(o);
            }
            // rows_pad is a multiple of 16: a half-warp is wholly inside this branch or wholly outside
            const unsigned half_mask = (lane & 16) ? 0xffff0000u : 0x0000ffffu;
#pragma unroll
            for (int o2 = 8; o2 > 0; o2 >>= 1) sx += __shfl_xor_sync(half_mask, sx, o2);
            if ((rl & 15) == 0) xsum[rl >> 4] = sx;
        }
        __syncthreads();
    } else {
        // ---- fused rmsnorm: the row statistic over the whole of K (not only this CTA's slice), fixed summation order
        if (p.prologue == kPrologueRmsNorm) {
            const bool writer = p.x_out != nullptr && blockIdx.x == 0 && blockIdx.y == 0;
            for (int m = 0; m < p.M; m++) {
                const float *xr = (const float *)p.x + (int64_t)m * p.K;
                float ss = 0.f;
                for (int k = tid * 4; k < p.K; k += nthreads * 4) {
                    float4 a = *reinterpret_cast<const float4 *>(xr + k);
                    if (p.delta) {
                        const float4 d = *reinterpret_cast<const float4 *>(p.delta + (int64_t)m * p.K + k);
                        a.x += d.x, a.y += d.y, a.z += d.z, a.w += d.w;
                        if (writer) *reinterpret_cast<float4 *>(p.x_out + (int64_t)m * p.K + k) = a;
                    }
                    ss = fmaf(a.x, a.x, ss), ss = fmaf(a.y, a.y, ss), ss = fmaf(a.z, a.z, ss), ss = fmaf(a.w, a.w, ss);
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                if (lane == 0) pro_red[warp] = ss;
                __syncthreads();
                if (tid == 0) {
                    float tsum = 0.f;
                    for (int i = 0; i < (nthreads >> 5); i++) tsum += pro_red[i];
                    pro_rstd[m] = rsqrtf(tsum / (float)p.K + p.eps);
                }
                __syncthreads();
            }
        }

        // ---- stage this slice of the activations in the MMA's k-slot order: (x0,x4)(x2,x6)(x1,x5)(x3,x7) per packed
        // row, zeros for the rows of a last partial chunk, plus the per-chunk sums used for the zero-point term ----
        for (int rl = tid; rl < rows_pad; rl += nthreads) {
            xs_hi[p.M * p.xs_stride + rl] = make_uint4(0, 0, 0, 0);
            if constexpr (EXACT) xs_lo[p.M * p.xs_stride + rl] = make_uint4(0, 0, 0, 0);
        }
        for (int idx = tid; idx < p.M * rows_pad; idx += nthreads) {
            const int m = idx / rows_pad, rl = idx - m * rows_pad;
            const int64_t k0 = (int64_t)(row_begin + rl) * 8;
            float v[8];
            auto load8 = [&](const float *src) {
                const float4 a = *reinterpret_cast<const float4 *>(src), b = *reinterpret_cast<const float4 *>(src + 4);
                v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
            };
            if (rl >= rows_cta) {
#pragma unroll
                for (int j = 0; j < 8; j++) v[j] = 0.f;
            } else if (p.prologue == kPrologueRmsNorm) {
                load8((const float *)p.x + (int64_t)m * p.K + k0);
                if (p.delta) {
                    const float4 a = *reinterpret_cast<const float4 *>(p.delta + (int64_t)m * p.K + k0);
                    const float4 b = *reinterpret_cast<const float4 *>(p.delta + (int64_t)m * p.K + k0 + 4);
                    v[0] += a.x, v[1] += a.y, v[2] += a.z, v[3] += a.w, v[4] += b.x, v[5] += b.y, v[6] += b.z, v[7] += b.w;
                }
                const float rstd = pro_rstd[m];
#pragma unroll
                for (int j = 0; j < 8; j++) v[j] = v[j] * rstd * p.norm_w[k0 + j];
            } else if (p.prologue == kPrologueSiluMul) {
                float u[8];
                load8(p.up + (int64_t)m * p.ld_x + k0);
#pragma unroll
                for (int j = 0; j < 8; j++) u[j] = v[j];
                load8((const float *)p.x + (int64_t)m * p.ld_x + k0);
#pragma unroll
                for (int j = 0; j < 8; j++) v[j] = v[j] / (1.f + expf(-v[j])) * u[j];
            } else if (p.x_f16) {
                const uint4 raw = *reinterpret_cast<const uint4 *>((const __half *)p.x + (int64_t)m * p.K + k0);
                const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float2 f = __half22float2(h[j]);
                    v[2 * j] = f.x;
                    v[2 * j + 1] = f.y;
                }
            } else {
                load8((const float *)p.x + (int64_t)m * p.K + k0);
            }
            __half hi[8];
#pragma unroll
            for (int j = 0; j < 8; j++) hi[j] = __float2half_rn(v[j]);
            uint4 o;
            o.x = h2_as_u32(__halves2half2(hi[0], hi[4]));
            o.y = h2_as_u32(__halves2half2(hi[2], hi[6]));
            o.z = h2_as_u32(__halves2half2(hi[1], hi[5]));
            o.w = h2_as_u32(__halves2half2(hi[3], hi[7]));
            xs_hi[m * p.xs_stride + rl] = o;
            if constexpr (EXACT) {
                __half lo[8];
#pragma unroll
                for (int j = 0; j < 8; j++) lo[j] = __float2half_rn(v[j] - __half2float(hi[j]));
                o.x = h2_as_u32(__halves2half2(lo[0], lo[4]));
                o.y = h2_as_u32(__halves2half2(lo[2], lo[6]));
                o.z = h2_as_u32(__halves2half2(lo[1], lo[5]));
                o.w = h2_as_u32(__halves2half2(lo[3], lo[7]));
                xs_lo[m * p.xs_stride + rl] = o;
            }
        }
        __syncthreads();
        // per (row m, chunk): sum of the staged operand values (hi + lo), 16 threads per sum, fixed order
        for (int idx = tid; idx < p.M * chunks_cta * 16; idx += nthreads) {
            const int task = idx >> 4, rr = idx & 15;
            const int m = task / chunks_cta, cl = task - m * chunks_cta;
            auto sum8 = [](const uint4 &o) {
                const float2 a = __half22float2(u32_as_h2(o.x)), b = __half22float2(u32_as_h2(o.y));
                const float2 cc = __half22float2(u32_as_h2(o.z)), d = __half22float2(u32_as_h2(o.w));
                return ((a.x + a.y) + (b.x + b.y)) + ((cc.x + cc.y) + (d.x + d.y));
            };
            float sx = sum8(xs_hi[m * p.xs_stride + cl * 16 + rr]);
            if constexpr (EXACT) sx += sum8(xs_lo[m * p.xs_stride + cl * 16 + rr]);
            // 16 consecutive lanes share a sum; a half-warp is either wholly inside this loop or wholly outside
            const unsigned half_mask = (lane & 16) ? 0xffff0000u : 0x0000ffffu;
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) sx += __shfl_xor_sync(half_mask, sx, o);
            if (rr == 0) xsum[task] = sx;
        }
        __syncthreads();
    }
    // ---- main loop over this CTA's column tiles ----
    float *red = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(smem_u4) + p.red_off);  // [wk][wn][MB*8][32]
    __shared__ int is_last;
    constexpr int J = MB * 8;
    const int tile_cols = p.wn * 32;
    const bool direct = p.S == 1;
    float *cl_part = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(smem_u4) + p.cl_off);  // [S][M * tile_cols]
    const uint32_t cl_dst = p.cluster ? cluster_map_shared(cl_part + (size_t)blockIdx.y * p.M * p.wn * 32, 0) : 0u;
    const uint32_t cl_bar_remote = p.cl_async ? cluster_map_shared(&cl_bar, 0) : 0u;
    int slot_use = 0, slot_req = p.stages - 1;
    for (int tj = 0; tj < tiles_cta; tj++) {
        const int tile = (int)blockIdx.x + tj * (int)gridDim.x;
        const int c = col_of(tj);
        float tot[MB][2][4];
#pragma unroll
        for (int mb = 0; mb < MB; mb++)
#pragma unroll
            for (int s = 0; s < 2; s++)
#pragma unroll
                for (int i = 0; i < 4; i++) tot[mb][s][i] = 0.f;
        for (int i = 0; i < n_i; i++) {
            ChunkRegs ra;
            if constexpr (DIRECT) {
                ra = pre;
            } else {
                request(slot_req);
                slot_req = slot_req + 1 == p.stages ? 0 : slot_req + 1;
                cp_async_wait(p.stages - 1);  // everything but the newest stages - 1 groups has landed
                read_slot(ring + slot_use * stage_stride, c, ra);
                slot_use = slot_use + 1 == p.stages ? 0 : slot_use + 1;
            }
            const int chunk = ch_begin + wk + i * p.wk;
            const int rl0 = chunk * 16 + t - row_begin;
            compute_chunk<MB, EXACT>(p, ra, rl0, g, t, xs_hi, xs_lo, xsum, chunk - ch_begin, chunks_cta, tot);
        }
        // reduce over the wk warps that share the column tile (fixed order), then write / split-K
#pragma unroll
        for (int mb = 0; mb < MB; mb++)
#pragma unroll
            for (int s = 0; s < 2; s++)
#pragma unroll
                for (int i = 0; i < 4; i++)
                    red[((wk * p.wn + wn) * J + (mb * 2 + s) * 4 + i) * 32 + lane] = tot[mb][s][i];
        __syncthreads();
        const int n_base = tile * tile_cols;
        const int outputs = p.M * tile_cols;
        for (int idx = tid; idx < outputs; idx += nthreads) {
            const int m = idx / tile_cols, cl_all = idx - m * tile_cols;
            const int n = n_base + cl_all;
            if (n >= p.N) continue;
            const int w_n = cl_all >> 5, cl = cl_all & 31;
            const int gg = cl >> 2, s = (cl & 3) >> 1, hi = cl & 1;
            const int mb = m >> 3, tt = (m & 7) >> 1, i = hi * 2 + (m & 1);
            const int src_lane = gg * 4 + tt, j = (mb * 2 + s) * 4 + i;
            float v = 0.f;
            for (int k = 0; k < p.wk; k++) v += red[((k * p.wn + w_n) * J + j) * 32 + src_lane];
            if (direct) {
                if (p.bias) v += (bias_pre_ok && tj == 0) ? bias_pre : p.bias[n];
                if (p.out_f16) ((__half *)p.out)[(int64_t)m * p.N + n] = __float2half_rn(v);
                else ((float *)p.out)[(int64_t)m * p.N + n] = v;
            } else if (p.cl_async) {
                if (blockIdx.y == 0) cl_part[idx] = v;
                else cluster_send_f32(cl_dst + (uint32_t)idx * 4u, v, cl_bar_remote);
            } else if (p.cluster) {
                cluster_store_f32(cl_dst + (uint32_t)idx * 4u, v);
            } else {
                p.partial[((int64_t)blockIdx.y * p.M + m) * p.N + n] = v;
            }
        }
        if (!direct && p.cluster) {
            // The S slices of this column tile are the CTAs of one cluster: each has just stored its partial tile into
            // the first CTA's shared memory; after the cluster barrier (or, with cl_async, once its mbarrier has counted
            // the other slices' bytes) that CTA adds them in slice order and the bias once. No workspace, fence or atomic,
            // and the result does not depend on scheduling.
            if (!p.cl_async) cluster_barrier();
            if (blockIdx.y == 0) {
                if (p.cl_async && tid < outputs) cluster_merge_wait(&cl_bar, p.status);  // the reader's own slice-0 value is its own store
                for (int idx = tid; idx < outputs; idx += nthreads) {
                    const int m = idx / tile_cols;
                    const int n = n_base + (idx - m * tile_cols);
                    if (n >= p.N) continue;
                    float v = 0.f;
                    for (int sl = 0; sl < p.S; sl++) v += cl_part[sl * outputs + idx];
                    if (p.bias) v += (bias_pre_ok && tj == 0) ? bias_pre : p.bias[n];
                    if (p.out_f16) ((__half *)p.out)[(int64_t)m * p.N + n] = __float2half_rn(v);
                    else ((float *)p.out)[(int64_t)m * p.N + n] = v;
                }
            }
            if (tj + 1 < tiles_cta) cluster_barrier();  // the buffer is rewritten by the next tile
        } else if (!direct) {
            // the last slice to arrive for this tile adds the slices in slice order and the bias once
            __threadfence();
            __syncthreads();
            if (tid == 0) is_last = (atomicAdd(&p.counters[tile], 1u) == (unsigned)(p.S - 1));
            __syncthreads();
            if (is_last) {
                __threadfence();
                for (int idx = tid; idx < outputs; idx += nthreads) {
                    const int m = idx / tile_cols;
                    const int n = n_base + (idx - m * tile_cols);
                    if (n >= p.N) continue;
                    float v = 0.f;
                    for (int s = 0; s < p.S; s++) v += __ldcg(&p.partial[((int64_t)s * p.M + m) * p.N + n]);
                    if (p.bias) v += (bias_pre_ok && tj == 0) ? bias_pre : p.bias[n];
                    if (p.out_f16) ((__half *)p.out)[(int64_t)m * p.N + n] = __float2half_rn(v);
                    else ((float *)p.out)[(int64_t)m * p.N + n] = v;
                }
                if (tid == 0) p.counters[tile] = 0u;  // leave the counters clean for the next call
            }
        }
        __syncthreads();  // red and is_last are reused by the next tile
    }
    cp_async_wait(0);
}

// =====================================================================================================
// fp16 dense GEMV (tied lm_head / embed, [N, K] row-major), 1 <= M <= 8. One warp per output row pair,
// lanes stride K in 16-byte chunks, activations in shared memory as f32, f32 accumulate, shuffle reduce.
// Replaces gemm_gemv_f16.wgsl for dense weights (src/gpu/kernels/gemm/gemm_gemv_f16.wgsl:36-69).
// =====================================================================================================
template <int MM>
__global__ void __launch_bounds__(256) dense_gemv_f16_kernel(const __half *__restrict__ W, const void *__restrict__ x,
                                                             void *__restrict__ out, const float *__restrict__ bias,
                                                             int M, int N, int K, int x_f16, int out_f16)
{
    extern __shared__ float xsf[];  // [M][K]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_sync();
    for (int idx = tid; idx < M * K; idx += blockDim.x)
        xsf[idx] = x_f16 ? __half2float(((const __half *)x)[idx]) : ((const float *)x)[idx];
    __syncthreads();

    constexpr int ROWS = 4;  // rows per warp pass: 4 independent 16-byte loads in flight per lane
    const int chunks = K >> 3;
    const int64_t warp_global = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
    const int64_t n0 = warp_global * ROWS;
    if (n0 >= N) return;

    float acc[ROWS][MM];
#pragma unroll
    for (int r = 0; r < ROWS; r++)
#pragma unroll
        for (int m = 0; m < MM; m++) acc[r][m] = 0.f;

    for (int ck = lane; ck < chunks; ck += 32) {
        uint4 wv[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; r++) {
            const int64_t n = n0 + r;
            wv[r] = n < N ? ldg_stream_v4(W + n * K + (int64_t)ck * 8) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int m = 0; m < MM; m++) {
            if (m >= M) break;
            const float4 xa = *reinterpret_cast<const float4 *>(&xsf[m * K + ck * 8]);
            const float4 xb = *reinterpret_cast<const float4 *>(&xsf[m * K + ck * 8 + 4]);
#pragma unroll
            for (int r = 0; r < ROWS; r++) {
                const float2 w0 = __half22float2(u32_as_h2(wv[r].x)), w1 = __half22float2(u32_as_h2(wv[r].y));
                const float2 w2 = __half22float2(u32_as_h2(wv[r].z)), w3 = __half22float2(u32_as_h2(wv[r].w));
                float a = acc[r][m];
                a = fmaf(w0.x, xa.x, a), a = fmaf(w0.y, xa.y, a), a = fmaf(w1.x, xa.z, a), a = fmaf(w1.y, xa.w, a);
                a = fmaf(w2.x, xb.x, a), a = fmaf(w2.y, xb.y, a), a = fmaf(w3.x, xb.z, a), a = fmaf(w3.y, xb.w, a);
                acc[r][m] = a;
            }
        }
    }
#pragma unroll
    for (int r = 0; r < ROWS; r++)
#pragma unroll
        for (int m = 0; m < MM; m++) {
            float v = acc[r][m];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            acc[r][m] = v;
        }
    if (lane == 0) {
#pragma unroll
        for (int r = 0; r < ROWS; r++) {
            const int64_t n = n0 + r;
            if (n >= N) break;
#pragma unroll
            for (int m = 0; m < MM; m++) {
                if (m >= M) break;
                float v = acc[r][m] + (bias ? bias[n] : 0.f);
                if (out_f16) ((__half *)out)[(int64_t)m * N + n] = __float2half_rn(v);
                else ((float *)out)[(int64_t)m * N + n] = v;
            }
        }
    }
}

// =====================================================================================================
// Shape-agnostic kernel: any M, N, K (K % 8 != 0, N % 4 != 0, small groups), GPTQ or dense fp16 weight.
// One thread per output, k ascending, double accumulator, bias added in double, one rounding on the
// store: the arithmetic of gemmNTRef (src/reference/qwen-ref.ts:126-145). Correctness path for ragged
// shapes such as the reference's own (N=53, K=42) and (M=37, N=53, K=41) tests, not a fast path.
// =====================================================================================================
__global__ void __launch_bounds__(128) linear_generic_kernel(const uint32_t *__restrict__ qw,
                                                             const uint32_t *__restrict__ qz,
                                                             const __half *__restrict__ sc,
                                                             const __half *__restrict__ dense,
                                                             const void *__restrict__ x, void *__restrict__ out,
                                                             const float *__restrict__ bias, int64_t M, int64_t N,
                                                             int64_t K, int64_t pack_rows, int64_t group,
                                                             int64_t zcols, int x_f16, int out_f16, int round_x_f16)
{
    pdl_sync();
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= M * N) return;
    const int64_t m = idx / N, n = idx - m * N;
    auto xat = [&](int64_t k) -> float {
        float v = x_f16 ? __half2float(((const __half *)x)[m * K + k]) : ((const float *)x)[m * K + k];
        return round_x_f16 ? __half2float(__float2half_rn(v)) : v;
    };
    double acc = 0.0;
    if (dense) {
        for (int64_t k = 0; k < K; k++) acc += (double)xat(k) * (double)__half2float(dense[n * K + k]);
    } else {
        for (int64_t r = 0; r < pack_rows; r++) {
            const uint32_t word = qw[r * N + n];
            const int64_t g = (r * 8) / group;
            const float scale = __half2float(sc[g * N + n]);
            int zero = 8;
            if (qz) zero = (int)((qz[g * zcols + (n >> 3)] >> (4 * (n & 7))) & 15u) + 1;
            for (int j = 0; j < 8; j++) {
                const int64_t k = r * 8 + j;
                if (k >= K) break;
                const float w = (float)((int)((word >> (4 * j)) & 15u) - zero) * scale;
                acc += (double)xat(k) * (double)w;
            }
        }
    }
    if (bias) acc += (double)bias[n];
    if (out_f16) ((__half *)out)[idx] = __float2half_rn((float)acc);
    else ((float *)out)[idx] = (float)acc;
}

// =====================================================================================================
// Planner and dispatch
// =====================================================================================================

int launch_gemm_tc(wb_context *ctx, const Weight &w, const void *A, void *C, const float *bias, int64_t M,
                   int act_dtype, int out_dtype, int exact, const wb_plan &plan);
// gemv_stream.cu
bool gemv_stream_supports(const Weight &w, int64_t M, int chunks, int S, bool has_lo);
int gemv_stream_grid_x(int sm_count, int64_t N, int S);
int launch_gemv_stream(wb_context *ctx, const Weight &w, const GemvParams &gp, bool has_lo);

// WEBLLM_B200_NO_STREAM=1 keeps every decode-size call on the general GEMV kernel (for comparisons).
static bool stream_enabled()
{
    static const bool on = [] { const char *e = getenv("WEBLLM_B200_NO_STREAM"); return !(e && e[0] == '1'); }();
    return on;
}
int plan_gemm_tc(wb_context *ctx, const Weight &w, int64_t M, int act_dtype, int exact, int pair_mode, wb_plan *plan);
bool gemm_tc_supports(const Weight &w, int64_t M);

static bool gemv_mma_shape_ok(const Weight &w)
{
    return w.kind == WeightKind::Gptq && w.K % 8 == 0 && w.N % 4 == 0 && w.group % 128 == 0;
}

static bool gemv_mma_supports(const Weight &w, int64_t M) { return M <= 32 && gemv_mma_shape_ok(w); }

static bool dense_gemv_supports(const Weight &w, int64_t M)
{
    return w.kind == WeightKind::DenseF16 && M <= 8 && w.K % 8 == 0 && (uint64_t)M * w.K * 4 <= 160 * 1024;
}

constexpr int kGemvSmemLimit = 200 * 1024;

// Dynamic shared memory of one GEMV CTA: staged activations (16 bytes per row per packed row, twice for f32
// activations; plus the per-chunk sums otherwise), then the cp.async ring (80 bytes per thread per stage).
// The cross-warp reduction reuses the front of the buffer. Returns the total; 0 stages = size without a ring.
static size_t gemv_smem_bytes(int64_t M, int cps, bool two_halves, int wn, int wk, int stages, int *ring_off,
                              int *red_off = nullptr, int cluster_slices = 0, int *cl_off = nullptr)
{
    const int MB = M <= 8 ? 1 : (M <= 16 ? 2 : 4);
    size_t xs = (size_t)(M + 1) * (cps * 16 + 4) * 16 * (two_halves ? 2 : 1) + (size_t)M * cps * 4;
    xs = (xs + 15) / 16 * 16;
    const size_t ring = (size_t)stages * wn * wk * 32 * 80;
    const size_t red = (size_t)wn * wk * MB * 8 * 32 * 4;
    if (ring_off) *ring_off = (int)xs;
    if (red_off) *red_off = (int)(xs + ring);
    if (cl_off) *cl_off = (int)(xs + ring + red);
    return xs + ring + red + (size_t)cluster_slices * M * wn * 32 * 4;
}

// Grid width: as many column tiles as are resident at once, evened out so that every CTA gets the same number
// of tiles (a partial second wave would otherwise double the time of a kernel that lasts one wave).
static int gemv_grid_x(int sm_count, int ctas_n, int S, int block, size_t smem)
{
    int per_sm = (int)((227 * 1024) / (smem + 1024));  // 228 KB per SM, 1 KB of it reserved per resident CTA
    const int by_threads = 2048 / block, by_regs = block <= 256 ? 3 : 1;
    if (per_sm > by_threads) per_sm = by_threads;
    if (per_sm > by_regs) per_sm = by_regs;
    if (per_sm < 1) per_sm = 1;
    int capacity = sm_count * per_sm / (S > 0 ? S : 1);
    if (capacity < 1) capacity = 1;
    const int waves = (ctas_n + capacity - 1) / capacity;
    return (ctas_n + waves - 1) / waves;
}

// Ring depth. `stages - 1` chunks are requested BEFORE the activations are staged (and before the wait on the
// previous kernel), so the depth must exceed 1 even when a warp has a single chunk: otherwise the first weight
// request is issued after the staging and its whole HBM latency lands on the critical path. A warp with one
// or two chunks gets all of them in flight up front; longer loops keep two slots (shared memory is what limits
// the resident CTAs of the large shapes).
static int gemv_pick_stages(int64_t M, int cps, bool two_halves, int wn, int wk)
{
    const int per_warp = (cps + wk - 1) / wk;
    int stages = per_warp <= 2 ? per_warp + 1 : 2;
    if (stages < 2) stages = 2;
    while (stages > 1 && gemv_smem_bytes(M, cps, two_halves, wn, wk, stages, nullptr) > (size_t)kGemvSmemLimit) stages--;
    return stages;
}

// Split-K slices of one column tile run as a thread-block cluster (and merge through its shared memory) when the
// cluster is portable (<= 8 CTAs) and the merge buffer is small; otherwise through the workspace and arrival counters.
static bool gemv_cluster_merge(int64_t M, int S) { return S > 1 && S <= 8 && M <= 8; }

// `stream`: 0 = the general kernel only, 1 = the streaming kernel where the shape suits it, 2 = the streaming kernel
// or nothing (plan->kernel stays 0 when it does not take the shape or the forced split).
static void plan_gemv_mma(wb_context *ctx, const Weight &w, int64_t M, int two_halves, wb_plan *plan, int stream)
{
    const int chunks = (int)((w.pack_rows + 15) / 16);
    const int col_tiles = (int)((w.N + 31) / 32);
    // Warps side by side along N (wn x 32 columns per CTA). Up to 8 rows ride in one MMA, so a wider CTA only pays where
    // the matrix has both many column tiles and a long K (7B-class: 3584 -> 3584 at M = 6 took 7.7 us with wn = 4, 10.6 with
    // wn = 1); on the 0.5B shapes narrow CTAs are 10 - 30 % faster at M = 5 .. 8 (down 4864 -> 896, M = 8: 8.1 -> 5.7 us).
    const bool wide_and_long = col_tiles >= 100 && chunks >= 24;
    int wn = M <= 2 ? 1 : M <= 4 ? 2 : M > 8 || wide_and_long ? 4 : M <= 6 ? 1 : 2;
    while (wn > 1 && col_tiles < wn) wn >>= 1;
    int wk = M <= 8 ? 8 / wn : 4;  // 256 threads up to 8 rows (3 CTAs per SM), 512 beyond
    if (wk > chunks) wk = chunks;
    const int ctas_n = (col_tiles + wn - 1) / wn;
    const int target = 2 * ctx->sm_count;
    int S = 1;
    const int per_warp = (chunks + wk - 1) / wk;
    if (M <= 8 && ctas_n < target && per_warp > 1) {
        // decode sizes: the slices of a tile merge through cluster shared memory (cheap), so K is split until a warp
        // holds a single chunk, as far as that fills the GPU and a portable cluster (8 CTAs) allows
        const int by_fill = (target + ctas_n - 1) / ctas_n;
        S = per_warp < by_fill ? per_warp : by_fill;
        if (S > 8) S = 8;
    } else if (ctas_n < target && per_warp > 2) {
        const int by_work = (per_warp + 1) / 2;
        const int by_fill = (target + ctas_n - 1) / ctas_n;
        S = by_work < by_fill ? by_work : by_fill;
    }
    // Bandwidth-bound shapes (M <= 4, whole chunks and tiles) go to the streaming kernel, whose CTAs are persistent
    // over 32-column tiles, two per SM: the split is the one that makes the longest CTA shortest (tiles per CTA x
    // chunks per slice) while a slice keeps at least 20 chunks.
    int stream_s = 0;
    if (stream != 0 && ctx->force_split > 0) {
        const int fs = ctx->force_split < chunks ? ctx->force_split : chunks;
        if (gemv_stream_supports(w, M, chunks, fs, two_halves != 0)) stream_s = fs;
    } else if (stream != 0) {
        const int tiles = (int)(w.N / 32);
        long best_cost = 0;
        for (int s = 1; s <= 8; s++) {
            if (!gemv_stream_supports(w, M, chunks, s, two_halves != 0)) continue;
            const int c = (chunks + s - 1) / s;
            int cap = 2 * ctx->sm_count / s;
            if (cap < 1) cap = 1;
            const int waves = (tiles + cap - 1) / cap;
            const long cost = (long)waves * c;
            const int ctas = (tiles + waves - 1) / waves * s;
            // too few CTAs to stream: the general kernel with clusters does better (unless this kernel was asked for)
            if (stream == 1 && ctas * 2 < ctx->sm_count) continue;
            if (stream_s == 0 || cost < best_cost) stream_s = s, best_cost = cost;
        }
    }
    if (stream_s > 0) {
        plan->kernel = WB_KERNEL_GEMV_STREAM;
        plan->split_k = stream_s;
        plan->grid_x = gemv_stream_grid_x(ctx->sm_count, w.N, stream_s);
        plan->grid_y = stream_s;
        plan->grid_z = 1;
        plan->block = 256;
        plan->tile_m = 0, plan->tile_n = 32;
        plan->launches = 1;
        plan->scratch_bytes = stream_s > 1 ? (uint64_t)stream_s * M * w.N * 4 : 0;
        return;
    }
    if (stream == 2) return;
    // shared memory: staged activations (16 bytes per row per packed row, twice in exact mode)
    auto smem_for = [&](int s) { return (uint64_t)gemv_smem_bytes(M, (chunks + s - 1) / s, two_halves, wn, wk, 1, nullptr); };
    while (smem_for(S) > (uint64_t)kGemvSmemLimit && S < chunks) S++;
    if (ctx->force_split > 0) S = ctx->force_split;
    if (S > chunks) S = chunks;
    if (S < 1) S = 1;
    int cps = (chunks + S - 1) / S;
    S = (chunks + cps - 1) / cps;  // drop empty slices
    plan->kernel = WB_KERNEL_GEMV_MMA;
    plan->split_k = S;
    plan->grid_x = ctas_n;
    plan->grid_y = S;
    plan->grid_z = 1;
    plan->block = wn * wk * 32;
    plan->tile_m = wn;  // reused to carry the warp layout to the launcher
    plan->tile_n = wk;
    plan->launches = 1;
    plan->scratch_bytes = S > 1 ? (uint64_t)S * M * w.N * 4 : 0;
}

// allow_stream = false: a decode-size call that fuses a prologue stays on the general GEMV kernel.
static int plan_linear_ex(wb_context *ctx, const Weight &w, int64_t M, int act_dtype, int exact, bool allow_stream, wb_plan *plan)
{
    memset(plan, 0, sizeof *plan);
    int kind = ctx->force_kernel;
    if (kind == 0) {
        // M <= 8: the GEMV (its one-row-block instance, 2 - 8 us). 9 <= M <= 16: its two-row-block instance costs 6 - 16 us
        // and grows with M and K, the tensor-core kernel a flat 5 - 8 us (+ 2.3 us for the cast of f32 activations); measured
        // on the 0.5B and the 7B-class shapes the GEMV still wins there only on short-K, wide-N projections (896 -> 4864,
        // 896 -> 9728): up to M = 12 with fp16 activations, up to 16 with f32 ones.
        const bool tc_ok = gemm_tc_supports(w, M) && !(exact && act_dtype == WB_F32);
        const bool short_wide = w.K <= 2048 && w.N >= 4096;
        const bool gemv_first = M <= 8 || (M <= 16 && (!tc_ok || (short_wide && M <= (act_dtype == WB_F32 ? 16 : 12))));
        if (gemv_mma_supports(w, M) && (gemv_first || !gemm_tc_supports(w, M))) kind = WB_KERNEL_GEMV_MMA;
        else if (dense_gemv_supports(w, M)) kind = WB_KERNEL_DENSE_GEMV;
        else if (gemm_tc_supports(w, M) && !(exact && act_dtype == WB_F32)) kind = WB_KERNEL_GEMM_TC;
        else kind = WB_KERNEL_GENERIC;  // incl. exact f32 activations at large M: k-ascending double sums
    }
    switch (kind) {
    case WB_KERNEL_GEMV_MMA:
    case WB_KERNEL_GEMV_STREAM: {
        if (!gemv_mma_supports(w, M))
            return fail(WB_ERR_UNSUPPORTED, "GEMV_MMA needs a GPTQ weight, M <= 32, K %% 8 == 0, N %% 4 == 0, group %% 128 == 0");
        // the planner's own choice may be either GEMV kernel; a forced kind means that kernel and no other
        const int stream = kind == WB_KERNEL_GEMV_STREAM ? 2 : (ctx->force_kernel == 0 && allow_stream && stream_enabled()) ? 1 : 0;
        plan_gemv_mma(ctx, w, M, act_dtype == WB_F32, plan, stream);
        if (plan->kernel == 0)
            return fail(WB_ERR_UNSUPPORTED, "GEMV_STREAM needs M <= 4, K %% 128 == 0, N %% 32 == 0, group %% 128 == 0 and K slices "
                                            "of >= 20 chunks of 128 (the last one >= 8)");
        if (plan->kernel == WB_KERNEL_GEMV_MMA && (uint64_t)plan->grid_x > (uint64_t)kMaxCounters)
            return fail(WB_ERR_UNSUPPORTED, "N too large for the split-K counter table");
        if (plan->scratch_bytes > kWorkspaceBytes) return fail(WB_ERR_OOM, "split-K partials exceed the workspace");
        return WB_OK;
    }
    case WB_KERNEL_DENSE_GEMV:
        if (!dense_gemv_supports(w, M)) return fail(WB_ERR_UNSUPPORTED, "DENSE_GEMV needs an fp16 weight, M <= 8, K %% 8 == 0");
        plan->kernel = kind;
        plan->split_k = 1;
        plan->block = 256;
        plan->grid_x = (int)((w.N + 31) / 32);  // 8 warps x 4 rows per CTA
        plan->grid_y = plan->grid_z = 1;
        plan->launches = 1;
        return WB_OK;
    case WB_KERNEL_GEMM_TC:
    case WB_KERNEL_GEMM_TC_PAIR: {
        if (!gemm_tc_supports(w, M)) return fail(WB_ERR_UNSUPPORTED, "GEMM_TC does not support this shape");
        // the planner's own choice may be either tensor-core kernel; a forced kind means that kernel and no other
        const int pair_mode = kind == WB_KERNEL_GEMM_TC_PAIR ? 2 : ctx->force_kernel == 0 ? 1 : 0;
        const int rc = plan_gemm_tc(ctx, w, M, act_dtype, exact, pair_mode, plan);
        if (rc == WB_OK && plan->kernel == 0)
            return fail(WB_ERR_UNSUPPORTED, "GEMM_TC_PAIR needs a GPTQ weight, M >= 128 and N >= 256");
        return rc;
    }
    case WB_KERNEL_GENERIC:
        plan->kernel = kind;
        plan->split_k = 1;
        plan->block = 128;
        plan->grid_x = (int)((M * w.N + 127) / 128);
        plan->grid_y = plan->grid_z = 1;
        plan->launches = 1;
        return WB_OK;
    }
    return fail(WB_ERR_BAD_ARG, "unknown kernel kind %d", kind);
}

int plan_linear(wb_context *ctx, const Weight &w, int64_t M, int act_dtype, int exact, wb_plan *plan)
{
    return plan_linear_ex(ctx, w, M, act_dtype, exact, true, plan);
}

// Most of a later weight that one call asks the L2 to fetch (a fraction of the 126 MB L2).
constexpr uint64_t kPrefetchLimit = 32ull << 20;

template <int MB, bool EXACT, bool DIRECT>
static cudaError_t launch_gemv_inst(const GemvParams &p, dim3 grid, int block, size_t smem, cudaStream_t st, bool pdl)
{
    cudaFuncSetAttribute(gptq_gemv_mma_kernel<MB, EXACT, DIRECT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemvSmemLimit);
    return launch_cluster_ex(gptq_gemv_mma_kernel<MB, EXACT, DIRECT>, grid, dim3(block), smem, st, p.cluster ? (unsigned)p.S : 1u, pdl, p);
}

template <int MB>
static cudaError_t launch_gemv_mb(const GemvParams &p, dim3 grid, int block, size_t smem, bool exact, cudaStream_t st, bool pdl = true)
{
    if constexpr (MB == 1) {
        if (p.direct)
            return exact ? launch_gemv_inst<1, true, true>(p, grid, block, smem, st, pdl) : launch_gemv_inst<1, false, true>(p, grid, block, smem, st, pdl);
    }
    return exact ? launch_gemv_inst<MB, true, false>(p, grid, block, smem, st, pdl) : launch_gemv_inst<MB, false, false>(p, grid, block, smem, st, pdl);
}

bool linear_fusion_supported(wb_context *ctx, const Weight &w, int64_t M)
{
    if (M < 1 || M > 8 || ctx->force_kernel != 0) return false;
    return gemv_mma_supports(w, M);  // what plan_linear picks first for M <= 8
}

int launch_linear(wb_context *ctx, const Weight &w, const void *A, void *C, const float *bias, int64_t M,
                  int act_dtype, int out_dtype, int exact, const LinearFusion *fusion)
{
    wb_plan plan;
    // exact mode only changes anything for f32 activations
    const int ex = (exact && act_dtype == WB_F32) ? 1 : 0;
    const bool fused = fusion && fusion->kind != 0;
    WB_CHECK(plan_linear_ex(ctx, w, M, act_dtype, ex, !fused, &plan));
    if (fused && (plan.kernel != WB_KERNEL_GEMV_MMA || M > 8 || act_dtype != WB_F32))
        return fail(WB_ERR_UNSUPPORTED, "a fused prologue needs the int4 GEMV kernel, M <= 8 and f32 activations");
    // The streaming kernel always keeps f32 activations at ~22 bits (hi + lo halves): the reference's
    // GEMV reads A as f32 (gemm_gemv_f16.wgsl:45-58) and the extra MMAs are free in an HBM-bound kernel.
    const int ex_gemv = act_dtype == WB_F32 ? 1 : 0;
    const char *base = ctx->arena[WB_ARENA_WEIGHTS].base;
    switch (plan.kernel) {
    case WB_KERNEL_GEMV_MMA:
    case WB_KERNEL_GEMV_STREAM: {
        GemvParams p;
        p.qw = (const uint32_t *)(base + w.off_main);
        p.qz = w.has_zeros ? (const uint32_t *)(base + w.off_zeros) : nullptr;
        p.sc = (const __half *)(base + w.off_scales);
        p.x = A, p.out = C, p.bias = bias;
        p.partial = (float *)ctx->workspace;
        p.counters = ctx->counters;
        p.M = (int)M, p.N = (int)w.N, p.K = (int)w.K;
        p.pack_rows = (int)w.pack_rows, p.zcols = (int)w.zcols;
        p.chunks = (int)((w.pack_rows + 15) / 16);
        p.S = plan.split_k;
        p.chunks_per_split = (p.chunks + p.S - 1) / p.S;
        p.group_chunks = (int)(w.group / 128);
        p.wn = plan.tile_m, p.wk = plan.tile_n;
        p.x_f16 = act_dtype == WB_F16, p.out_f16 = out_dtype == WB_F16;
        p.xs_stride = p.chunks_per_split * 16 + 4;
        if (plan.kernel == WB_KERNEL_GEMV_STREAM) {
            // bandwidth-bound shape: whole chunks, M <= 4, weights straight into registers
            ctx->prefetch_weight = -1;
            return launch_gemv_stream(ctx, w, p, ex_gemv != 0);
        }
        p.prologue = kPrologueNone, p.delta = nullptr, p.x_out = nullptr, p.norm_w = nullptr, p.eps = 0.f, p.up = nullptr;
        p.ld_x = (int)w.K;
        if (fusion && fusion->kind != 0) {
            p.prologue = fusion->kind, p.delta = fusion->delta, p.x_out = fusion->x_out, p.norm_w = fusion->norm_w;
            p.eps = fusion->eps, p.up = fusion->up;
            if (fusion->kind == kPrologueSiluMul) p.ld_x = fusion->ld;
        }
        p.pf_ptr = nullptr, p.pf_bytes = 0;
        static const bool l2pf = [] { const char *e = getenv("WEBLLM_B200_NO_L2PF"); return !(e && e[0] == '1'); }();
        if (l2pf && ctx->prefetch_weight >= 0 && ctx->prefetch_weight < (int)ctx->weights.size()) {
            const Weight &nx = ctx->weights[ctx->prefetch_weight];
            p.pf_ptr = base + nx.off_main;  // qweight, scales and zeros of one registration are contiguous
            p.pf_bytes = (unsigned)std::min<uint64_t>(nx.bytes, kPrefetchLimit);
        }
        ctx->prefetch_weight = -1;
        const int MB = M <= 8 ? 1 : (M <= 16 ? 2 : 4);
        p.stages = gemv_pick_stages(M, p.chunks_per_split, ex_gemv, p.wn, p.wk);
        p.cluster = gemv_cluster_merge(M, p.S) ? 1 : 0;
        // register path: one chunk per warp and one tile per CTA, at most one CTA per SM (see the kernel's comment)
        p.direct = (M <= 8 && (p.cluster || p.S == 1) && p.chunks_per_split <= p.wk && plan.grid_x * plan.grid_y <= ctx->sm_count) ? 1 : 0;
        // a ring one slot shallower where that is what lets the launch fit one wave of resident CTAs (7B-class 3584 -> 3584 at
        // M = 8 with f32 activations: 117 KB per CTA = one per SM and two waves, 13.6 us; 97 KB = two per SM)
        auto waves_with = [&](int stages) {
            const size_t sm = gemv_smem_bytes(M, p.chunks_per_split, ex_gemv, p.wn, p.wk, stages, nullptr, nullptr, p.cluster ? p.S : 0, nullptr);
            const int gx = gemv_grid_x(ctx->sm_count, plan.grid_x, plan.grid_y, plan.block, sm);
            return (plan.grid_x + gx - 1) / gx;
        };
        while (p.stages > 2 && waves_with(p.stages - 1) < waves_with(p.stages)) p.stages--;
        const size_t smem = gemv_smem_bytes(M, p.chunks_per_split, ex_gemv, p.wn, p.wk, p.stages, &p.ring_off, &p.red_off,
                                            p.cluster ? p.S : 0, &p.cl_off);
        if (smem > (size_t)kGemvSmemLimit) return fail(WB_ERR_UNSUPPORTED, "GEMV_MMA: activations do not fit shared memory");
        // plan.grid_x counts column tiles; the launch covers them with one evenly loaded wave of CTAs
        dim3 grid(gemv_grid_x(ctx->sm_count, plan.grid_x, plan.grid_y, plan.block, smem), plan.grid_y);
        // slices of a cluster send their partial tiles to an mbarrier of the first CTA where every CTA has one whole tile
        // WEBLLM_B200_CLUSTER_ASYNC: 0 = closing cluster barrier instead, 2 = the receiver expects bytes that never come
        static const int cl_async_mode = [] { const char *e = getenv("WEBLLM_B200_CLUSTER_ASYNC"); return e ? atoi(e) : 1; }();
        p.cl_async = (cl_async_mode > 0 && p.cluster && (int)grid.x == plan.grid_x && w.N % (p.wn * 32) == 0) ? (cl_async_mode == 2 ? 2 : 1) : 0;
        p.status = ctx->status_word;
        cudaError_t e = MB == 1   ? launch_gemv_mb<1>(p, grid, plan.block, smem, ex_gemv, ctx->stream)
                        : MB == 2 ? launch_gemv_mb<2>(p, grid, plan.block, smem, ex_gemv, ctx->stream)
                                  : launch_gemv_mb<4>(p, grid, plan.block, smem, ex_gemv, ctx->stream);
        ctx->launches++;
        WB_CUDA(e);
        return WB_OK;
    }
    case WB_KERNEL_DENSE_GEMV: {
        const __half *W = (const __half *)(base + w.off_main);
        const size_t smem = (size_t)M * w.K * 4;
        auto go = [&](auto kern) {
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
            return launch_pdl(kern, dim3(plan.grid_x), dim3(256), smem, ctx->stream, W, A, C, bias, (int)M, (int)w.N, (int)w.K,
                              (int)(act_dtype == WB_F16), (int)(out_dtype == WB_F16));
        };
        const cudaError_t e = M == 1 ? go(dense_gemv_f16_kernel<1>) : M == 2 ? go(dense_gemv_f16_kernel<2>)
                              : M <= 4 ? go(dense_gemv_f16_kernel<4>) : go(dense_gemv_f16_kernel<8>);
        ctx->launches++;
        WB_CUDA(e);
        return WB_OK;
    }
    case WB_KERNEL_GEMM_TC:
    case WB_KERNEL_GEMM_TC_PAIR:
        return launch_gemm_tc(ctx, w, A, C, bias, M, act_dtype, out_dtype, ex, plan);
    case WB_KERNEL_GENERIC: {
        const bool gptq = w.kind == WeightKind::Gptq;
        // f32 activations are rounded to fp16 for M > 1 unless exact mode is on, as the reference's
        // tiled GEMM does when it stages A (gemm_nt_f16_from_f32.wgsl:58-62); its GEMV keeps f32.
        const int round_x = (act_dtype == WB_F32 && !ex && M > 1) ? 1 : 0;
        const cudaError_t e = launch_pdl(linear_generic_kernel, dim3(plan.grid_x), dim3(128), 0, ctx->stream,
            gptq ? (const uint32_t *)(base + w.off_main) : nullptr,
            (gptq && w.has_zeros) ? (const uint32_t *)(base + w.off_zeros) : nullptr,
            gptq ? (const __half *)(base + w.off_scales) : nullptr, gptq ? nullptr : (const __half *)(base + w.off_main),
            A, C, bias, M, w.N, w.K, w.pack_rows, gptq ? w.group : 8, w.zcols, (int)(act_dtype == WB_F16),
            (int)(out_dtype == WB_F16), round_x);
        ctx->launches++;
        WB_CUDA(e);
        return WB_OK;
    }
    }
    return fail(WB_ERR_BAD_ARG, "unknown kernel kind %d", plan.kernel);
}

}  // namespace wb

// =====================================================================================================
// wb_gptq_gemv_static: the split-K int4 GEMV for callers that must not allocate device memory.
//
// Some hosts cannot call cudaMalloc where they run this kernel: code inside a region where the allocator
// is off limits (a real-time audio/control loop, a driver callback, a sandboxed plugin that was handed
// its buffers up front), or an embedding application that owns every byte of the GPU and gives a plugin
// only input and output pointers. The regular path needs a context, and creating one allocates the
// workspace where split-K slices park their partial sums. Here that workspace is a fixed array inside the
// library image instead; every GPU that loads the library carries it until the process exits.
// =====================================================================================================
namespace {

constexpr size_t kStaticCounterWords = 4096;                 // one arrival counter per column tile
constexpr size_t kStaticPartialBytes = 4u << 20;             // split-K partial sums
constexpr size_t kStaticScratchBytes = kStaticCounterWords * sizeof(unsigned) + kStaticPartialBytes;

// Counters first (they must be zero when a call starts), partial sums after them.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
// Device address of g_static_scratch per device ordinal, filled by the first call on that device. Threads that race
// on a first call all store the same value (the address is a property of the device), hence relaxed atomics.
std::atomic<void *> g_static_scratch_addr[kMaxDevices];

bool misaligned(const void *p, uintptr_t a) { return ((uintptr_t)p & (a - 1)) != 0; }

}  // namespace

extern "C" int wb_gptq_gemv_static(const void *qweight, const void *qzeros, const void *scales_f16, const void *x,
                                   void *y, const float *bias, int64_t in_features, int64_t out_features,
                                   int64_t group_size, int64_t M, int act_dtype, int out_dtype, int split_k,
                                   void *cuda_stream)
{
    using namespace wb;
    if (!qweight || !scales_f16 || !x || !y) return fail(WB_ERR_BAD_ARG, "wb_gptq_gemv_static: NULL device pointer");
    if ((act_dtype != WB_F32 && act_dtype != WB_F16) || (out_dtype != WB_F32 && out_dtype != WB_F16))
        return fail(WB_ERR_BAD_ARG, "wb_gptq_gemv_static: dtype must be WB_F32 or WB_F16");
    const int64_t K = in_features, N = out_features;
    if (K <= 0 || N <= 0 || M <= 0) return fail(WB_ERR_BAD_ARG, "wb_gptq_gemv_static: sizes must be positive");
    if (M > 32 || K % 8 != 0 || N % 4 != 0 || group_size <= 0 || group_size % 128 != 0)
        return fail(WB_ERR_UNSUPPORTED, "wb_gptq_gemv_static needs M <= 32, K %% 8 == 0, N %% 4 == 0, group %% 128 == 0");
    // The kernel copies qweight in 16-byte pieces, reads x as 16-byte vectors and scales as 8-byte pairs: a pointer into
    // the middle of a larger buffer that breaks these would fault on the device, so it is refused here instead.
    if (misaligned(qweight, 16) || misaligned(x, 16) || misaligned(y, 16))
        return fail(WB_ERR_BAD_ARG, "wb_gptq_gemv_static: qweight, x and y must be 16-byte aligned");
    if (misaligned(scales_f16, 8)) return fail(WB_ERR_BAD_ARG, "wb_gptq_gemv_static: scales_f16 must be 8-byte aligned");
    if (misaligned(qzeros, 4) || misaligned(bias, 4))
        return fail(WB_ERR_BAD_ARG, "wb_gptq_gemv_static: qzeros and bias must be 4-byte aligned");
    int device = 0;
    WB_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) return fail(WB_ERR_UNSUPPORTED, "device ordinal %d is beyond %d", device, kMaxDevices);
    void *scratch = g_static_scratch_addr[device].load(std::memory_order_relaxed);
    if (!scratch) {
        // In host code the array's name is only a handle; its device address has to be asked for, once per
        // device, with that device current. This is the set-up the first call on a device performs.
        WB_CUDA(cudaGetSymbolAddress(&scratch, g_static_scratch));
        g_static_scratch_addr[device].store(scratch, std::memory_order_relaxed);
    }
    unsigned *counters = (unsigned *)scratch;
    float *partial = (float *)((unsigned char *)scratch + kStaticCounterWords * sizeof(unsigned));

    // launch shape: the regular planner's layout for M, the caller's (or a simple automatic) split
    const int pack_rows = (int)(K / 8), chunks = (pack_rows + 15) / 16, col_tiles = (int)((N + 31) / 32);
    // Warps side by side along N (wn x 32 columns per CTA). Up to 8 rows ride in one MMA, so a wider CTA only pays where
    // the matrix has both many column tiles and a long K (7B-class: 3584 -> 3584 at M = 6 took 7.7 us with wn = 4, 10.6 with
    // wn = 1); on the 0.5B shapes narrow CTAs are 10 - 30 % faster at M = 5 .. 8 (down 4864 -> 896, M = 8: 8.1 -> 5.7 us).
    const bool wide_and_long = col_tiles >= 100 && chunks >= 24;
    int wn = M <= 2 ? 1 : M <= 4 ? 2 : M > 8 || wide_and_long ? 4 : M <= 6 ? 1 : 2;
    while (wn > 1 && col_tiles < wn) wn >>= 1;
    int wk = M <= 8 ? 8 / wn : 4;
    if (wk > chunks) wk = chunks;
    const int ctas_n = (col_tiles + wn - 1) / wn;
    int S = split_k;
    if (S <= 0) {
        int sms = 148;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        const int per_warp = (chunks + wk - 1) / wk;
        S = (ctas_n < 2 * sms && per_warp > 2) ? std::min((per_warp + 1) / 2, (2 * sms + ctas_n - 1) / ctas_n) : 1;
    }
    if (S > chunks) S = chunks;
    const int cps = (chunks + S - 1) / S;
    S = (chunks + cps - 1) / cps;
    const bool two_halves = act_dtype == WB_F32;
    const int MB = M <= 8 ? 1 : (M <= 16 ? 2 : 4);
    const int xs_stride = cps * 16 + 4;
    const int stages = gemv_pick_stages(M, cps, two_halves, wn, wk);
    int ring_off = 0;
    int red_off = 0;
    const size_t smem = gemv_smem_bytes(M, cps, two_halves, wn, wk, stages, &ring_off, &red_off);
    if (smem > (size_t)kGemvSmemLimit)
        return fail(WB_ERR_UNSUPPORTED, "wb_gptq_gemv_static: %lld x %lld activations per slice do not fit shared memory; raise split_k",
                    (long long)M, (long long)(cps * 128));
    if ((size_t)ctas_n > kStaticCounterWords)
        return fail(WB_ERR_UNSUPPORTED, "wb_gptq_gemv_static: N = %lld needs %d column-tile counters, the static scratch holds %zu",
                    (long long)N, ctas_n, kStaticCounterWords);
    if (S > 1 && (size_t)S * M * N * sizeof(float) > kStaticPartialBytes)
        return fail(WB_ERR_UNSUPPORTED,
                    "wb_gptq_gemv_static: split_k * M * N * 4 = %zu bytes of partial sums exceed the static scratch of %zu bytes",
                    (size_t)S * M * N * sizeof(float), kStaticPartialBytes);

    cudaStream_t st = (cudaStream_t)cuda_stream;
    // The array keeps whatever the previous call left; the counters must start at zero.
    if (S > 1) WB_CUDA(cudaMemsetAsync(counters, 0, (size_t)ctas_n * sizeof(unsigned), st));
    GemvParams p;
    p.qw = (const uint32_t *)qweight, p.qz = (const uint32_t *)qzeros, p.sc = (const __half *)scales_f16;
    p.x = x, p.out = y, p.bias = bias, p.partial = partial, p.counters = counters;
    p.M = (int)M, p.N = (int)N, p.K = (int)K, p.pack_rows = pack_rows, p.zcols = (int)((N + 7) / 8);
    p.chunks = chunks, p.chunks_per_split = cps, p.group_chunks = (int)(group_size / 128), p.S = S;
    p.wn = wn, p.wk = wk, p.x_f16 = act_dtype == WB_F16, p.out_f16 = out_dtype == WB_F16, p.xs_stride = xs_stride;
    p.stages = stages, p.ring_off = ring_off, p.red_off = red_off, p.cluster = 0, p.cl_off = 0, p.direct = 0, p.cl_async = 0, p.status = nullptr;
    p.pf_ptr = nullptr, p.pf_bytes = 0;
    p.prologue = kPrologueNone, p.delta = nullptr, p.x_out = nullptr, p.norm_w = nullptr, p.eps = 0.f, p.up = nullptr, p.ld_x = (int)K;
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    dim3 grid(gemv_grid_x(sms, ctas_n, S, wn * wk * 32, smem), S);
    const int block = wn * wk * 32;
    // Launched WITHOUT programmatic stream serialization: the tensors are the caller's, and whatever the caller
    // enqueued before this call on the stream (a kernel that still writes qweight or x) must have completed before
    // the first weight is requested.
    cudaError_t e = MB == 1   ? launch_gemv_mb<1>(p, grid, block, smem, two_halves, st, false)
                    : MB == 2 ? launch_gemv_mb<2>(p, grid, block, smem, two_halves, st, false)
                              : launch_gemv_mb<4>(p, grid, block, smem, two_halves, st, false);
    WB_CUDA(e);
    return WB_OK;
}
